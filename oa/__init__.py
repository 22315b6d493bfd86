"""`oa`: the public Python surface of the framework, name for name the one the reference ships
(Source/Python/oa/_surface.py: root `Oa*` values, the namespace modules OaFnMatrix / OaFnLoss / OaFnAutograd /
OaFnMetric, and the `Context` scope), bound here to oa_b200.

    import oa
    oa.OaInitComputeEngine()
    model = oa.OaNlpSuiteModel(oa.OaNlpSuiteRecipe())
    opt = oa.OaAdamW(model.AllParameterPtrs(), 1e-2)
    with oa.OaGradientTape() as tape: ...
    with oa.Context(): ...            # Execute + Sync of the default context on scope exit

Names of the reference surface that this build does not provide (video codecs, plot, ui, renderer) are listed in `oa.UNAVAILABLE`; touching one raises an AttributeError that says so.
"""
from __future__ import annotations

import sys
import types

import oa_b200 as _impl
from oa_b200.core import fn_matrix as _F
from oa_b200.core import types as _T
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as _AG
from oa_b200.ml import callbacks as _CB
from oa_b200.ml import fn_loss as _L
from oa_b200.ml import metric as _M
from oa_b200.ml import module as _MOD
from oa_b200.ml import nlp_suite as _NS
from oa_b200.ml import optim as _O
from oa_b200.ml import training as _TR
from oa_b200.ml import training_session as _TS
from oa_b200.ml.byte import OaByteEmbedding, OaByteEncoder, OaByteHead
from oa_b200.ml.checkpoint import OaCheckpointManager, OaCheckpointManagerConfig
from oa_b200.ml.nn import layers as _NN
from oa_b200.ml.nn.mamba3 import OaMamba3Module
from oa_b200.ml.nn.empyrealm import OaEmpyrealmCore, OaEmpyrealmModule
from oa_b200.ml.nn.conv import (OaAdaptiveAvgPool2d, OaAvgPool2d, OaBatchNorm2d, OaConv1d, OaConv2d, OaConvTranspose1d, OaConvTranspose2d, OaMaxPool2d,
                                 OaUpsample)
from oa_b200.ml.nn.moe import OaMoE, OaMoeExpert
from oa_b200.ml.nn.recurrent import OaGru, OaGruCell, OaRnn, OaRnnCell
from oa_b200.ml.tokenizer import OaBpeTokenizer
from oa_b200.ml.nn.vq import (OaResidualVectorQuantizer, OaResidualVqResult, OaVectorQuantizer, OaVectorQuantizerConfig, OaVqAssignResult,
                              OaVqResult)
from oa_b200.ml.nn.flow import (OaFlowDenoiser, OaFlowDenoiserConfig, OaFlowTimeEmbedding, OaFlowTransformer, OaFlowTransformerConfig)
from oa_b200.ml import rl as _RL
from oa_b200.ml.rl import fn_rl as _FRL
from oa_b200.runtime import engine as _RT
from oa_b200.utils.paths import OaFilesystem, OaPath, OaPaths

__version__ = _impl.__version__

# ---- root values
OaScalarType, OaMatMulPrecision, OaMatrixShape, OaPrecision = _T.OaScalarType, _T.OaMatMulPrecision, _T.OaMatrixShape, _T.OaPrecision
OaStatus, OaStatusCode, OaError = _T.OaStatus, _T.OaStatusCode, _T.OaError
OaEnumToString, OaEnumFromString = _T.OaEnumToString, _T.OaEnumFromString
OaScalarTypeToString, OaScalarTypeFromString = _T.OaScalarTypeToString, _T.OaScalarTypeFromString
OaPrecisionToString, OaPrecisionFromString = _T.OaPrecisionToString, _T.OaPrecisionFromString
OaMatMulPrecisionToString, OaMatMulPrecisionFromString = _T.OaMatMulPrecisionToString, _T.OaMatMulPrecisionFromString
OaContext, OaContextGetDefault = _RT.OaContext, _RT.OaContextGetDefault
OaInitComputeEngine, OaShutdownComputeEngine = _RT.OaInitComputeEngine, _RT.OaShutdownComputeEngine
OaEngine, OaEngineConfig = _RT.OaEngine, _RT.OaEngineConfig
OaGradientTape, OaGradNo = _AG.OaGradientTape, _AG.OaGradNo
OaModule, OaParameter = _MOD.OaModule, _MOD.OaParameter
OaOptimizer, OaOptimizerNoOp, OaOptimizerComposite = _O.OaOptimizer, _O.OaOptimizerNoOp, _O.OaOptimizerComposite
OaAdam, OaAdamW, OaSGD, OaMuon, OaMuonAdamWConfig = _O.OaAdam, _O.OaAdamW, _O.OaSGD, _O.OaMuon, _O.OaMuonAdamWConfig
OaItTraining, OaItTrainingConfig, OaGpuTimingStats = _TR.OaItTraining, _TR.OaItTrainingConfig, _TR.OaGpuTimingStats
OaAccumulatedStep = _TR.OaAccumulatedStep
from oa_b200.core.validation import OA_VALIDATE, OaValidation, OaValidationSeverity  # noqa: E402
from oa_b200.utils.cli import OaCli  # noqa: E402
from oa_b200.crypto.sign import (OA_SIGN_PUBKEY_SIZE, OA_SIGN_SECRET_SIZE, OA_SIGN_SIG_SIZE, OaGenerateKeypair, OaKeypair, OaPublicKey,  # noqa: E402
                                 OaSecretKey, OaSign, OaSignature, OaVerify)
from oa_b200.extensions.rig import (OaHumanIkCharacterization, OaHumanIkSlot, OaJoint, OaRefJoint, OaRefPose, OaRefPoseFor, OaSkelJoint,  # noqa: E402
                                    OaSkeleton, OaSkHumanIk, OaSkHumanMl3d, OaSkMetaHuman, OaTransform)
from oa_b200.extensions.anim import OaFbxWriter, OaPoseClip, OaPosePack, OaRetarget, OaUsd, OaUsdNamedClip, OaUsdSkelClip  # noqa: E402
from oa_b200.runtime.gemm_tuner import OaGemmTuner  # noqa: E402
OaCallback, OaCbTraining = _TR.OaCallback, _TR.OaCbTraining
OaCbProgressBar, OaCbSummary, OaCbValidation, OaCbCheckpoint = _CB.OaCbProgressBar, _CB.OaCbSummary, _CB.OaCbValidation, _CB.OaCbCheckpoint
OaCbEarlyStop, OaCbLrScheduler, OaCbCsvLogger, OaCbPhase = _CB.OaCbEarlyStop, _CB.OaCbLrScheduler, _CB.OaCbCsvLogger, _CB.OaCbPhase
OaMetric, OaMetricLoss, OaMetricAccuracy = _M.OaMetric, _M.OaMetricLoss, _M.OaMetricAccuracy
OaTrainingSession, OaTrainingSnapshot, OaTrainingState = _TS.OaTrainingSession, _TS.OaTrainingSnapshot, _TS.OaTrainingState
OaTrainingCommandDisposition, OaTrainingCommandResult = _TS.OaTrainingCommandDisposition, _TS.OaTrainingCommandResult
OaTrainingMetricSample, OaTrainingValue = _TS.OaTrainingMetricSample, _TS.OaTrainingValue
OaLinear, OaEmbedding, OaLayerNorm, OaRmsNorm, OaTransformerBlock = _NN.OaLinear, _NN.OaEmbedding, _NN.OaLayerNorm, _NN.OaRmsNorm, _NN.OaTransformerBlock
OaMultiHeadAttention, OaFfn, OaSequential, OaDropout, OaRoPE, OaSwiGLU = _NN.OaMultiHeadAttention, _NN.OaFfn, _NN.OaSequential, _NN.OaDropout, _NN.OaRoPE, _NN.OaSwiGLU
OaRelu, OaGelu, OaSilu, OaSoftmax, OaIdentity, OaFlatten = _NN.OaRelu, _NN.OaGelu, _NN.OaSilu, _NN.OaSoftmax, _NN.OaIdentity, _NN.OaFlatten
OaNlpArchitecture, OaNlpTokenizerKind = _NS.OaNlpArchitecture, _NS.OaNlpTokenizerKind
OaNlpSuiteRecipe, OaNlpSuiteModel, OaNlpSuiteSampler, OaNlpSuiteGenerate = _NS.OaNlpSuiteRecipe, _NS.OaNlpSuiteModel, _NS.OaNlpSuiteSampler, _NS.OaNlpSuiteGenerate
OaNlpSuiteBatchSize, OaNlpSuiteContextLength, OaNlpSuiteModelWidth = _NS.OaNlpSuiteBatchSize, _NS.OaNlpSuiteContextLength, _NS.OaNlpSuiteModelWidth
OaNlpSuiteHiddenWidth, OaNlpSuiteTrainingSteps, OaNlpSuiteRngSeed = _NS.OaNlpSuiteHiddenWidth, _NS.OaNlpSuiteTrainingSteps, _NS.OaNlpSuiteRngSeed
OaNlpSuiteGenerationPrompt, OaNlpSuiteGenerationSourceUnits = _NS.OaNlpSuiteGenerationPrompt, _NS.OaNlpSuiteGenerationSourceUnits


# ---- reinforcement learning
for _n in ("OaItRlTraining", "OaItRlTrainingConfig", "OaDqnLossConfig", "OaDqnLossResult", "OaGaeConfig", "OaGaeResult", "OaPpoLossConfig",
           "OaPpoLossResult", "OaRlContinuousPolicyResult", "OaRlEnvironmentSpec", "OaRlFieldSpec", "OaRlPolicyResult", "OaRlReplayBatch",
           "OaRlReplayBuffer", "OaRlReplayConfig", "OaRlRolloutBatch", "OaRlRolloutBuffer", "OaRlRolloutConfig", "OaRlSpaceKind",
           "OaRlTrainingPhase", "OaSacCriticLossResult", "OaSacLossConfig", "OaRlEnvironment", "OaRlEnvironmentTransition",
           "OaRlTransition", "OaRlReplayTransition", "OaRlActorCritic", "OaRlActorCriticOutput", "OaCategoricalActorCritic",
           "OaCategoricalActorCriticConfig", "OaRlCollector", "OaRlCollectorConfig", "OaRlCollectorMetrics", "OaRlEvaluationConfig",
           "OaRlEvaluationMetrics", "OaPpoTrainer", "OaPpoTrainerConfig", "OaPpoTrainerMetrics", "OaDqnTrainer", "OaDqnTrainerConfig",
           "OaDqnTrainerMetrics", "OaSacTrainer", "OaSacTrainerConfig", "OaSacTrainerMetrics", "OaCartPoleConfig", "OaCartPoleEnvironment",
           "OaLunarLander3dConfig", "OaLunarLander3dEnvironment"):
    globals()[_n] = getattr(_RL, _n)
del _n


class OaActivation:
    """Activation selector of fused Linear layers."""
    none, Relu, Gelu, Silu = 0, 1, 2, 3


# ---- namespace modules (Python views of the C++ namespaces)
def _namespace(name: str, doc: str, source, names, renames=None) -> types.ModuleType:
    m = types.ModuleType(f"oa.{name}", doc)
    for n in names:
        setattr(m, n, getattr(source, (renames or {}).get(n, n)))
    m.__all__ = tuple(names)
    sys.modules[f"oa.{name}"] = m
    return m


_FN_MATRIX = [n for n in dir(_F) if n[0].isupper()]
OaFnMatrix = _namespace("OaFnMatrix", "Tensor factories and differentiable operations.", _F, _FN_MATRIX)
OaFnLoss = _namespace("OaFnLoss", "Loss functions and their explicit backward forms.", _L,
                      ["Bce", "BceBwd", "CrossEntropy", "CrossEntropyBwd", "MaskedCrossEntropy", "L1", "L1Bwd", "Mse", "MseBwd", "SmoothL1",
                       "SmoothL1Bwd", "LastName"])
for _n in ("PpoClippedPolicy", "PpoClippedPolicyBwd", "Ppo", "Dqn", "SacCritic", "SacActor"):
    setattr(OaFnLoss, _n, getattr(_FRL, _n))
OaFnLoss.__all__ = OaFnLoss.__all__ + ("PpoClippedPolicy", "PpoClippedPolicyBwd", "Ppo", "Dqn", "SacCritic", "SacActor")
for _n in ("MaskedMse", "SmoothL1Mean", "VelSmoothL1"):
    setattr(OaFnLoss, _n, getattr(_F, _n))
OaFnLoss.__all__ = OaFnLoss.__all__ + ("MaskedMse", "SmoothL1Mean", "VelSmoothL1")
from oa_b200.ml import fn_optim as _FO
OaFnOptim = _namespace("OaFnOptim", "Stateless optimizer steps (AdamW, SGD, Muon, gradient-norm clipping).", _FO,
                       ["OaAdamWParamSet", "MakeAdamWState", "AdamWAdvanceGraphState", "AdamWStep", "AdamWStepGraph", "AdamWStepMany",
                        "AdamWStepManyGraph", "SgdStep", "MuonStep", "ClipGradNorm"])
OaFnRl = _namespace("OaFnRl", "Advantage estimation, policy distributions, transforms and evaluation.", _RL.OaFnRl,
                    ["Gae", "GaeInto", "NormalizeAdvantages", "SampleCategoricalPolicy", "EvaluateCategoricalPolicy", "SampleTanhNormalPolicy",
                     "EvaluateTanhNormalPolicy", "NormalizeObservation", "ScaleAction", "ClipReward", "SampleLogits", "EvaluateCategorical"])
from oa_b200.core.registry import (OaDifferentiation, OaEffects, OaKernelInfo, OaKernelRegistry, OaLowering, OaOperationContract,
                                   OaOperationKind, OaOperationRegistry)
from oa_b200.crypto import fn_hash as _FH
from oa_b200.audio import fn_audio as _FA
from oa_b200.audio.fn_audio import (OaAudio, OaChannelLayout, OaChannelsForLayout, OaLayoutForChannels, OaMelConfig, OaMfccConfig,
                                    OaNormalizeAudioConfig, OaResampleConfig, OaStftConfig)
OaFnAudio = _namespace("OaFnAudio", "Waveform operations and audio features (STFT, mel, MFCC).", _FA,
                       ["Normalize", "Resample", "Gain", "Clip", "PreEmphasis", "ToMono", "Fade", "Mix", "AmplitudeToDb", "WaveformEnvelope",
                        "Stft", "MelSpectrogram", "Mfcc"])
OaFnHash = _namespace("OaFnHash", "Batched SHAKE / Keccak hashing and the SHAKE-256 Merkle root.", _FH,
                      ["Shake256", "Shake128", "KeccakF1600", "MerkleRoot"])
from oa_b200.vision import fn_detection as _FD
from oa_b200.vision import fn_image as _FI
from oa_b200.vision import (OaBorderMode, OaDetectionMetricsResult, OaImage, OaImageFormat, OaImageFormatChannels, OaImageLayout,
                            OaInterpolationMode, OaNmsConfig, OaNmsResult, OaNormalizationParams, OaSegmentationMetricsResult)
OaFnImage = _namespace("OaFnImage", "Image operations on planar fp32 NCHW tensors and the semantic OaImage overloads.", _FI,
                       ["AdaptiveThresholdGaussian", "AdaptiveThresholdMean", "AlphaBlend", "AverageBlur", "BilateralFilter",
                        "BrightnessContrast", "CenterCrop", "ChannelReorder", "Clamp", "ColorTwist", "Composite", "ConvertColor", "Convolve2d",
                        "Crop", "Dilate", "Erase", "Erode", "Flip", "GammaContrast", "GaussianBlur", "GaussianNoise", "Grayscale", "InRange",
                        "Invert", "Laplacian", "MedianBlur", "MorphologyBlackHat", "MorphologyClose", "MorphologyGradient", "MorphologyOpen",
                        "MorphologyTopHat", "Normalize", "Pad", "Posterize", "Remap", "Resize", "ResizeBatch", "ResizeBilinearBwd", "ResizeNearestBwd", "ResizeNormalize", "Rotate",
                        "SaltPepperNoise", "Scharr", "SegmentationOverlay", "SeparableConvolve2d", "Sharpen", "Sobel", "Solarize",
                        "ThresholdBinary", "ThresholdBinaryInv", "ThresholdToZero", "ThresholdToZeroInv", "ThresholdTruncate", "UnsharpMask",
                        "WarpAffine", "WarpPerspective"])
OaFnVision = OaFnImage            # the reference keeps this older name as an alias
OaFnDetection = _namespace("OaFnDetection", "Box IoU, NMS, confusion matrices and detection / segmentation metrics.", _FD,
                           ["BinaryMaskCounts", "BoxIou", "ConfusionMatrix", "Evaluate", "EvaluateSegmentation", "Nms"])
OaFnAutograd = _namespace("OaFnAutograd", "Autograd recording switch.", _AG, ["IsEnabled", "SetEnabled"])
OaFnMetric = _namespace("OaFnMetric", "Host-side metrics of device results.", _M.OaFnMetric, ["Accuracy", "ScalarLoss"])


# ---- host primitives, streams and the native executor pieces
from oa_b200.core.host import (OaAlignedBuffer, OaChannel, OaCoreInfo, OaCpuTopology, OaMemcpyNT, OaMemEqual, OaSimd, OaTask, OaThreadPool,
                               OaThreadPoolConfig)
from oa_b200.runtime.graph import OaAccess, OaComputeGraph
from oa_b200.runtime.device import (DescribeDevice as OaDescribeDevice, OaDeviceBuilder, OaDeviceHardwareInfo, OaDeviceInfo, OaDevicePerformance,
                                    OaDeviceSoftwareInfo, OaDeviceType, OaFeatureModule)
from oa_b200.runtime.session import (OaAnalyzeSemanticLowering, OaExecutionPlan, OaExecutionSession, OaSemanticGraph,
                                     OaSemanticLoweringAnalysis, OaValidateSemanticLowering)
from oa_b200.runtime.stream import (OaCompletionToken, OaComputeClass, OaDispatch, OaDispatchHint, OaExternalMemory, OaExternalMemoryHandle,
                                    OaFence, OaInferencePool, OaInferencePoolConfig, OaPqcPool, OaPqcPoolConfig, OaScheduler, OaSecureBuffer, OaStream, OaStreamPool,
                                    OaTimelineSemaphore, OaWorkItem, OaWorkQueue)


# ---- data layer
from oa_b200.data.dataframe import OaDataFrame, OaDataOhlcv, OaRecordOhlcv, OaSeries, OaTimeSeries
from oa_b200.data.datasets import (OaAsyncReader, OaDsDailyDialog, OaDsHumanMl3d, OaDsMnist, OaDsSharded, OaDsSubset, OaDsTinyShakespeare,
                                   OaFnDataset, OaHumanMl3dCaption, OaHumanMl3dEvaluateMotion, OaHumanMl3dMotionMetrics, OaHumanMl3dMpjpeCm,
                                   OaHumanMl3dRecoverWorldJoints, OaIoUringReader, OaReadFileParallel)
from oa_b200.data.stores import OaContractTicker, OaDataSummary, OaKeyValueStore, OaOhlcvStore, OaSqlStore, OaStoreKind


# ---- extensions: animation language model, precision policy
from oa_b200.extensions.alm import (OaAlmAg, OaAlmDatasetConfig, OaAlmFfnType, OaAlmPriorAg, OaAlmPriorConfig, OaAlmTokenizerAg,
                                    OaAlmTokenizerConfig, OaClipTextAg, OaClipTextConfig, OaClipTextWeightName, OaClipTokenizer)
from oa_b200.ml.precision import (OaLoadStoreStrideBytes, OaLookupPrecision, OaPipelineNameIsF32Variant, OaPrecisionDtype, OaPrecisionTag)


# ---- codecs and transport
from oa_b200.audio.codec import OaAudioDecoder, OaAudioEncoder
from oa_b200.network import OaTcpFramed, OaTcpListener, OaTcpStream
from oa_b200.vision.codec import OaFilter, OaImageBatch, OaImageCodec, OaImageDecoder, OaImageEncoder, OaImageIo, OaPixelFormat
from oa_b200.crypto.hashes import OaHash, OaHasher
OaLinearWeightBiasBwdResult = _F.OaLinearWeightBiasBwdResult


# ---- animation
from oa_b200.animation import (OaCurveColor, OaCurveFloat, OaCurveQuat, OaCurveVec3, OaEasing, OaFrameRate, OaKeyInterpolation, OaKeyframe,
                               OaKeyframeTrack, OaTimeCode, OaTimeDirection, OaTimeTransform, OaTimeline, OaTimelineState)


# ---- logging, performance records
from oa_b200.utils.log import (OA_LOG_DEBUG, OA_LOG_ERROR, OA_LOG_INFO, OA_LOG_TRACE, OA_LOG_WARN, OaGetComponentName, OaLog, OaLogComponent,
                               OaLogLevel, OaLogSummary, OaMetricsWriter)
from oa_b200.utils.perf import OaNvtxRange, OaPerfRecord, OaPerfStat, OaPerfStore


# ---- rank health and host-side fault injection
from oa_b200.parallel.health import OaFault, OaFaultInjector, OaFaultKind, OaRankFailure, OaRankMonitor, OaRankState


class Context:
    """Executes and synchronises the default context on scope exit."""

    def __enter__(self) -> "Context":
        self._ctx = OaContextGetDefault()
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        self._ctx.Execute()
        self._ctx.Sync()


UNAVAILABLE = ("OaPlot", "OaViewer", "OaVideo", "OaRenderer",
               # video codecs and containers, camera / screen capture: the reference drives the vendor's decode engine and the
               # desktop through a graphics API
               "OaCameraCapture", "OaCameraCaptureConfig", "OaContainerInfo", "OaContainerKind", "OaScreenCapture", "OaScreenCaptureConfig",
               "OaScreenCaptureCursor", "OaScreenCaptureTarget", "OaVideoCodec", "OaVideoConfig", "OaVideoDecodeCapabilities",
               "OaVideoEncodeCapabilities", "OaVideoEncodeProfile", "OaVideoFrame", "OaVideoFrameResource", "OaVideoPacket",
               "OaVideoRateControl", "OaVideoRecorder", "OaVideoRecorderConfig", "OaVideoStream", "OaVideoStreamOptions",
               "OaVideoStreamStats", "OaYCbCrModel")


def __getattr__(name: str):
    if name in UNAVAILABLE:
        raise AttributeError(f"oa.{name} belongs to a part of the reference surface (video and capture, plot / ui / renderer, ML-DSA signatures) that this build does not provide")
    raise AttributeError(f"module 'oa' has no attribute '{name}'")


__all__ = sorted(n for n in globals() if n.startswith("Oa")) + ["Context"]
