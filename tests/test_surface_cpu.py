"""The `oa` package exposes the reference's public names; the tutorial training contract runs through it on CPU."""
import pytest
import torch

import oa


def test_root_names_and_namespaces():
    for n in ("OaMatrix", "OaScalarType", "OaContext", "OaContextGetDefault", "OaInitComputeEngine", "OaShutdownComputeEngine", "OaAdam",
              "OaAdamW", "OaSGD", "OaMuon", "OaByteEmbedding", "OaCallback", "OaCbProgressBar", "OaCbSummary", "OaEmbedding", "OaGradientTape",
              "OaGru", "OaRnn", "OaItTraining", "OaItTrainingConfig", "OaLayerNorm", "OaLinear", "OaMamba3Module", "OaMetric",
              "OaMetricAccuracy", "OaMetricLoss", "OaModule", "OaNlpSuiteModel", "OaNlpSuiteRecipe", "OaNlpSuiteSampler", "OaOptimizer",
              "OaOptimizerComposite", "OaOptimizerNoOp", "OaParameter", "OaTrainingSession", "OaTransformerBlock", "OaFilesystem", "OaPath",
              "OaPaths", "OaMatrixShape", "OaMatMulPrecision", "OaGpuTimingStats"):
        assert hasattr(oa, n), n
    for n in ("Add", "AddScalar", "Argmax", "Cast", "CausalMask", "CopyToHost", "CopyToHost2D", "Detach", "Div", "DivScalar", "Empty", "Exp",
              "FromBytes", "FromFloats", "FromInt32", "Full", "Gather", "GatherBwd", "Gelu", "GeluBwd", "GetWeightDtype", "LinearDataBwd",
              "LinearWeightBiasBwd", "Log", "LogSoftmax", "MatMulNt", "Max", "Mean", "Mul", "Ones", "Pow", "Rand", "RandGlorotUniform",
              "RandKaimingUniform", "RandN", "RandXavier", "Relu", "ReluBwd", "Reshape", "Scalar", "Scale", "SetRngSeed", "SetWeightDtype",
              "Sigmoid", "Silu", "SiluBwd", "Slice", "Softmax", "SoftmaxBwd", "Sqrt", "Sub", "SubScalar", "Sum", "Tanh", "TanhBwd", "Transpose",
              "Zeros"):
        assert hasattr(oa.OaFnMatrix, n), n
    for n in ("Bce", "BceBwd", "CrossEntropy", "CrossEntropyBwd", "L1", "L1Bwd", "Mse", "MseBwd", "SmoothL1", "SmoothL1Bwd"):
        assert hasattr(oa.OaFnLoss, n), n
    assert oa.OaFnAutograd.IsEnabled() is False
    with pytest.raises(AttributeError, match="does not provide"):
        oa.OaPlot
    assert len(oa.OaFnImage.__all__) >= 50 and oa.OaFnVision is oa.OaFnImage and hasattr(oa.OaFnDetection, "Nms")
    for n in ("OaRlReplayBuffer", "OaRlRolloutBuffer", "OaPpoLossConfig", "OaItRlTraining", "OaGaeConfig", "OaRlSpaceKind", "OaFnRl"):
        assert hasattr(oa, n), n
    import oa.OaFnMatrix as ns          # namespace modules are importable
    assert ns.Zeros([2, 2]).Tensor().sum().item() == 0


def test_tutorial_contract():
    """engine init -> seed -> OaNlpSuiteModel -> OaAdamW -> OaItTraining -> tape -> Next(loss) -> generation."""
    oa.OaFnMatrix.SetRngSeed(oa.OaNlpSuiteRngSeed)
    recipe = oa.OaNlpSuiteRecipe(oa.OaNlpArchitecture.Gru, oa.OaNlpTokenizerKind.Byte)
    model = oa.OaNlpSuiteModel(recipe)
    sampler = oa.OaNlpSuiteSampler(recipe, 8)
    opt = oa.OaAdamW(model.AllParameterPtrs(), recipe.LearningRate())
    training = oa.OaItTraining(opt, oa.OaItTrainingConfig(TotalSteps=5, BatchSize=8, SequenceLength=recipe.ContextLength()))
    with oa.Context():
        while not training.IsDone():
            x, y = sampler.Next()
            opt.ZeroGrad()
            with oa.OaGradientTape() as tape:
                loss = oa.OaFnLoss.CrossEntropy(model.Forward(x), y.Reshape([y.NumElements()]))
                tape.Backward(loss)
            training.Next(loss)
        training.Finish()
    assert training.StepCount() == 5 and training.LastLoss() == training.LastLoss()
    assert oa.OaNlpSuiteGenerate(model, sampler, source_units=4).startswith("to be")
