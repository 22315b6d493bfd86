"""Vision: tensor-native image operations (`fn_image`) and detection post-processing / metrics (`fn_detection`)."""
from . import fn_detection, fn_image
from .fn_detection import OaDetectionMetricsResult, OaNmsConfig, OaNmsResult, OaSegmentationMetricsResult
from .fn_image import (OaBorderMode, OaImage, OaImageFormat, OaImageFormatChannels, OaImageLayout, OaInterpolationMode,
                       OaNormalizationParams)
