"""Audio: the OaAudio value type and the OaFnAudio DSP namespace (Source/Public/Oa/Audio/{Type,FnAudio}.h)."""
from . import fn_audio as OaFnAudio  # noqa: F401
from .fn_audio import (OaAudio, OaChannelLayout, OaChannelsForLayout, OaLayoutForChannels, OaMelConfig, OaMfccConfig,  # noqa: F401
                       OaNormalizeAudioConfig, OaResampleConfig, OaStftConfig)
