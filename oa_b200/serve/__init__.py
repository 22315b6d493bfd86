from .decoder import OaGptDecoder, OaKvCache  # noqa: F401
from .tp_decoder import OaOneShotAllReduce, OaTpGptDecoder  # noqa: F401
