from .decoder import OaGptDecoder, OaKvCache  # noqa: F401
