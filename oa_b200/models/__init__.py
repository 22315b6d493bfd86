from .gpt import OaGptConfig, OaGptModel  # noqa: F401
