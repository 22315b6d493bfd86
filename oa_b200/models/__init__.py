from .gpt import OaGptConfig, OaGptModel  # noqa: F401
from .mamba3_lm import OaMamba3Block, OaMamba3Config, OaMamba3LmModel  # noqa: F401
