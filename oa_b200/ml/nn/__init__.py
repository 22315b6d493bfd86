from .layers import *  # noqa: F401,F403
