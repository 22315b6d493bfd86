from .engine import *  # noqa: F401,F403
