"""Hashing on the device (the OaFnHash namespace of the reference) and its host-side companions."""
from . import fn_hash as OaFnHash  # noqa: F401
from .fn_hash import OaHashCombine, OaMerkleRoot, OaShake128, OaShake256  # noqa: F401
