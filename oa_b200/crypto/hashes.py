"""Digest value type and the incremental hasher (Source/Python/Crypto/Hash.cpp: OaHash = 32-byte SHAKE-256 digest with
FromHex / Zero / ToHex / ToShortHex / IsZero / Bytes; OaHasher = Update / Finalize / Reset).  Batches of messages are
hashed on the GPU by `OaFnHash`; this host-side pair is for single values (file identities, manifest entries)."""
from __future__ import annotations

import hashlib


class OaHash:
    def __init__(self, Data: bytes = b"\0" * 32):
        data = bytes(Data)
        if len(data) != 32:
            raise ValueError("a digest is exactly 32 bytes")
        self._d = data

    @staticmethod
    def FromHex(Hex: str) -> "OaHash":
        if len(Hex) != 64:
            raise ValueError("a digest is exactly 64 hexadecimal characters")
        return OaHash(bytes.fromhex(Hex))

    @staticmethod
    def Zero() -> "OaHash": return OaHash()
    @staticmethod
    def Of(data: bytes) -> "OaHash": return OaHash(hashlib.shake_256(bytes(data)).digest(32))

    def ToHex(self) -> str: return self._d.hex()
    def ToShortHex(self) -> str: return self._d[:4].hex()
    def IsZero(self) -> bool: return self._d == b"\0" * 32
    def Bytes(self) -> bytes: return self._d
    def __eq__(self, other) -> bool: return isinstance(other, OaHash) and other._d == self._d
    def __hash__(self) -> int: return hash(self._d)
    def __repr__(self) -> str: return f"OaHash({self.ToShortHex()}...)"


class OaHasher:
    """Incremental SHAKE-256 with a 32-byte output."""

    def __init__(self):
        self._h = hashlib.shake_256()

    def Update(self, data: bytes) -> "OaHasher":
        self._h.update(bytes(data))
        return self

    def Finalize(self) -> OaHash: return OaHash(self._h.digest(32))
    def Reset(self) -> None: self._h = hashlib.shake_256()
