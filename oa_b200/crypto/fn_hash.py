"""OaFnHash: batched SHAKE-128 / SHAKE-256, the Keccak-f[1600] permutation and the SHAKE-256 Merkle root.

Reference: Source/Public/Oa/Crypto/FnHash.h:21-41 (device functions) and Source/Private/Oa/Crypto/Hash.cpp:7-84
(OaHashCombine = SHAKE-256(left || right), OaMerkleRoot with the last node paired with itself on odd levels).
Inputs and outputs are UInt8 matrices, one message / state / node per row.  CUDA tensors run csrc/kernels/hash.cu (one
thread per Keccak state); CPU tensors use hashlib and a vectorised uint64 permutation, which are also the test oracles.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

from .. import _native as N
from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ops import kernels as K

_RC = np.array([0x0000000000000001, 0x0000000000008082, 0x800000000000808A, 0x8000000080008000, 0x000000000000808B, 0x0000000080000001,
                0x8000000080008081, 0x8000000000008009, 0x000000000000008A, 0x0000000000000088, 0x0000000080008009, 0x000000008000000A,
                0x000000008000808B, 0x800000000000008B, 0x8000000000008089, 0x8000000000008003, 0x8000000000008002, 0x8000000000000080,
                0x000000000000800A, 0x800000008000000A, 0x8000000080008081, 0x8000000000008080, 0x0000000080000001, 0x8000000080008008],
               dtype=np.uint64)
_PI = (10, 7, 11, 17, 18, 3, 5, 16, 8, 21, 24, 4, 15, 23, 19, 13, 12, 2, 20, 14, 22, 9, 6, 1)
_RHO = (1, 3, 6, 10, 15, 21, 28, 36, 45, 55, 2, 14, 27, 41, 56, 8, 25, 43, 62, 18, 39, 61, 20, 44)


def _rotl(v: np.ndarray, n: int) -> np.ndarray:
    return (v << np.uint64(n)) | (v >> np.uint64(64 - n))


def keccak_f1600_host(states: np.ndarray) -> np.ndarray:
    """states uint64 [n, 25] -> permuted copy (vectorised over n)."""
    a = [states[:, k].copy() for k in range(25)]
    for rnd in range(24):
        c = [a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20] for x in range(5)]
        for x in range(5):
            d = c[(x + 4) % 5] ^ _rotl(c[(x + 1) % 5], 1)
            for y in range(0, 25, 5):
                a[y + x] = a[y + x] ^ d
        cur = a[1]
        for dst, rot in zip(_PI, _RHO):
            nxt = a[dst]
            a[dst] = _rotl(cur, rot)
            cur = nxt
        for y in range(0, 25, 5):
            r = a[y:y + 5]
            a[y:y + 5] = [r[i] ^ (~r[(i + 1) % 5] & r[(i + 2) % 5]) for i in range(5)]
        a[0] = a[0] ^ _RC[rnd]
    return np.stack(a, 1)


def _bytes2d(m: OaMatrix) -> torch.Tensor:
    t = m.Tensor()
    if t.dtype != torch.uint8 or t.dim() != 2:
        raise ValueError("OaFnHash functions take UInt8 matrices [rows, bytes]")
    return F._c(t)


def _shake(bits: int, m: OaMatrix, out_len: int) -> OaMatrix:
    t = _bytes2d(m)
    n, msg_len = t.shape
    if out_len <= 0:
        raise ValueError("output length must be positive")
    padded = (out_len + 7) // 8 * 8
    F._ctx_add(f"Shake{bits}")
    out = torch.zeros(n, padded, dtype=torch.uint8, device=t.device)
    if t.is_cuda:
        lib = N.require()
        K._launch(lib.oa_shake(bits, t.data_ptr(), out.data_ptr(), n, msg_len, t.stride(0), out_len, padded, N.stream()), "oa_shake")
        return OaMatrix(out)
    h = hashlib.shake_128 if bits == 128 else hashlib.shake_256
    rows = t.numpy()
    for i in range(n):
        out[i, :out_len] = torch.frombuffer(bytearray(h(rows[i].tobytes()).digest(out_len)), dtype=torch.uint8)
    return OaMatrix(out)


def Shake256(m: OaMatrix, output_length: int = 32) -> OaMatrix:
    """[N, MsgLen] bytes -> [N, ceil(OutLen / 8) * 8] bytes; row i = SHAKE256(message i) (zero padded to the row width)."""
    return _shake(256, m, output_length)


def Shake128(m: OaMatrix, output_length: int = 16) -> OaMatrix:
    return _shake(128, m, output_length)


def KeccakF1600(m: OaMatrix) -> OaMatrix:
    """Batch permutation of [N, 200]-byte states (25 little-endian u64 lanes each); out of place."""
    t = _bytes2d(m)
    if t.shape[1] != 200:
        raise ValueError("KeccakF1600 takes [N, 200] byte states")
    F._ctx_add("KeccakF1600")
    if t.is_cuda:
        out = torch.empty_like(t)
        lib = N.require()
        K._launch(lib.oa_keccak_f1600(t.data_ptr(), out.data_ptr(), t.shape[0], N.stream()), "oa_keccak_f1600")
        return OaMatrix(out)
    lanes = np.frombuffer(t.numpy().tobytes(), dtype="<u8").reshape(-1, 25)
    return OaMatrix(torch.frombuffer(bytearray(keccak_f1600_host(lanes).astype("<u8").tobytes()), dtype=torch.uint8).reshape(-1, 200))


def MerkleRoot(m: OaMatrix) -> OaMatrix:
    """[N, 32] leaf hashes (N a power of two) -> [1, 32] root by SHAKE-256 pair reduction, one launch per level."""
    t = _bytes2d(m)
    n = t.shape[0]
    if t.shape[1] != 32 or n < 1 or n & (n - 1):
        raise ValueError("MerkleRoot takes [N, 32] leaves with N a power of two")
    F._ctx_add("MerkleRoot")
    if not t.is_cuda:
        level = [bytes(r) for r in t.numpy()]
        while len(level) > 1:
            level = [hashlib.shake_256(level[i] + level[i + 1]).digest(32) for i in range(0, len(level), 2)]
        return OaMatrix(torch.frombuffer(bytearray(level[0]), dtype=torch.uint8).reshape(1, 32))
    lib, cur = N.require(), t
    while cur.shape[0] > 1:
        nxt = torch.empty(cur.shape[0] // 2, 32, dtype=torch.uint8, device=t.device)
        K._launch(lib.oa_merkle_level(cur.data_ptr(), nxt.data_ptr(), cur.shape[0], N.stream()), "oa_merkle_level")
        cur = nxt
    return OaMatrix(cur.clone() if cur is t else cur)


# ---- host-side companions (Hash.h)
def OaShake256(data: bytes, out_len: int = 32) -> bytes:
    return hashlib.shake_256(data).digest(out_len)


def OaShake128(data: bytes, out_len: int = 16) -> bytes:
    return hashlib.shake_128(data).digest(out_len)


def OaHashCombine(left: bytes, right: bytes) -> bytes:
    return hashlib.shake_256(left + right).digest(32)


def OaMerkleRoot(leaves) -> bytes:
    """Arbitrary leaf counts: an odd level pairs its last node with itself; no leaves -> 32 zero bytes."""
    level = [bytes(l) for l in leaves]
    if not level:
        return bytes(32)
    while len(level) > 1:
        level = [OaHashCombine(level[i], level[i + 1] if i + 1 < len(level) else level[i]) for i in range(0, len(level), 2)]
    return level[0]
