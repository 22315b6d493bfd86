"""ML-DSA-65 signatures (FIPS 204) and the number-theoretic transform they run on.

Reference surface: Source/Public/Oa/Crypto/Sign.h (OaPublicKey 1952 bytes, OaSecretKey 4032 bytes, OaSignature 3309 bytes,
OaKeypair, OaGenerateKeypair / OaSign / OaVerify; the reference links liboqs for the arithmetic and keeps unfinished NTT
compute shaders under Crypto/Shader).  Here the scheme is written out from the standard: key generation (Algorithms 1 / 6),
signing with the hedged or deterministic variant (2 / 7), verification (3 / 8), and the auxiliary algorithms 14-42
(bit packing, samplers, Power2Round / Decompose / hints, NTT).  Polynomials are int64 tensors of 256 coefficients; every
routine takes leading batch dimensions, so `Ntt` / `NttInverse` transform any number of polynomials at once on whatever
device the tensor lives on.  SHAKE comes from hashlib.

Not constant time: secret-dependent branches (rejection loops) and tensor indexing are as the standard's pseudocode states
them; this is an implementation for verification and tooling, not for hostile timing environments.
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

Q = 8380417
N = 256
D = 13
K_ROWS, L_COLS = 6, 5
ETA = 4
TAU = 49
BETA = TAU * ETA                 # 196
GAMMA1 = 1 << 19
GAMMA2 = (Q - 1) // 32
OMEGA = 55
CTILDE_BYTES = 48                # lambda / 4, lambda = 192
ZETA = 1753
OA_SIGN_PUBKEY_SIZE, OA_SIGN_SECRET_SIZE, OA_SIGN_SIG_SIZE = 1952, 4032, 3309


def _brv8(x: int) -> int:
    return int(f"{x:08b}"[::-1], 2)


_ZETAS = [pow(ZETA, _brv8(k), Q) for k in range(256)]
_INV256 = pow(256, Q - 2, Q)     # 8347681


def _H(data: bytes, n: int) -> bytes:
    return hashlib.shake_256(data).digest(n)


# ------------------------------------------------------------------------------------------------------------------ NTT
def Ntt(w: torch.Tensor) -> torch.Tensor:
    """Algorithm 41 over the last axis (256 coefficients), any leading batch shape; int64 in, int64 in [0, q) out."""
    w = w.clone() % Q
    lead = w.shape[:-1]
    m, ln = 0, 128
    while ln >= 1:
        blocks = N // (2 * ln)
        z = torch.tensor(_ZETAS[m + 1:m + 1 + blocks], dtype=torch.int64, device=w.device).view(blocks, 1)
        v = w.view(*lead, blocks, 2, ln)
        lo, hi = v[..., 0, :], v[..., 1, :]
        t = (z * hi) % Q
        w = torch.stack([(lo + t) % Q, (lo - t) % Q], -2).reshape(*lead, N)
        m += blocks
        ln //= 2
    return w


def NttInverse(w: torch.Tensor) -> torch.Tensor:
    """Algorithm 42."""
    w = w.clone() % Q
    lead = w.shape[:-1]
    m, ln = 256, 1
    while ln < N:
        blocks = N // (2 * ln)
        # the standard walks m downwards while start walks upwards: block b of this level uses -zetas[m - 1 - b]
        z = torch.tensor([Q - _ZETAS[m - 1 - b] for b in range(blocks)], dtype=torch.int64, device=w.device).view(blocks, 1)
        v = w.view(*lead, blocks, 2, ln)
        lo, hi = v[..., 0, :], v[..., 1, :]
        w = torch.stack([(lo + hi) % Q, (z * ((lo - hi) % Q)) % Q], -2).reshape(*lead, N)
        m -= blocks
        ln *= 2
    return (w * _INV256) % Q


def _mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (a * b) % Q


def _matvec(A: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """A [k, l, 256], v [l, 256] (both in the NTT domain) -> [k, 256]."""
    return ((A * v.unsqueeze(0)) % Q).sum(1) % Q


def _center(x: torch.Tensor, alpha: int = Q) -> torch.Tensor:
    """mod+-: representative in (-alpha/2, alpha/2]."""
    r = x % alpha
    return torch.where(r > alpha // 2, r - alpha, r)


def _inf_norm(x: torch.Tensor) -> int:
    return int(_center(x).abs().max())


# ----------------------------------------------------------------------------------------------------------- bit packing
def _pack_bits(vals: torch.Tensor, bits: int) -> bytes:
    """Non-negative integers, `bits` bits each, little-endian bit order across the stream."""
    v = vals.reshape(-1).to(torch.int64)
    b = ((v.unsqueeze(-1) >> torch.arange(bits)) & 1).reshape(-1).to(torch.uint8)
    by = (b.view(-1, 8).to(torch.int64) << torch.arange(8)).sum(-1)
    return bytes(by.tolist())


def _unpack_bits(data: bytes, bits: int, count: int) -> torch.Tensor:
    by = torch.tensor(list(data), dtype=torch.int64)
    b = ((by.unsqueeze(-1) >> torch.arange(8)) & 1).reshape(-1)[:bits * count]
    return (b.view(count, bits) << torch.arange(bits)).sum(-1)


def _simple_bit_pack(w: torch.Tensor, b: int) -> bytes:
    return _pack_bits(w, b.bit_length())


def _bit_pack(w: torch.Tensor, a: int, b: int) -> bytes:
    return _pack_bits(b - w, (a + b).bit_length())


def _bit_unpack(data: bytes, a: int, b: int, count: int = N) -> torch.Tensor:
    return b - _unpack_bits(data, (a + b).bit_length(), count)


# -------------------------------------------------------------------------------------------------------------- samplers
def _rej_ntt_poly(seed: bytes) -> torch.Tensor:
    """Algorithm 30: coefficients below q from three-byte groups of a SHAKE-128 stream."""
    out: List[int] = []
    n = 840
    while True:
        s = hashlib.shake_128(seed).digest(n)
        out = []
        for i in range(0, len(s) - 2, 3):
            z = s[i] | (s[i + 1] << 8) | ((s[i + 2] & 0x7F) << 16)
            if z < Q:
                out.append(z)
                if len(out) == N:
                    return torch.tensor(out, dtype=torch.int64)
        n *= 2


def _rej_bounded_poly(seed: bytes) -> torch.Tensor:
    """Algorithm 31 for eta = 4: half-bytes below 9 give 4 - b."""
    n = 272
    while True:
        s = hashlib.shake_256(seed).digest(n)
        out: List[int] = []
        for z in s:
            for hb in (z & 15, z >> 4):
                if hb < 9:
                    out.append(ETA - hb)
                    if len(out) == N:
                        return torch.tensor(out, dtype=torch.int64)
        n *= 2


def _expand_a(rho: bytes) -> torch.Tensor:
    return torch.stack([torch.stack([_rej_ntt_poly(rho + bytes([s, r])) for s in range(L_COLS)]) for r in range(K_ROWS)])


def _expand_s(rho_p: bytes) -> Tuple[torch.Tensor, torch.Tensor]:
    s1 = torch.stack([_rej_bounded_poly(rho_p + r.to_bytes(2, "little")) for r in range(L_COLS)])
    s2 = torch.stack([_rej_bounded_poly(rho_p + (r + L_COLS).to_bytes(2, "little")) for r in range(K_ROWS)])
    return s1, s2


def _expand_mask(rho_pp: bytes, mu: int) -> torch.Tensor:
    c = 1 + (GAMMA1 - 1).bit_length()       # 20
    return torch.stack([_bit_unpack(_H(rho_pp + (mu + r).to_bytes(2, "little"), 32 * c), GAMMA1 - 1, GAMMA1) for r in range(L_COLS)])


def _sample_in_ball(ctilde: bytes) -> torch.Tensor:
    """Algorithm 29: tau coefficients of +-1, the rest zero."""
    need = 8 + 4 * TAU
    while True:
        s = hashlib.shake_256(ctilde).digest(need)
        signs = int.from_bytes(s[:8], "little")
        c = [0] * N
        pos = 8
        ok = True
        for i in range(N - TAU, N):
            while True:
                if pos >= len(s):
                    ok = False
                    break
                j = s[pos]
                pos += 1
                if j <= i:
                    break
            if not ok:
                break
            c[i] = c[j]
            c[j] = 1 - 2 * ((signs >> (i + TAU - N)) & 1)
        if ok:
            return torch.tensor(c, dtype=torch.int64)
        need *= 2


# ------------------------------------------------------------------------------------------------- rounding and hints
def _power2round(r: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    rp = r % Q
    r0 = _center(rp, 1 << D)
    return (rp - r0) >> D, r0


def _decompose(r: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    rp = r % Q
    r0 = _center(rp, 2 * GAMMA2)
    wrap = (rp - r0) == Q - 1
    r1 = torch.where(wrap, torch.zeros_like(rp), (rp - r0) // (2 * GAMMA2))
    r0 = torch.where(wrap, r0 - 1, r0)
    return r1, r0


def _high_bits(r):
    return _decompose(r)[0]


def _low_bits(r):
    return _decompose(r)[1]


def _make_hint(z: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    return (_high_bits(r) != _high_bits(r + z)).to(torch.int64)


def _use_hint(h: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    m = (Q - 1) // (2 * GAMMA2)             # 16
    r1, r0 = _decompose(r)
    up, down = (r1 + 1) % m, (r1 - 1) % m
    return torch.where(h == 1, torch.where(r0 > 0, up, down), r1)


def _hint_pack(h: torch.Tensor) -> bytes:
    y = [0] * (OMEGA + K_ROWS)
    idx = 0
    for i in range(K_ROWS):
        for j in torch.nonzero(h[i]).reshape(-1).tolist():
            y[idx] = j
            idx += 1
        y[OMEGA + i] = idx
    return bytes(y)


def _hint_unpack(y: bytes) -> Optional[torch.Tensor]:
    h = torch.zeros(K_ROWS, N, dtype=torch.int64)
    idx = 0
    for i in range(K_ROWS):
        end = y[OMEGA + i]
        if end < idx or end > OMEGA:
            return None
        first = idx
        while idx < end:
            if idx > first and y[idx - 1] >= y[idx]:
                return None
            h[i, y[idx]] = 1
            idx += 1
    if any(b != 0 for b in y[idx:OMEGA]):
        return None
    return h


# ------------------------------------------------------------------------------------------------------------ encodings
def _pk_encode(rho: bytes, t1: torch.Tensor) -> bytes:
    return rho + b"".join(_simple_bit_pack(t1[i], (1 << ((Q - 1).bit_length() - D)) - 1) for i in range(K_ROWS))


def _pk_decode(pk: bytes) -> Tuple[bytes, torch.Tensor]:
    t1 = torch.stack([_unpack_bits(pk[32 + 320 * i:32 + 320 * (i + 1)], 10, N) for i in range(K_ROWS)])
    return pk[:32], t1


def _sk_encode(rho, key, tr, s1, s2, t0) -> bytes:
    out = rho + key + tr
    out += b"".join(_bit_pack(s1[i], ETA, ETA) for i in range(L_COLS))
    out += b"".join(_bit_pack(s2[i], ETA, ETA) for i in range(K_ROWS))
    out += b"".join(_bit_pack(t0[i], (1 << (D - 1)) - 1, 1 << (D - 1)) for i in range(K_ROWS))
    return out


def _sk_decode(sk: bytes):
    rho, key, tr = sk[:32], sk[32:64], sk[64:128]
    p = 128
    s1 = torch.stack([_bit_unpack(sk[p + 128 * i:p + 128 * (i + 1)], ETA, ETA) for i in range(L_COLS)])
    p += 128 * L_COLS
    s2 = torch.stack([_bit_unpack(sk[p + 128 * i:p + 128 * (i + 1)], ETA, ETA) for i in range(K_ROWS)])
    p += 128 * K_ROWS
    t0 = torch.stack([_bit_unpack(sk[p + 416 * i:p + 416 * (i + 1)], (1 << (D - 1)) - 1, 1 << (D - 1)) for i in range(K_ROWS)])
    return rho, key, tr, s1, s2, t0


def _w1_encode(w1: torch.Tensor) -> bytes:
    return b"".join(_simple_bit_pack(w1[i], (Q - 1) // (2 * GAMMA2) - 1) for i in range(K_ROWS))


def _sig_encode(ctilde: bytes, z: torch.Tensor, h: torch.Tensor) -> bytes:
    return ctilde + b"".join(_bit_pack(z[i], GAMMA1 - 1, GAMMA1) for i in range(L_COLS)) + _hint_pack(h)


def _sig_decode(sig: bytes):
    ctilde = sig[:CTILDE_BYTES]
    p = CTILDE_BYTES
    z = torch.stack([_bit_unpack(sig[p + 640 * i:p + 640 * (i + 1)], GAMMA1 - 1, GAMMA1) for i in range(L_COLS)])
    return ctilde, z, _hint_unpack(sig[p + 640 * L_COLS:])


# ---------------------------------------------------------------------------------------------------- internal algorithms
def KeyGenInternal(xi: bytes) -> Tuple[bytes, bytes]:
    """Algorithm 6: (public key, secret key) from a 32-byte seed."""
    if len(xi) != 32:
        raise ValueError("the key generation seed is 32 bytes")
    g = _H(xi + bytes([K_ROWS, L_COLS]), 128)
    rho, rho_p, key = g[:32], g[32:96], g[96:128]
    A = _expand_a(rho)
    s1, s2 = _expand_s(rho_p)
    t = (NttInverse(_matvec(A, Ntt(s1))) + s2) % Q
    t1, t0 = _power2round(t)
    pk = _pk_encode(rho, t1)
    return pk, _sk_encode(rho, key, _H(pk, 64), s1, s2, t0)


def SignInternal(sk: bytes, m_prime: bytes, rnd: bytes) -> bytes:
    """Algorithm 7."""
    rho, key, tr, s1, s2, t0 = _sk_decode(sk)
    s1h, s2h, t0h = Ntt(s1), Ntt(s2), Ntt(t0)
    A = _expand_a(rho)
    mu = _H(tr + m_prime, 64)
    rho_pp = _H(key + rnd + mu, 64)
    kappa = 0
    while True:
        y = _expand_mask(rho_pp, kappa)
        w = NttInverse(_matvec(A, Ntt(y)))
        w1 = _high_bits(w)
        ctilde = _H(mu + _w1_encode(w1), CTILDE_BYTES)
        ch = Ntt(_sample_in_ball(ctilde))
        cs1 = NttInverse(_mul(ch, s1h))
        cs2 = NttInverse(_mul(ch, s2h))
        z = y + _center(cs1)
        r0 = _low_bits(w - cs2)
        kappa += L_COLS
        if _inf_norm(z) >= GAMMA1 - BETA or int(r0.abs().max()) >= GAMMA2 - BETA:
            continue
        ct0 = NttInverse(_mul(ch, t0h))
        h = _make_hint(-ct0, w - cs2 + ct0)
        if _inf_norm(ct0) >= GAMMA2 or int(h.sum()) > OMEGA:
            continue
        return _sig_encode(ctilde, _center(z), h)


def VerifyInternal(pk: bytes, m_prime: bytes, sig: bytes) -> bool:
    """Algorithm 8."""
    if len(pk) != OA_SIGN_PUBKEY_SIZE or len(sig) != OA_SIGN_SIG_SIZE:
        return False
    rho, t1 = _pk_decode(pk)
    ctilde, z, h = _sig_decode(sig)
    if h is None:
        return False
    A = _expand_a(rho)
    mu = _H(_H(pk, 64) + m_prime, 64)
    ch = Ntt(_sample_in_ball(ctilde))
    w_approx = NttInverse((_matvec(A, Ntt(z)) - _mul(ch, Ntt(t1 << D))) % Q)
    w1 = _use_hint(h, w_approx)
    return _inf_norm(z) < GAMMA1 - BETA and _H(mu + _w1_encode(w1), CTILDE_BYTES) == ctilde


def _m_prime(message: bytes, ctx: bytes) -> bytes:
    if len(ctx) > 255:
        raise ValueError("the context string is at most 255 bytes")
    return bytes([0, len(ctx)]) + ctx + message


# ------------------------------------------------------------------------------------------------------------- public API
@dataclass(frozen=True)
class OaPublicKey:
    Bytes: bytes = bytes(OA_SIGN_PUBKEY_SIZE)

    def IsZero(self) -> bool:
        return not any(self.Bytes)

    def ToShortHex(self) -> str:
        return self.Bytes[:16].hex()


@dataclass
class OaSecretKey:
    Bytes: bytes = bytes(OA_SIGN_SECRET_SIZE)

    def SecureZero(self) -> None:
        self.Bytes = bytes(OA_SIGN_SECRET_SIZE)

    def IsZero(self) -> bool:
        return not any(self.Bytes)


@dataclass(frozen=True)
class OaSignature:
    Bytes: bytes = bytes(OA_SIGN_SIG_SIZE)

    def IsZero(self) -> bool:
        return not any(self.Bytes)


@dataclass
class OaKeypair:
    Public: OaPublicKey = field(default_factory=OaPublicKey)
    Secret: OaSecretKey = field(default_factory=OaSecretKey)


def OaGenerateKeypair(seed: Optional[bytes] = None) -> OaKeypair:
    """A fresh key pair (Algorithm 1); `seed` (32 bytes) makes it reproducible."""
    pk, sk = KeyGenInternal(os.urandom(32) if seed is None else seed)
    return OaKeypair(OaPublicKey(pk), OaSecretKey(sk))


def OaSign(secret: OaSecretKey, message: bytes, ctx: bytes = b"", deterministic: bool = False) -> OaSignature:
    """Algorithm 2: hedged by default (32 fresh random bytes per signature), `deterministic` uses the all-zero string."""
    if len(secret.Bytes) != OA_SIGN_SECRET_SIZE or secret.IsZero():
        raise ValueError("not an ML-DSA-65 secret key")
    return OaSignature(SignInternal(secret.Bytes, _m_prime(bytes(message), ctx), bytes(32) if deterministic else os.urandom(32)))


def OaVerify(public: OaPublicKey, message: bytes, signature: OaSignature, ctx: bytes = b"") -> bool:
    """Algorithm 3."""
    if len(ctx) > 255:
        return False
    return VerifyInternal(public.Bytes, _m_prime(bytes(message), ctx), signature.Bytes)
