"""FLAC decoder and a compact encoder (the format of xiph.org's specification, RFC 9639).

The reference's audio decoder reads FLAC through a bundled decoder (Source/Private/Oa/Audio/AudioDecoder.cpp); this one is
written from the format description.  Decoder: STREAMINFO and skipping of the other metadata blocks, frame headers with every
block-size / sample-rate / sample-size code, UTF-8 coded frame or sample numbers, CRC-8 of the header and CRC-16 of the
frame (both checked), the four channel assignments (independent, left/side, right/side, mid/side), subframe types CONSTANT,
VERBATIM, FIXED (orders 0-4) and LPC (orders 1-32), wasted bits, residuals in both Rice partition methods with escape
partitions.  Encoder (for tools and tests): fixed block size, per-channel choice between CONSTANT, VERBATIM, the best FIXED
order and a quantised LPC predictor, one Rice partition with the best parameter, mid/side for stereo when it is smaller,
STREAMINFO with the MD5 of the samples.  Decoding is bit exact; `DecodeFlac` returns integers, `OaAudioDecoder` scales them
to float.
"""
from __future__ import annotations

import hashlib
import struct
from typing import List, Tuple

import numpy as np


def _crc_table(poly: int, bits: int) -> List[int]:
    top, mask = 1 << (bits - 1), (1 << bits) - 1
    t = []
    for i in range(256):
        c = i << (bits - 8)
        for _ in range(8):
            c = ((c << 1) ^ poly) & mask if c & top else (c << 1) & mask
        t.append(c)
    return t


_CRC8, _CRC16 = _crc_table(0x07, 8), _crc_table(0x8005, 16)


def crc8(data: bytes) -> int:
    c = 0
    for b in data:
        c = _CRC8[c ^ b]
    return c


def crc16(data: bytes) -> int:
    c = 0
    for b in data:
        c = ((c << 8) & 0xFFFF) ^ _CRC16[(c >> 8) ^ b]
    return c


class _Reader:
    def __init__(self, data: bytes, pos: int = 0):
        self.d, self.p, self.acc, self.n = data, pos, 0, 0

    def bits(self, k: int) -> int:
        while self.n < k:
            if self.p >= len(self.d):
                raise ValueError("FLAC stream ends inside a frame")
            self.acc = (self.acc << 8) | self.d[self.p]
            self.p += 1
            self.n += 8
        self.n -= k
        v = (self.acc >> self.n) & ((1 << k) - 1)
        self.acc &= (1 << self.n) - 1
        return v

    def signed(self, k: int) -> int:
        v = self.bits(k)
        return v - (1 << k) if v >> (k - 1) else v

    def unary(self) -> int:
        n = 0
        while self.bits(1) == 0:
            n += 1
        return n

    def align(self) -> None:
        self.acc = self.n = 0

    def utf8(self) -> int:
        b = self.bits(8)
        if b < 0x80:
            return b
        n = 0
        while b & (0x80 >> n):
            n += 1
        if n < 2 or n > 7:
            raise ValueError("bad UTF-8 coded number")
        v = b & ((1 << (7 - n)) - 1)
        for _ in range(n - 1):
            c = self.bits(8)
            if c & 0xC0 != 0x80:
                raise ValueError("bad UTF-8 continuation")
            v = (v << 6) | (c & 0x3F)
        return v


_BLOCK = {1: 192, 2: 576, 3: 1152, 4: 2304, 5: 4608, 8: 256, 9: 512, 10: 1024, 11: 2048, 12: 4096, 13: 8192, 14: 16384, 15: 32768}
_RATE = {1: 88200, 2: 176400, 3: 192000, 4: 8000, 5: 16000, 6: 22050, 7: 24000, 8: 32000, 9: 44100, 10: 48000, 11: 96000}
_BPS = {1: 8, 2: 12, 4: 16, 5: 20, 6: 24, 7: 32}
_FIXED = {0: [], 1: [1], 2: [2, -1], 3: [3, -3, 1], 4: [4, -6, 4, -1]}


def _residual(r: _Reader, blocksize: int, order: int) -> List[int]:
    method = r.bits(2)
    if method > 1:
        raise ValueError("reserved residual coding method")
    pbits, esc = (4, 15) if method == 0 else (5, 31)
    porder = r.bits(4)
    parts = 1 << porder
    if blocksize % parts or (blocksize >> porder) < order and porder:
        raise ValueError("residual partitions do not divide the block")
    out: List[int] = []
    for p in range(parts):
        n = (blocksize >> porder) - (order if p == 0 else 0)
        k = r.bits(pbits)
        if k == esc:
            nb = r.bits(5)
            out.extend(r.signed(nb) if nb else 0 for _ in range(n))
        else:
            for _ in range(n):
                u = (r.unary() << k) | (r.bits(k) if k else 0)
                out.append((u >> 1) ^ -(u & 1))
    return out


def _predict(warm: List[int], res: List[int], coefs: List[int], shift: int) -> List[int]:
    out = list(warm)
    order = len(coefs)
    for e in res:
        acc = 0
        for j in range(order):
            acc += coefs[j] * out[-1 - j]
        out.append(e + (acc >> shift))
    return out


def _subframe(r: _Reader, blocksize: int, bps: int) -> List[int]:
    if r.bits(1):
        raise ValueError("subframe padding bit is set")
    kind = r.bits(6)
    wasted = 0
    if r.bits(1):
        wasted = r.unary() + 1
        bps -= wasted
    if kind == 0:
        out = [r.signed(bps)] * blocksize
    elif kind == 1:
        out = [r.signed(bps) for _ in range(blocksize)]
    elif 8 <= kind <= 12:
        order = kind - 8
        warm = [r.signed(bps) for _ in range(order)]
        out = _predict(warm, _residual(r, blocksize, order), _FIXED[order], 0)
    elif kind >= 32:
        order = kind - 31
        warm = [r.signed(bps) for _ in range(order)]
        prec = r.bits(4) + 1
        if prec == 16:
            raise ValueError("reserved predictor precision")
        shift = r.signed(5)
        if shift < 0:
            raise ValueError("negative predictor shift")
        coefs = [r.signed(prec) for _ in range(order)]
        out = _predict(warm, _residual(r, blocksize, order), coefs, shift)
    else:
        raise ValueError("reserved subframe type")
    return [v << wasted for v in out] if wasted else out


def DecodeFlac(data: bytes, verify_md5: bool = True) -> Tuple[np.ndarray, int, int]:
    """-> (int32 samples [channels, n], sample rate, bits per sample).  The MD5 signature of STREAMINFO (when the encoder
    wrote one) is checked against the decoded samples."""
    if data[:4] != b"fLaC":
        raise ValueError("no fLaC marker")
    pos = 4
    info = None
    while True:
        if pos + 4 > len(data):
            raise ValueError("truncated metadata")
        last, kind = data[pos] >> 7, data[pos] & 0x7F
        ln = int.from_bytes(data[pos + 1:pos + 4], "big")
        body = data[pos + 4:pos + 4 + ln]
        pos += 4 + ln
        if kind == 0:
            if len(body) < 34:
                raise ValueError("short STREAMINFO")
            v = int.from_bytes(body[10:18], "big")
            info = {"rate": v >> 44, "channels": ((v >> 41) & 7) + 1, "bps": ((v >> 36) & 31) + 1, "total": v & ((1 << 36) - 1), "md5": body[18:34],
                    "max_block": struct.unpack(">H", body[2:4])[0]}
        if last:
            break
    if info is None:
        raise ValueError("no STREAMINFO block")
    chans: List[List[int]] = [[] for _ in range(info["channels"])]
    while pos < len(data):
        if pos + 2 > len(data) or data[pos] != 0xFF or (data[pos + 1] & 0xFE) != 0xF8:
            raise ValueError("lost frame synchronisation")
        start = pos
        r = _Reader(data, pos)
        r.bits(15)
        r.bits(1)                                  # blocking strategy: the coded number is a frame or a sample number
        bs_code, sr_code = r.bits(4), r.bits(4)
        ch_code, bps_code = r.bits(4), r.bits(3)
        if r.bits(1) or bs_code == 0 or sr_code == 15 or bps_code == 3:
            raise ValueError("reserved frame header value")
        r.utf8()
        blocksize = r.bits(8) + 1 if bs_code == 6 else (r.bits(16) + 1 if bs_code == 7 else _BLOCK[bs_code])
        if sr_code in (12, 13, 14):
            r.bits(8 if sr_code == 12 else 16)
        bps = info["bps"] if bps_code == 0 else _BPS[bps_code]
        if crc8(data[start:r.p]) != r.bits(8):
            raise ValueError("frame header CRC-8 mismatch")
        if ch_code < 8:
            nch = ch_code + 1
            subs = [_subframe(r, blocksize, bps) for _ in range(nch)]
        elif ch_code <= 10:
            nch = 2
            extra = (0, 1) if ch_code == 8 else ((1, 0) if ch_code == 9 else (0, 1))
            a = _subframe(r, blocksize, bps + extra[0])
            b = _subframe(r, blocksize, bps + extra[1])
            if ch_code == 8:                       # left, side
                subs = [a, [x - y for x, y in zip(a, b)]]
            elif ch_code == 9:                     # side, right
                subs = [[x + y for x, y in zip(a, b)], b]
            else:                                  # mid, side
                left = [((m << 1) | (s & 1)) + s >> 1 for m, s in zip(a, b)]
                subs = [left, [l - s for l, s in zip(left, b)]]
        else:
            raise ValueError("reserved channel assignment")
        if nch != info["channels"]:
            raise ValueError("frame channel count differs from STREAMINFO")
        r.align()
        if crc16(data[start:r.p]) != struct.unpack(">H", data[r.p:r.p + 2])[0]:
            raise ValueError("frame CRC-16 mismatch")
        pos = r.p + 2
        for c in range(nch):
            chans[c].extend(subs[c])
    out = np.array(chans, dtype=np.int64)
    if info["total"]:
        out = out[:, :info["total"]]
    if verify_md5 and any(info["md5"]) and hashlib.md5(PcmBytes(out, info["bps"])).digest() != info["md5"]:
        raise ValueError("decoded samples do not match the MD5 signature of the stream")
    return out.astype(np.int32), info["rate"], info["bps"]


def PcmBytes(samples: np.ndarray, bps: int) -> bytes:
    """Interleaved little-endian signed samples, the form the STREAMINFO MD5 is taken over."""
    nbytes = (bps + 7) // 8
    inter = samples.T.astype(np.int64).reshape(-1)
    raw = (inter & ((1 << (8 * nbytes)) - 1)).astype("<u8").view(np.uint8).reshape(-1, 8)[:, :nbytes]
    return raw.tobytes()


# --------------------------------------------------------------------------------------------------------------- encoder
class _Writer:
    def __init__(self):
        self.out = bytearray()
        self.acc = self.n = 0

    def put(self, v: int, k: int) -> None:
        if k == 0:
            return
        self.acc = (self.acc << k) | (v & ((1 << k) - 1))
        self.n += k
        while self.n >= 8:
            self.out.append((self.acc >> (self.n - 8)) & 0xFF)
            self.n -= 8
        self.acc &= (1 << self.n) - 1

    def unary(self, q: int) -> None:
        while q > 32:
            self.put(0, 32)
            q -= 32
        self.put(1, q + 1)

    def align(self) -> None:
        if self.n:
            self.put(0, 8 - self.n)


def _utf8(v: int) -> bytes:
    if v < 0x80:
        return bytes([v])
    n = 2
    while v >= 1 << (5 * n + 1):
        n += 1
    out = [((0xFF << (8 - n)) & 0xFF) | (v >> (6 * (n - 1)))]
    for i in range(n - 2, -1, -1):
        out.append(0x80 | ((v >> (6 * i)) & 0x3F))
    return bytes(out)


def _rice_cost(res: np.ndarray) -> Tuple[int, int]:
    u = np.where(res >= 0, res << 1, ((-res) << 1) - 1).astype(np.int64)
    best = (1 << 62, 0)
    for k in range(0, 15):
        bits = int((u >> k).sum()) + (k + 1) * len(u)
        if bits < best[0]:
            best = (bits, k)
    return best


def _lpc(x: np.ndarray, order: int, precision: int = 12):
    """Quantised forward predictor from the autocorrelation method; None when the block is degenerate."""
    w = x.astype(np.float64) * np.hanning(len(x))
    ac = np.array([np.dot(w[:len(w) - k], w[k:]) for k in range(order + 1)])
    if ac[0] <= 0:
        return None
    a = np.zeros(order)
    err = ac[0]
    for i in range(order):                                   # Levinson-Durbin
        k = (ac[i + 1] - np.dot(a[:i], ac[i:0:-1])) / err
        a_new = a.copy()
        a_new[i] = k
        a_new[:i] = a[:i] - k * a[:i][::-1]
        a = a_new
        err *= 1 - k * k
        if err <= 0:
            return None
    peak = np.max(np.abs(a))
    if peak == 0:
        return None
    shift = int(np.clip(precision - 1 - np.floor(np.log2(peak)) - 1, 0, 15))
    q = np.clip(np.rint(a * (1 << shift)), -(1 << (precision - 1)), (1 << (precision - 1)) - 1).astype(np.int64)
    return q, shift, precision


def _encode_subframe(w: _Writer, x: np.ndarray, bps: int) -> None:
    n = len(x)
    x = x.astype(np.int64)
    if np.all(x == x[0]):
        w.put(0, 8)                                          # padding 0, type 000000, no wasted bits
        w.put(int(x[0]), bps)
        return
    best = ("verbatim", n * bps, None)
    for order in range(0, 5):
        if n <= order:
            break
        res = x.copy()
        for _ in range(order):
            res = res[1:] - res[:-1]
        bits, k = _rice_cost(res)
        total = order * bps + 6 + 4 + bits
        if total < best[1]:
            best = ("fixed", total, (order, res, k))
    for order in (8,):
        if n > 4 * order:
            q = _lpc(x, order)
            if q is not None:
                coefs, shift, prec = q
                pred = np.zeros(n - order, np.int64)
                for j in range(order):
                    pred += coefs[j] * x[order - 1 - j:n - 1 - j]
                res = x[order:] - (pred >> shift)
                if np.max(np.abs(res)) < (1 << 30):
                    bits, k = _rice_cost(res)
                    total = order * bps + 4 + 5 + order * prec + 6 + 4 + bits
                    if total < best[1]:
                        best = ("lpc", total, (order, res, k, coefs, shift, prec))
    kind = best[0]
    if kind == "verbatim":
        w.put(0b00000010, 8)
        for v in x:
            w.put(int(v), bps)
        return
    if kind == "fixed":
        order, res, k = best[2]
        w.put((0b001000 | order) << 1, 8)
    else:
        order, res, k, coefs, shift, prec = best[2]
        w.put((0b100000 | (order - 1)) << 1, 8)
    for v in x[:order]:
        w.put(int(v), bps)
    if kind == "lpc":
        w.put(prec - 1, 4)
        w.put(shift, 5)
        for c in coefs:
            w.put(int(c), prec)
    w.put(0, 2)                                              # Rice method 0
    w.put(0, 4)                                              # one partition
    w.put(k, 4)
    for e in res.tolist():
        u = (e << 1) if e >= 0 else ((-e) << 1) - 1
        w.unary(u >> k)
        w.put(u & ((1 << k) - 1), k)


def EncodeFlac(samples: np.ndarray, rate: int, bps: int = 16, blocksize: int = 4096) -> bytes:
    """int samples [channels, n] (values within `bps` bits) -> FLAC stream."""
    x = np.atleast_2d(np.asarray(samples)).astype(np.int64)
    nch, total = x.shape
    if not (1 <= nch <= 8) or not (4 <= bps <= 32) or total == 0 or not (16 <= blocksize <= 65535):
        raise ValueError("EncodeFlac: 1-8 channels, 4-32 bits, a non-empty signal and a block size of 16..65535")
    lim = 1 << (bps - 1)
    if x.min() < -lim or x.max() >= lim:
        raise ValueError("samples exceed the stated bit depth")
    frames = bytearray()
    sizes = []
    bps_code = {8: 1, 12: 2, 16: 4, 20: 5, 24: 6, 32: 7}.get(bps, 0)
    for fi, start in enumerate(range(0, total, blocksize)):
        blk = x[:, start:start + blocksize]
        n = blk.shape[1]
        plans = [(nch - 1, [(blk[c], bps) for c in range(nch)])]
        if nch == 2 and bps < 32:
            side = blk[0] - blk[1]
            mid = (blk[0] + blk[1]) >> 1
            plans.append((10, [(mid, bps), (side, bps + 1)]))
        best = None
        for ch_code, subs in plans:
            w = _Writer()
            head = bytearray([0xFF, 0xF8])
            bs_code = 6 if n - 1 < 256 else 7
            head.append((bs_code << 4) | 0)                  # sample rate: from STREAMINFO
            head.append((ch_code << 4) | (bps_code << 1))
            head += _utf8(fi)
            head += bytes([n - 1]) if bs_code == 6 else struct.pack(">H", n - 1)
            head.append(crc8(bytes(head)))
            for sx, sb in subs:
                _encode_subframe(w, sx, sb)
            w.align()
            body = bytes(head) + bytes(w.out)
            frame = body + struct.pack(">H", crc16(body))
            if best is None or len(frame) < len(best):
                best = frame
        frames += best
        sizes.append(len(best))
    info = struct.pack(">HH", blocksize, blocksize) + min(sizes).to_bytes(3, "big") + max(sizes).to_bytes(3, "big")
    info += ((rate << 44) | ((nch - 1) << 41) | ((bps - 1) << 36) | total).to_bytes(8, "big")
    info += hashlib.md5(PcmBytes(x, bps)).digest()
    return b"fLaC" + bytes([0x80]) + len(info).to_bytes(3, "big") + info + bytes(frames)
