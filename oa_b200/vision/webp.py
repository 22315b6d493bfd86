"""Lossless WebP (VP8L) decode and encode, written out from the format description (RIFF container, LSB-first bit stream,
canonical prefix codes, LZ77 with the 2-D distance map, colour cache, and the four transforms: predictor, cross-colour,
subtract-green, colour indexing).

The reference reaches WebP through libwebp when its build has it (Source/Private/Oa/Vision/Image/Codec/WebpImageCodec.cpp:
40-140) and answers "this build does not include libwebp" otherwise.  Here the lossless bit stream is decoded on the host with
numpy; the lossy bit stream (`VP8 ` chunks: boolean-coded DCT blocks with intra prediction and a loop filter) is not built and
is refused with NotImplementedError.  The encoder writes a valid VP8L stream with the subtract-green transform, per-channel
prefix codes built from the image's histograms and run-length back references; it makes files every WebP reader opens, not
small ones.
"""
from __future__ import annotations

import heapq
import struct
from typing import List, Optional, Sequence, Tuple

import numpy as np

_CODE_LENGTH_ORDER = (17, 18, 0, 1, 2, 3, 4, 5, 16, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15)
_NUM_LENGTH_CODES, _NUM_DISTANCE_CODES = 24, 40

# (dx, dy) of the 120 short distance codes: the neighbourhood of the current pixel in order of increasing distance
_DISTANCE_MAP = (
    (0, 1), (1, 0), (1, 1), (-1, 1), (0, 2), (2, 0), (1, 2), (-1, 2), (2, 1), (-2, 1), (2, 2), (-2, 2), (0, 3), (3, 0), (1, 3),
    (-1, 3), (3, 1), (-3, 1), (2, 3), (-2, 3), (3, 2), (-3, 2), (0, 4), (4, 0), (1, 4), (-1, 4), (4, 1), (-4, 1), (3, 3), (-3, 3),
    (2, 4), (-2, 4), (4, 2), (-4, 2), (0, 5), (3, 4), (-3, 4), (4, 3), (-4, 3), (5, 0), (1, 5), (-1, 5), (5, 1), (-5, 1), (2, 5),
    (-2, 5), (5, 2), (-5, 2), (4, 4), (-4, 4), (3, 5), (-3, 5), (5, 3), (-5, 3), (0, 6), (6, 0), (1, 6), (-1, 6), (6, 1), (-6, 1),
    (2, 6), (-2, 6), (6, 2), (-6, 2), (4, 5), (-4, 5), (5, 4), (-5, 4), (3, 6), (-3, 6), (6, 3), (-6, 3), (0, 7), (7, 0), (1, 7),
    (-1, 7), (5, 5), (-5, 5), (7, 1), (-7, 1), (4, 6), (-4, 6), (6, 4), (-6, 4), (2, 7), (-2, 7), (7, 2), (-7, 2), (3, 7), (-3, 7),
    (7, 3), (-7, 3), (5, 6), (-5, 6), (6, 5), (-6, 5), (8, 0), (4, 7), (-4, 7), (7, 4), (-7, 4), (8, 1), (8, 2), (6, 6), (-6, 6),
    (8, 3), (5, 7), (-5, 7), (7, 5), (-7, 5), (8, 4), (6, 7), (-6, 7), (7, 6), (-7, 6), (8, 5), (7, 7), (-7, 7), (8, 6), (8, 7))
assert len(_DISTANCE_MAP) == 120


class _Bits:
    """LSB-first bit reader over a bytes object (Python integers as the bit reservoir)."""

    def __init__(self, data: bytes):
        self.v = int.from_bytes(data, "little")
        self.n = len(data) * 8
        self.pos = 0

    def read(self, k: int) -> int:
        if k == 0:
            return 0
        if self.pos + k > self.n:
            raise ValueError("bit stream ends early")
        r = (self.v >> self.pos) & ((1 << k) - 1)
        self.pos += k
        return r


class _Prefix:
    """Canonical prefix code from code lengths; symbols are decoded one bit at a time, most significant code bit first."""

    def __init__(self, lengths: Sequence[int]):
        used = [(l, s) for s, l in enumerate(lengths) if l > 0]
        self.single: Optional[int] = None
        if len(used) == 0:
            self.single = 0
            return
        if len(used) == 1:
            self.single = used[0][1]            # one symbol: no bits are read for it
            return
        used.sort()
        self.table = {}
        code, prev = 0, used[0][0]
        for l, s in used:
            code <<= (l - prev)
            prev = l
            self.table[(l, code)] = s
            code += 1
        self.max_len = used[-1][0]
        # complete (or over-subscribed) codes only: an incomplete code leaves bit patterns without a symbol
        if sum(1 << (self.max_len - l) for l, _ in used) != (1 << self.max_len):
            raise ValueError("prefix code is not complete")

    def read(self, br: _Bits) -> int:
        if self.single is not None:
            return self.single
        code = 0
        for l in range(1, self.max_len + 1):
            code = (code << 1) | br.read(1)
            s = self.table.get((l, code))
            if s is not None:
                return s
        raise ValueError("invalid prefix code")


def _read_code_lengths(br: _Bits, alphabet: int) -> List[int]:
    if br.read(1):                                        # simple code: one or two symbols
        n = br.read(1) + 1
        first = br.read(8 if br.read(1) else 1)
        lengths = [0] * alphabet
        if first >= alphabet:
            raise ValueError("symbol outside the alphabet")
        lengths[first] = 1
        if n == 2:
            second = br.read(8)
            if second >= alphabet:
                raise ValueError("symbol outside the alphabet")
            lengths[second] = 1
        return lengths
    ncl = 4 + br.read(4)
    cl = [0] * 19
    for i in range(ncl):
        cl[_CODE_LENGTH_ORDER[i]] = br.read(3)
    cl_code = _Prefix(cl)
    if br.read(1):
        nbits = 2 + 2 * br.read(3)
        max_symbol = 2 + br.read(nbits)
        if max_symbol > alphabet:
            raise ValueError("more code lengths than symbols")
    else:
        max_symbol = alphabet
    lengths = [0] * alphabet
    i, prev = 0, 8
    while i < alphabet and max_symbol > 0:
        max_symbol -= 1
        s = cl_code.read(br)
        if s < 16:
            lengths[i] = s
            i += 1
            if s:
                prev = s
        else:
            rep = {16: (2, 3), 17: (3, 3), 18: (7, 11)}[s]
            count = br.read(rep[0]) + rep[1]
            if i + count > alphabet:
                raise ValueError("code length run past the alphabet")
            if s == 16:
                lengths[i:i + count] = [prev] * count
            i += count
    return lengths


def _prefix_value(br: _Bits, prefix: int) -> int:
    if prefix < 4:
        return prefix + 1
    extra = (prefix - 2) >> 1
    return ((2 + (prefix & 1)) << extra) + br.read(extra) + 1


def _decode_image(br: _Bits, w: int, h: int, top: bool) -> np.ndarray:
    """One entropy-coded ARGB image (uint32 [h*w]); `top`: the main image, which may carry a meta prefix image."""
    cache_bits = br.read(4) if br.read(1) else 0
    if cache_bits and not (1 <= cache_bits <= 11):
        raise ValueError("colour cache size out of range")
    cache = [0] * (1 << cache_bits) if cache_bits else None
    meta, meta_bits, meta_w, groups = None, 0, 0, 1
    if top and br.read(1):
        meta_bits = br.read(3) + 2
        meta_w = (w + (1 << meta_bits) - 1) >> meta_bits
        meta_h = (h + (1 << meta_bits) - 1) >> meta_bits
        meta = (_decode_image(br, meta_w, meta_h, False) >> 8) & 0xFFFF
        groups = int(meta.max()) + 1
    sizes = (256 + _NUM_LENGTH_CODES + (1 << cache_bits if cache_bits else 0), 256, 256, 256, _NUM_DISTANCE_CODES)
    codes = [[_Prefix(_read_code_lengths(br, a)) for a in sizes] for _ in range(groups)]
    n = w * h
    out = [0] * n
    pos = 0
    g = codes[0]
    meta_list = meta.tolist() if meta is not None else None
    while pos < n:
        if meta is not None:
            y, x = divmod(pos, w)
            g = codes[meta_list[(y >> meta_bits) * meta_w + (x >> meta_bits)]]
        s = g[0].read(br)
        if s < 256:
            r = g[1].read(br)
            b = g[2].read(br)
            a = g[3].read(br)
            px = (a << 24) | (r << 16) | (s << 8) | b
            out[pos] = px
            pos += 1
            if cache is not None:
                cache[((0x1E35A7BD * px) & 0xFFFFFFFF) >> (32 - cache_bits)] = px
        elif s < 256 + _NUM_LENGTH_CODES:
            length = _prefix_value(br, s - 256)
            dcode = _prefix_value(br, g[4].read(br))
            if dcode > 120:
                dist = dcode - 120
            else:
                dx, dy = _DISTANCE_MAP[dcode - 1]
                dist = max(1, dx + dy * w)
            if dist > pos or pos + length > n:
                raise ValueError("back reference outside the image")
            for _ in range(length):
                px = out[pos - dist]
                out[pos] = px
                pos += 1
                if cache is not None:
                    cache[((0x1E35A7BD * px) & 0xFFFFFFFF) >> (32 - cache_bits)] = px
        else:
            if cache is None or s - 280 >= len(cache):
                raise ValueError("colour cache index without a cache")
            px = cache[s - 280]
            out[pos] = px
            pos += 1
    return np.array(out, dtype=np.uint32)


# ------------------------------------------------------------------------------------------------ inverse transforms
def _channels(px: np.ndarray):
    return (px >> 24) & 0xFF, (px >> 16) & 0xFF, (px >> 8) & 0xFF, px & 0xFF


def _avg2(a: int, b: int) -> int:
    return (((a ^ b) & 0xFEFEFEFE) >> 1) + (a & b)


def _add_px(a: int, b: int) -> int:
    """Per-channel sum modulo 256 of two packed ARGB values."""
    ag = (a & 0xFF00FF00) + (b & 0xFF00FF00)
    rb = (a & 0x00FF00FF) + (b & 0x00FF00FF)
    return (ag & 0xFF00FF00) | (rb & 0x00FF00FF)


def _select(l: int, t: int, tl: int) -> int:
    def dist(a, b):
        return (abs((a >> 24) - (b >> 24)) + abs(((a >> 16) & 255) - ((b >> 16) & 255)) + abs(((a >> 8) & 255) - ((b >> 8) & 255)) +
                abs((a & 255) - (b & 255)))
    return l if dist(t, tl) < dist(l, tl) else t          # |T - TL| is the distance of the gradient prediction from L


def _clamp_add_sub_full(a: int, b: int, c: int) -> int:
    out = 0
    for sh in (24, 16, 8, 0):
        v = ((a >> sh) & 255) + ((b >> sh) & 255) - ((c >> sh) & 255)
        out |= (0 if v < 0 else 255 if v > 255 else v) << sh
    return out


def _clamp_add_sub_half(a: int, b: int) -> int:
    out = 0
    for sh in (24, 16, 8, 0):
        x, y = (a >> sh) & 255, (b >> sh) & 255
        d = x - y
        v = x + (d // 2 if d >= 0 else -((-d) // 2))      # C division: towards zero
        out |= (0 if v < 0 else 255 if v > 255 else v) << sh
    return out


def _inverse_predictor(px: np.ndarray, w: int, h: int, bits: int, modes: np.ndarray) -> np.ndarray:
    res = px.tolist()
    out = [0] * (w * h)
    mw = (w + (1 << bits) - 1) >> bits
    mode_list = ((modes >> 8) & 0xFF).tolist()
    for y in range(h):
        row = y * w
        for x in range(w):
            i = row + x
            if y == 0:
                pred = 0xFF000000 if x == 0 else out[i - 1]
            elif x == 0:
                pred = out[i - w]
            else:
                m = mode_list[(y >> bits) * mw + (x >> bits)]
                l, t, tl, tr = out[i - 1], out[i - w], out[i - w - 1], out[i - w + 1]
                if m == 0: pred = 0xFF000000
                elif m == 1: pred = l
                elif m == 2: pred = t
                elif m == 3: pred = tr
                elif m == 4: pred = tl
                elif m == 5: pred = _avg2(_avg2(l, tr), t)
                elif m == 6: pred = _avg2(l, tl)
                elif m == 7: pred = _avg2(l, t)
                elif m == 8: pred = _avg2(tl, t)
                elif m == 9: pred = _avg2(t, tr)
                elif m == 10: pred = _avg2(_avg2(l, tl), _avg2(t, tr))
                elif m == 11: pred = _select(l, t, tl)
                elif m == 12: pred = _clamp_add_sub_full(l, t, tl)
                elif m == 13: pred = _clamp_add_sub_half(_avg2(l, t), tl)
                else: raise ValueError("predictor mode out of range")
            out[i] = _add_px(res[i], pred)
    return np.array(out, dtype=np.uint32)


def _s8(v: np.ndarray) -> np.ndarray:
    return ((v.astype(np.int32) + 128) & 0xFF) - 128


def _inverse_color(px: np.ndarray, w: int, h: int, bits: int, elems: np.ndarray) -> np.ndarray:
    mw = (w + (1 << bits) - 1) >> bits
    ys, xs = np.divmod(np.arange(w * h), w)
    e = elems[(ys >> bits) * mw + (xs >> bits)]
    _, r2b, g2b, g2r = _channels(e)                        # stored as red = red_to_blue, green = green_to_blue, blue = green_to_red
    a, r, g, b = _channels(px)
    sg = _s8(g)
    r = (r.astype(np.int32) + ((_s8(g2r) * sg) >> 5)) & 0xFF
    b = (b.astype(np.int32) + ((_s8(g2b) * sg) >> 5) + ((_s8(r2b) * _s8(r)) >> 5)) & 0xFF
    return ((a.astype(np.uint32) << 24) | (r.astype(np.uint32) << 16) | (g.astype(np.uint32) << 8) | b.astype(np.uint32)).astype(np.uint32)


def _inverse_subtract_green(px: np.ndarray) -> np.ndarray:
    a, r, g, b = _channels(px)
    return ((a << 24) | (((r + g) & 0xFF) << 16) | (g << 8) | ((b + g) & 0xFF)).astype(np.uint32)


def _inverse_indexing(px: np.ndarray, w: int, h: int, packed_w: int, width_bits: int, table: np.ndarray) -> np.ndarray:
    idx = ((px >> 8) & 0xFF).reshape(h, packed_w)
    if width_bits:
        per, bpp = 1 << width_bits, 8 >> width_bits
        parts = [(idx >> (bpp * k)) & ((1 << bpp) - 1) for k in range(per)]
        idx = np.stack(parts, -1).reshape(h, packed_w * per)[:, :w]
    lut = np.zeros(256, dtype=np.uint32)                   # indices past the table read transparent black
    lut[:len(table)] = table
    return lut[idx.reshape(-1)]


def DecodeWebp(data: bytes) -> np.ndarray:
    """uint8 [H, W, 3 or 4] of a lossless WebP file (alpha kept when the stream says it is used)."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WEBP":
        raise ValueError("not a WebP file")
    pos, payload = 12, None
    while pos + 4 <= len(data):
        tag = data[pos:pos + 4]
        if tag == b"VP8 ":
            raise NotImplementedError("lossy WebP (VP8) decoding is not part of this build")
        if pos + 8 > len(data):
            break
        size = struct.unpack_from("<I", data, pos + 4)[0]
        if tag == b"VP8L":
            payload = data[pos + 8:pos + 8 + size]
            break
        pos += 8 + size + (size & 1)
    if payload is None or len(payload) < 5 or payload[0] != 0x2F:
        raise ValueError("no VP8L bit stream in the file")
    br = _Bits(payload[1:])
    w, h = br.read(14) + 1, br.read(14) + 1
    has_alpha = br.read(1)
    if br.read(3) != 0:
        raise ValueError("unknown VP8L version")
    transforms, seen, cur_w = [], set(), w
    while br.read(1):
        kind = br.read(2)
        if kind in seen:
            raise ValueError("a transform appears twice")
        seen.add(kind)
        if kind in (0, 1):
            bits = br.read(3) + 2
            sub = _decode_image(br, (cur_w + (1 << bits) - 1) >> bits, (h + (1 << bits) - 1) >> bits, False)
            transforms.append((kind, bits, sub, cur_w))
        elif kind == 2:
            transforms.append((2, 0, None, cur_w))
        else:
            size = br.read(8) + 1
            table = _decode_image(br, size, 1, False)
            a, r, g, b = (np.cumsum(c.astype(np.int64)) & 0xFF for c in _channels(table))      # entries are stored as differences
            table = ((a << 24) | (r << 16) | (g << 8) | b).astype(np.uint32)
            width_bits = 3 if size <= 2 else 2 if size <= 4 else 1 if size <= 16 else 0
            transforms.append((3, width_bits, table, cur_w))
            cur_w = (cur_w + (1 << width_bits) - 1) >> width_bits
    px = _decode_image(br, cur_w, h, True)
    for kind, bits, aux, tw in reversed(transforms):
        if kind == 0:
            px = _inverse_predictor(px, tw, h, bits, aux)
        elif kind == 1:
            px = _inverse_color(px, tw, h, bits, aux)
        elif kind == 2:
            px = _inverse_subtract_green(px)
        else:
            px = _inverse_indexing(px, tw, h, (tw + (1 << bits) - 1) >> bits, bits, aux)
    a, r, g, b = _channels(px.reshape(h, w))
    chans = [r, g, b] + ([a] if has_alpha else [])
    return np.stack(chans, -1).astype(np.uint8)


# ------------------------------------------------------------------------------------------------------ encoder
class _BitWriter:
    def __init__(self):
        self.v, self.n = 0, 0

    def put(self, value: int, bits: int) -> None:
        self.v |= (value & ((1 << bits) - 1)) << self.n
        self.n += bits

    def bytes(self) -> bytes:
        return self.v.to_bytes((self.n + 7) // 8, "little")


def _huffman_lengths(hist: Sequence[int], limit: int = 15) -> List[int]:
    """Code lengths of a Huffman code over the symbols with a non-zero count, at most `limit` bits (the counts are flattened and
    the tree rebuilt until it fits)."""
    counts = list(hist)
    while True:
        heap = [(c, i, (i,)) for i, c in enumerate(counts) if c > 0]
        lengths = [0] * len(counts)
        if len(heap) == 1:
            lengths[heap[0][1]] = 1
            return lengths
        heapq.heapify(heap)
        tie = len(counts)
        while len(heap) > 1:
            c0, _, s0 = heapq.heappop(heap)
            c1, _, s1 = heapq.heappop(heap)
            for s in s0 + s1:
                lengths[s] += 1
            heapq.heappush(heap, (c0 + c1, tie, s0 + s1))
            tie += 1
        if max(lengths) <= limit:
            return lengths
        counts = [0 if c == 0 else (c >> 1) + 1 for c in counts]


def _canonical_codes(lengths: Sequence[int]) -> List[int]:
    codes, code, prev = [0] * len(lengths), 0, 0
    for l, s in sorted((l, s) for s, l in enumerate(lengths) if l > 0):
        code <<= (l - prev)
        prev = l
        codes[s] = code
        code += 1
    return codes


def _value_prefix(v: int) -> Tuple[int, int, int]:
    """(prefix symbol, number of extra bits, extra bits) of a length or distance value >= 1."""
    if v <= 4:
        return v - 1, 0, 0
    d = v - 1
    hb = d.bit_length() - 1
    return 2 * hb + ((d >> (hb - 1)) & 1), hb - 1, d & ((1 << (hb - 1)) - 1)


def _write_code(bw: _BitWriter, lengths: Sequence[int]) -> None:
    used = [s for s, l in enumerate(lengths) if l > 0]
    if len(used) <= 2 and all(s < 256 for s in used):
        if not used:
            used = [0]
        bw.put(1, 1)
        bw.put(len(used) - 1, 1)
        if used[0] < 2:
            bw.put(0, 1)
            bw.put(used[0], 1)
        else:
            bw.put(1, 1)
            bw.put(used[0], 8)
        if len(used) == 2:
            bw.put(used[1], 8)
        return
    bw.put(0, 1)
    bw.put(15, 4)                                          # all 19 code-length code lengths follow
    for sym in _CODE_LENGTH_ORDER:
        bw.put(4 if sym < 16 else 0, 3)                    # lengths 0..15 as a flat 4-bit code, no repeat symbols
    bw.put(0, 1)                                           # every symbol's length is listed
    for l in lengths:
        bw.put(int(f"{l:04b}"[::-1], 2), 4)                # canonical code of value l is l itself, most significant bit first


def EncodeWebp(pixels: np.ndarray) -> bytes:
    """Lossless WebP of a uint8 [H, W, C] image (C = 1 grey, 3 RGB, 4 RGBA)."""
    px = np.ascontiguousarray(pixels)
    if px.ndim == 2:
        px = px[:, :, None]
    if px.dtype != np.uint8 or px.ndim != 3 or px.shape[2] not in (1, 3, 4):
        raise ValueError("EncodeWebp takes uint8 [H, W, 1|3|4]")
    h, w, c = px.shape
    if not (1 <= w <= 16384 and 1 <= h <= 16384):
        raise ValueError("WebP images are at most 16384 x 16384")
    if c == 1:
        px = np.repeat(px, 3, 2)
    r, g, b = (px[:, :, k].astype(np.uint32) for k in range(3))
    a = px[:, :, 3].astype(np.uint32) if c == 4 else np.full((h, w), 255, np.uint32)
    argb = ((a << 24) | (((r - g) & 0xFF) << 16) | (g << 8) | ((b - g) & 0xFF)).reshape(-1)     # subtract-green applied
    n = w * h
    # run lengths against the previous pixel (distance 1) and the pixel above (distance w), from the end backwards
    def runs(dist: int) -> np.ndarray:
        same = np.zeros(n, dtype=bool)
        same[dist:] = argb[dist:] == argb[:-dist] if dist < n else False
        out = np.zeros(n + 1, dtype=np.int64)
        idx = np.arange(n)
        breaks = np.where(~same)[0]
        nxt = np.searchsorted(breaks, idx, side="left")
        end = np.where(nxt < len(breaks), breaks[np.minimum(nxt, len(breaks) - 1)], n)
        return (end - idx)[:n]
    run1, runw = runs(1).tolist(), (runs(w).tolist() if w > 1 and h > 1 else [0] * n)
    vals = argb.tolist()
    tokens = []                                            # (kind 0, argb) literal or (kind 1, length, distance code)
    pos = 0
    while pos < n:
        l1, lw = min(run1[pos], 4096), min(runw[pos], 4096)
        if max(l1, lw) >= 3:
            if l1 >= lw:
                tokens.append((1, l1, 2))                  # distance code 2 = (dx 1, dy 0): the previous pixel
                pos += l1
            else:
                tokens.append((1, lw, 1))                  # distance code 1 = (dx 0, dy 1): the pixel above
                pos += lw
        else:
            tokens.append((0, vals[pos], 0))
            pos += 1
    hist = [[0] * (256 + _NUM_LENGTH_CODES), [0] * 256, [0] * 256, [0] * 256, [0] * _NUM_DISTANCE_CODES]
    for kind, x, d in tokens:
        if kind == 0:
            hist[0][(x >> 8) & 255] += 1
            hist[1][(x >> 16) & 255] += 1
            hist[2][x & 255] += 1
            hist[3][x >> 24] += 1
        else:
            hist[0][256 + _value_prefix(x)[0]] += 1
            hist[4][_value_prefix(d)[0]] += 1
    lengths = [_huffman_lengths(hh) for hh in hist]
    codes = [_canonical_codes(l) for l in lengths]
    single = [sum(1 for l in ll if l > 0) <= 1 for ll in lengths]
    bw = _BitWriter()
    bw.put(w - 1, 14)
    bw.put(h - 1, 14)
    bw.put(1 if c == 4 else 0, 1)
    bw.put(0, 3)
    bw.put(1, 1); bw.put(2, 2)                             # one transform: subtract green
    bw.put(0, 1)                                           # no more transforms
    bw.put(0, 1)                                           # no colour cache
    bw.put(0, 1)                                           # one prefix-code group for the whole image
    for ll in lengths:
        _write_code(bw, ll)

    def emit(k: int, sym: int) -> None:
        if single[k]:
            return                                         # a code with one symbol takes no bits
        l = lengths[k][sym]
        bw.put(int(f"{codes[k][sym]:0{l}b}"[::-1], 2), l)
    for kind, x, d in tokens:
        if kind == 0:
            emit(0, (x >> 8) & 255); emit(1, (x >> 16) & 255); emit(2, x & 255); emit(3, x >> 24)
        else:
            p, nb, ex = _value_prefix(x)
            emit(0, 256 + p)
            bw.put(ex, nb)
            p, nb, ex = _value_prefix(d)
            emit(4, p)
            bw.put(ex, nb)
    payload = b"\x2f" + bw.bytes()
    pad = b"\0" if len(payload) & 1 else b""
    return b"RIFF" + struct.pack("<I", 4 + 8 + len(payload) + len(pad)) + b"WEBP" + b"VP8L" + struct.pack("<I", len(payload)) + payload + pad
