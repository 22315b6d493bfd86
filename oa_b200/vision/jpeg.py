"""Baseline JPEG decoder and encoder (ITU-T T.81 sequential DCT, Huffman coding).

The reference decodes JPEG through a bundled decoder (Source/Private/Oa/Vision/Image); this is a from-the-standard
implementation.  Decoder: SOF0 / SOF1 frames with 8-bit samples, 1 or 3 components, any sampling factors up to 2 x 2 (4:4:4,
4:2:2, 4:2:0, 4:4:0), DQT with 8- or 16-bit entries, DHT, DRI / RSTn restart intervals, JFIF and Adobe APP14 colour hints
(YCbCr by default, RGB when Adobe says transform 0), stuffed bytes and fill bytes, and progressive frames (SOF2: spectral
selection and successive approximation, interleaved DC and per-component AC scans, end-of-band runs).  Lossless, hierarchical and
arithmetic-coded streams are refused with NotImplementedError.  The entropy decode walks the bit stream on the host; the
inverse DCT, chroma up-sampling (the centred triangular filter that libjpeg applies by default for a factor of 2, pixel
replication otherwise) and colour conversion run as batched array operations over all blocks.  Encoder: baseline, quality-scaled Annex K tables, 4:4:4 or 4:2:0, optional restart interval.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Optional, Tuple

import numpy as np

ZIGZAG = np.array([0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6, 7, 14, 21, 28, 35, 42, 49, 56,
                   57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63])

# 8 x 8 DCT-II basis: C[u, x] = a(u) cos((2x + 1) u pi / 16) / 2
_C = np.array([[(np.sqrt(0.5) if u == 0 else 1.0) * np.cos((2 * x + 1) * u * np.pi / 16) / 2 for x in range(8)] for u in range(8)])


class _Huff:
    """Canonical Huffman table: code lengths 1..16 -> (mincode, maxcode, value pointer) lookup as in Annex F.2.2.3."""

    def __init__(self, counts: List[int], values: List[int]):
        self.values = values
        self.mincode, self.maxcode, self.valptr = [0] * 17, [-1] * 17, [0] * 17
        code = k = 0
        for ln in range(1, 17):
            self.valptr[ln] = k
            self.mincode[ln] = code
            code += counts[ln - 1]
            k += counts[ln - 1]
            self.maxcode[ln] = code - 1 if counts[ln - 1] else -1
            code <<= 1
        # encoder side: value -> (code, length)
        self.enc: Dict[int, Tuple[int, int]] = {}
        code = k = 0
        for ln in range(1, 17):
            for _ in range(counts[ln - 1]):
                self.enc[values[k]] = (code, ln)
                code += 1
                k += 1
            code <<= 1


class _Bits:
    """Entropy-coded segment reader: removes byte stuffing, stops at markers."""

    def __init__(self, data: bytes, pos: int):
        self.d, self.p, self.acc, self.n, self.marker = data, pos, 0, 0, 0

    def _fill(self) -> None:
        while self.n <= 24:
            if self.marker or self.p >= len(self.d):
                b = 0
            else:
                b = self.d[self.p]
                self.p += 1
                if b == 0xFF:
                    nxt = self.d[self.p] if self.p < len(self.d) else 0xD9
                    if nxt == 0:
                        self.p += 1
                    else:
                        self.marker = nxt          # a marker ends the segment: feed zeros from here on
                        self.p -= 1
                        b = 0
            self.acc = (self.acc << 8) | b
            self.n += 8

    def bits(self, k: int) -> int:
        if k == 0:
            return 0
        if self.n < k:
            self._fill()
        self.n -= k
        return (self.acc >> self.n) & ((1 << k) - 1)

    def decode(self, h: _Huff) -> int:
        code = 0
        for ln in range(1, 17):
            code = (code << 1) | self.bits(1)
            if h.maxcode[ln] >= 0 and code <= h.maxcode[ln] and code >= h.mincode[ln]:
                return h.values[h.valptr[ln] + code - h.mincode[ln]]
        raise ValueError("bad Huffman code")

    def receive_extend(self, s: int) -> int:
        if s == 0:
            return 0
        v = self.bits(s)
        return v if v >= (1 << (s - 1)) else v - (1 << s) + 1

    def restart(self) -> None:
        """Byte-align and step over the RSTn marker."""
        self.acc = self.n = 0
        if self.marker and 0xD0 <= self.marker <= 0xD7:
            self.p += 2
            self.marker = 0
        else:                                       # tolerate fill bytes before the marker
            while self.p + 1 < len(self.d) and not (self.d[self.p] == 0xFF and 0xD0 <= self.d[self.p + 1] <= 0xD7):
                self.p += 1
            self.p += 2
            self.marker = 0


def _upsample(plane: np.ndarray, fy: int, fx: int) -> np.ndarray:
    """Chroma up-sampling by 2 with the centred triangular filter (3/4, 1/4), by replication for other factors."""
    p = plane.astype(np.float32)
    if fx == 2:
        left = np.concatenate([p[:, :1], p[:, :-1]], 1)
        right = np.concatenate([p[:, 1:], p[:, -1:]], 1)
        out = np.empty((p.shape[0], p.shape[1] * 2), np.float32)
        out[:, 0::2] = 0.75 * p + 0.25 * left
        out[:, 1::2] = 0.75 * p + 0.25 * right
        p = out
    elif fx > 1:
        p = np.repeat(p, fx, 1)
    if fy == 2:
        up = np.concatenate([p[:1], p[:-1]], 0)
        down = np.concatenate([p[1:], p[-1:]], 0)
        out = np.empty((p.shape[0] * 2, p.shape[1]), np.float32)
        out[0::2] = 0.75 * p + 0.25 * up
        out[1::2] = 0.75 * p + 0.25 * down
        p = out
    elif fy > 1:
        p = np.repeat(p, fy, 0)
    return p


def DecodeJpeg(data: bytes) -> np.ndarray:
    """-> uint8 [H, W, 1] (greyscale) or [H, W, 3] (RGB)."""
    if data[:2] != b"\xff\xd8":
        raise ValueError("no SOI marker")
    pos = 2
    qt: Dict[int, np.ndarray] = {}
    huff: Dict[Tuple[int, int], _Huff] = {}
    frame = None
    restart_interval = 0
    adobe_transform: Optional[int] = None
    coeffs = None
    while pos < len(data):
        if data[pos] != 0xFF:
            pos += 1
            continue
        while pos < len(data) and data[pos] == 0xFF:
            pos += 1
        m = data[pos]
        pos += 1
        if m == 0xD9:
            break
        if m == 0x01 or 0xD0 <= m <= 0xD7:
            continue
        ln = struct.unpack(">H", data[pos:pos + 2])[0]
        seg = data[pos + 2:pos + ln]
        if len(seg) != ln - 2:
            raise ValueError("truncated segment")
        pos += ln
        if m == 0xDB:
            i = 0
            while i < len(seg):
                pq, tq = seg[i] >> 4, seg[i] & 15
                i += 1
                if pq:
                    vals = np.frombuffer(seg[i:i + 128], ">u2").astype(np.float32)
                    i += 128
                else:
                    vals = np.frombuffer(seg[i:i + 64], np.uint8).astype(np.float32)
                    i += 64
                if vals.size != 64:
                    raise ValueError("short quantisation table")
                q = np.zeros(64, np.float32)
                q[ZIGZAG] = vals
                qt[tq] = q
        elif m == 0xC4:
            i = 0
            while i < len(seg):
                tc, th = seg[i] >> 4, seg[i] & 15
                counts = list(seg[i + 1:i + 17])
                n = sum(counts)
                values = list(seg[i + 17:i + 17 + n])
                if len(counts) != 16 or len(values) != n:
                    raise ValueError("short Huffman table")
                huff[(tc, th)] = _Huff(counts, values)
                i += 17 + n
        elif m in (0xC0, 0xC1, 0xC2):
            prec, h, w, nc = seg[0], struct.unpack(">H", seg[1:3])[0], struct.unpack(">H", seg[3:5])[0], seg[5]
            if prec != 8:
                raise NotImplementedError("JPEG with samples other than 8 bits")
            if nc not in (1, 3) or h == 0 or w == 0:
                raise NotImplementedError(f"JPEG with {nc} components")
            comps = [{"id": seg[6 + 3 * c], "h": seg[7 + 3 * c] >> 4, "v": seg[7 + 3 * c] & 15, "tq": seg[8 + 3 * c]} for c in range(nc)]
            if any(not (1 <= c["h"] <= 2 and 1 <= c["v"] <= 2) for c in comps):
                raise NotImplementedError("JPEG sampling factors above 2")
            if nc == 1:
                comps[0]["h"] = comps[0]["v"] = 1      # a single component is never interleaved: its sampling factors do not order anything
            frame = {"h": h, "w": w, "comps": comps, "progressive": m == 0xC2}
            if m == 0xC2:
                _geometry(frame)
                coeffs = [np.zeros((frame["mcuy"] * c["v"], frame["mcux"] * c["h"], 64), np.int32) for c in comps]
        elif m in (0xC3, 0xC5, 0xC6, 0xC7, 0xC9, 0xCA, 0xCB, 0xCD, 0xCE, 0xCF):
            raise NotImplementedError("lossless, hierarchical or arithmetic-coded JPEG")
        elif m == 0xDD:
            restart_interval = struct.unpack(">H", seg[:2])[0]
        elif m == 0xEE and seg[:5] == b"Adobe" and len(seg) >= 12:
            adobe_transform = seg[11]
        elif m == 0xDA:
            if frame is None:
                raise ValueError("scan before frame header")
            ns = seg[0]
            if frame["progressive"]:
                scan = []
                for k in range(ns):
                    cid, tbl = seg[1 + 2 * k], seg[2 + 2 * k]
                    ci = next(i for i, c in enumerate(frame["comps"]) if c["id"] == cid)
                    scan.append((ci, tbl >> 4, tbl & 15))
                ss, se, ah, al = seg[1 + 2 * ns], seg[2 + 2 * ns], seg[3 + 2 * ns] >> 4, seg[3 + 2 * ns] & 15
                pos = _decode_progressive_scan(data, pos, frame, huff, restart_interval, scan, ss, se, ah, al, coeffs)
                continue
            if ns != len(frame["comps"]):
                raise NotImplementedError("non-interleaved baseline scans")
            for k in range(ns):
                cid, tbl = seg[1 + 2 * k], seg[2 + 2 * k]
                comp = next(c for c in frame["comps"] if c["id"] == cid)
                comp["td"], comp["ta"] = tbl >> 4, tbl & 15
            coeffs, pos = _decode_scan(data, pos, frame, huff, restart_interval)
    if frame is None or coeffs is None:
        raise ValueError("no image data")
    return _reconstruct(frame, coeffs, qt, adobe_transform)


def _geometry(frame) -> None:
    comps = frame["comps"]
    hmax, vmax = max(c["h"] for c in comps), max(c["v"] for c in comps)
    mcux, mcuy = -(-frame["w"] // (8 * hmax)), -(-frame["h"] // (8 * vmax))
    frame.update(hmax=hmax, vmax=vmax, mcux=mcux, mcuy=mcuy)


def _next_marker(data, end: int) -> int:
    while end + 1 < len(data) and not (data[end] == 0xFF and data[end + 1] not in (0, 0xFF) and not (0xD0 <= data[end + 1] <= 0xD7)):
        end += 1
    return end


def _decode_progressive_scan(data, pos, frame, huff, restart_interval, scan, ss, se, ah, al, coeffs) -> int:
    """One scan of a progressive frame (ITU T.81 Annex G): a band [ss, se] of the zig-zag order at bit position al, either its first
    pass (ah = 0) or a refinement of one more bit.  DC scans may interleave components; AC scans carry one component and use
    end-of-band runs.  The coefficients accumulate in `coeffs` (natural order) and are dequantised after the last scan."""
    comps = frame["comps"]
    if ss > se or se > 63 or (ss == 0 and se != 0) or (ss > 0 and len(scan) != 1):
        raise ValueError("bad spectral selection")
    br = _Bits(data, pos)
    p1, m1 = 1 << al, -(1 << al)
    if len(scan) == 1:                          # non-interleaved: the component's own blocks in raster order
        ci = scan[0][0]
        c = comps[ci]
        bw = -(-(-(-frame["w"] * c["h"] // frame["hmax"])) // 8)
        bh = -(-(-(-frame["h"] * c["v"] // frame["vmax"])) // 8)
        units = [[(ci, y, x)] for y in range(bh) for x in range(bw)]
    else:
        units = []
        for my in range(frame["mcuy"]):
            for mx in range(frame["mcux"]):
                units.append([(ci, my * comps[ci]["v"] + by, mx * comps[ci]["h"] + bx)
                              for ci, _, _ in scan for by in range(comps[ci]["v"]) for bx in range(comps[ci]["h"])])
    tables = {ci: (huff.get((0, td)), huff.get((1, ta))) for ci, td, ta in scan}
    pred = {ci: 0 for ci, _, _ in scan}
    eobrun = 0
    for n, unit in enumerate(units):
        if restart_interval and n and n % restart_interval == 0:
            br.restart()
            pred = {ci: 0 for ci in pred}
            eobrun = 0
        for ci, by, bx in unit:
            blk = coeffs[ci][by, bx]
            dc_t, ac_t = tables[ci]
            if ss == 0:
                if ah == 0:
                    if dc_t is None:
                        raise ValueError("missing DC table")
                    pred[ci] += br.receive_extend(br.decode(dc_t))
                    blk[0] = pred[ci] * p1
                elif br.bits(1):
                    blk[0] |= p1
                continue
            if ac_t is None:
                raise ValueError("missing AC table")
            if ah == 0:                         # first pass of an AC band
                if eobrun:
                    eobrun -= 1
                    continue
                k = ss
                while k <= se:
                    rs = br.decode(ac_t)
                    r, s_ = rs >> 4, rs & 15
                    if s_ == 0:
                        if r < 15:
                            eobrun = (1 << r) - 1 + (br.bits(r) if r else 0)
                            break
                        k += 16
                        continue
                    k += r
                    if k > se:
                        raise ValueError("AC coefficient index beyond the band")
                    blk[ZIGZAG[k]] = br.receive_extend(s_) * p1
                    k += 1
                continue
            # refinement of an AC band: new coefficients of magnitude 1 << al, one correction bit for every known non-zero one
            k = ss
            if eobrun == 0:
                while k <= se:
                    rs = br.decode(ac_t)
                    r, s_ = rs >> 4, rs & 15
                    value = 0
                    if s_ == 0:
                        if r < 15:
                            eobrun = (1 << r) + (br.bits(r) if r else 0)     # this block counts as the first of the run
                            break
                    elif s_ == 1:
                        value = p1 if br.bits(1) else m1
                    else:
                        raise ValueError("refinement coefficient larger than one bit")
                    while k <= se:
                        z = ZIGZAG[k]
                        k += 1
                        if blk[z] != 0:
                            if br.bits(1) and (blk[z] & p1) == 0:
                                blk[z] += p1 if blk[z] > 0 else m1
                        else:
                            if r == 0:
                                if value:
                                    blk[z] = value
                                break
                            r -= 1
            if eobrun:
                while k <= se:                  # the rest of the band only receives correction bits
                    z = ZIGZAG[k]
                    k += 1
                    if blk[z] != 0 and br.bits(1) and (blk[z] & p1) == 0:
                        blk[z] += p1 if blk[z] > 0 else m1
                eobrun -= 1
    return _next_marker(data, br.p)


def _decode_scan(data, pos, frame, huff, restart_interval):
    comps = frame["comps"]
    _geometry(frame)
    hmax, vmax, mcux, mcuy = frame["hmax"], frame["vmax"], frame["mcux"], frame["mcuy"]
    out = [np.zeros((mcuy * c["v"], mcux * c["h"], 64), np.int32) for c in comps]
    br = _Bits(data, pos)
    pred = [0] * len(comps)
    tables = [(huff[(0, c["td"])], huff[(1, c["ta"])]) for c in comps]
    count = 0
    for my in range(mcuy):
        for mx in range(mcux):
            if restart_interval and count and count % restart_interval == 0:
                br.restart()
                pred = [0] * len(comps)
            count += 1
            for ci, c in enumerate(comps):
                dc_t, ac_t = tables[ci]
                for by in range(c["v"]):
                    for bx in range(c["h"]):
                        blk = out[ci][my * c["v"] + by, mx * c["h"] + bx]
                        pred[ci] += br.receive_extend(br.decode(dc_t))
                        blk[0] = pred[ci]
                        k = 1
                        while k < 64:
                            rs = br.decode(ac_t)
                            r, s = rs >> 4, rs & 15
                            if s == 0:
                                if r == 15:
                                    k += 16
                                    continue
                                break
                            k += r
                            if k > 63:
                                raise ValueError("AC coefficient index beyond the block")
                            blk[ZIGZAG[k]] = br.receive_extend(s)
                            k += 1
    end = br.p
    # continue after the entropy-coded segment: the next marker
    while end + 1 < len(data) and not (data[end] == 0xFF and data[end + 1] not in (0, 0xFF) and not (0xD0 <= data[end + 1] <= 0xD7)):
        end += 1
    return out, end


def _reconstruct(frame, coeffs, qt, adobe_transform) -> np.ndarray:
    comps = frame["comps"]
    planes = []
    for ci, c in enumerate(comps):
        if c["tq"] not in qt:
            raise ValueError("missing quantisation table")
        blocks = coeffs[ci].astype(np.float32) * qt[c["tq"]]
        by, bx = blocks.shape[:2]
        f = blocks.reshape(by, bx, 8, 8)
        px = np.einsum("ua,yzuv,vb->yzab", _C, f, _C) + 128.0          # C^T F C per block
        plane = px.transpose(0, 2, 1, 3).reshape(by * 8, bx * 8)
        planes.append(_upsample(plane, frame["vmax"] // c["v"], frame["hmax"] // c["h"]))
    h, w = frame["h"], frame["w"]
    planes = [p[:h, :w] for p in planes]
    if len(planes) == 1:
        return np.clip(np.rint(planes[0]), 0, 255).astype(np.uint8)[:, :, None]
    ids = bytes(c["id"] for c in comps)
    is_rgb = adobe_transform == 0 or (adobe_transform is None and ids == b"RGB")
    if is_rgb:
        rgb = np.stack(planes, -1)
    else:
        y, cb, cr = planes[0], planes[1] - 128.0, planes[2] - 128.0
        rgb = np.stack([y + 1.402 * cr, y - 0.344136 * cb - 0.714136 * cr, y + 1.772 * cb], -1)
    return np.clip(np.rint(rgb), 0, 255).astype(np.uint8)


# ------------------------------------------------------------------------------------------------------------- encoder
_QL = [16, 11, 10, 16, 24, 40, 51, 61, 12, 12, 14, 19, 26, 58, 60, 55, 14, 13, 16, 24, 40, 57, 69, 56, 14, 17, 22, 29, 51, 87, 80, 62,
       18, 22, 37, 56, 68, 109, 103, 77, 24, 35, 55, 64, 81, 104, 113, 92, 49, 64, 78, 87, 103, 121, 120, 101, 72, 92, 95, 98, 112, 100, 103, 99]
_QC = [17, 18, 24, 47, 99, 99, 99, 99, 18, 21, 26, 66, 99, 99, 99, 99, 24, 26, 56, 99, 99, 99, 99, 99, 47, 66, 99, 99, 99, 99, 99, 99] + [99] * 32
# Annex K.3 typical Huffman tables: (counts per code length, values)
_DC_L = ([0, 1, 5, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0], list(range(12)))
_DC_C = ([0, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0], list(range(12)))
_AC_L = ([0, 2, 1, 3, 3, 2, 4, 3, 5, 5, 4, 4, 0, 0, 1, 0x7d],
         [0x01, 0x02, 0x03, 0x00, 0x04, 0x11, 0x05, 0x12, 0x21, 0x31, 0x41, 0x06, 0x13, 0x51, 0x61, 0x07, 0x22, 0x71, 0x14, 0x32, 0x81, 0x91, 0xa1, 0x08,
          0x23, 0x42, 0xb1, 0xc1, 0x15, 0x52, 0xd1, 0xf0, 0x24, 0x33, 0x62, 0x72, 0x82, 0x09, 0x0a, 0x16, 0x17, 0x18, 0x19, 0x1a, 0x25, 0x26, 0x27, 0x28,
          0x29, 0x2a, 0x34, 0x35, 0x36, 0x37, 0x38, 0x39, 0x3a, 0x43, 0x44, 0x45, 0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58, 0x59,
          0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68, 0x69, 0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a, 0x83, 0x84, 0x85, 0x86, 0x87, 0x88, 0x89,
          0x8a, 0x92, 0x93, 0x94, 0x95, 0x96, 0x97, 0x98, 0x99, 0x9a, 0xa2, 0xa3, 0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4, 0xb5, 0xb6,
          0xb7, 0xb8, 0xb9, 0xba, 0xc2, 0xc3, 0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6, 0xd7, 0xd8, 0xd9, 0xda, 0xe1, 0xe2,
          0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf1, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8, 0xf9, 0xfa])
_AC_C = ([0, 2, 1, 2, 4, 4, 3, 4, 7, 5, 4, 4, 0, 1, 2, 0x77],
         [0x00, 0x01, 0x02, 0x03, 0x11, 0x04, 0x05, 0x21, 0x31, 0x06, 0x12, 0x41, 0x51, 0x07, 0x61, 0x71, 0x13, 0x22, 0x32, 0x81, 0x08, 0x14, 0x42, 0x91,
          0xa1, 0xb1, 0xc1, 0x09, 0x23, 0x33, 0x52, 0xf0, 0x15, 0x62, 0x72, 0xd1, 0x0a, 0x16, 0x24, 0x34, 0xe1, 0x25, 0xf1, 0x17, 0x18, 0x19, 0x1a, 0x26,
          0x27, 0x28, 0x29, 0x2a, 0x35, 0x36, 0x37, 0x38, 0x39, 0x3a, 0x43, 0x44, 0x45, 0x46, 0x47, 0x48, 0x49, 0x4a, 0x53, 0x54, 0x55, 0x56, 0x57, 0x58,
          0x59, 0x5a, 0x63, 0x64, 0x65, 0x66, 0x67, 0x68, 0x69, 0x6a, 0x73, 0x74, 0x75, 0x76, 0x77, 0x78, 0x79, 0x7a, 0x82, 0x83, 0x84, 0x85, 0x86, 0x87,
          0x88, 0x89, 0x8a, 0x92, 0x93, 0x94, 0x95, 0x96, 0x97, 0x98, 0x99, 0x9a, 0xa2, 0xa3, 0xa4, 0xa5, 0xa6, 0xa7, 0xa8, 0xa9, 0xaa, 0xb2, 0xb3, 0xb4,
          0xb5, 0xb6, 0xb7, 0xb8, 0xb9, 0xba, 0xc2, 0xc3, 0xc4, 0xc5, 0xc6, 0xc7, 0xc8, 0xc9, 0xca, 0xd2, 0xd3, 0xd4, 0xd5, 0xd6, 0xd7, 0xd8, 0xd9, 0xda,
          0xe2, 0xe3, 0xe4, 0xe5, 0xe6, 0xe7, 0xe8, 0xe9, 0xea, 0xf2, 0xf3, 0xf4, 0xf5, 0xf6, 0xf7, 0xf8, 0xf9, 0xfa])


def _scaled(table, quality: int) -> np.ndarray:
    quality = min(100, max(1, int(quality)))
    scale = 5000 // quality if quality < 50 else 200 - 2 * quality
    return np.clip((np.array(table) * scale + 50) // 100, 1, 255).astype(np.int32)


class _Writer:
    def __init__(self):
        self.out = bytearray()
        self.acc = self.n = 0

    def put(self, code: int, ln: int) -> None:
        self.acc = (self.acc << ln) | (code & ((1 << ln) - 1))
        self.n += ln
        while self.n >= 8:
            b = (self.acc >> (self.n - 8)) & 0xFF
            self.out.append(b)
            if b == 0xFF:
                self.out.append(0)
            self.n -= 8
        self.acc &= (1 << self.n) - 1

    def flush(self) -> None:
        if self.n:
            self.put((1 << (8 - self.n)) - 1, 8 - self.n)          # pad with ones


def _blocks(plane: np.ndarray, q: np.ndarray) -> np.ndarray:
    """[H, W] (multiples of 8) -> quantised coefficients [H/8, W/8, 64] in natural order."""
    h, w = plane.shape
    b = (plane.astype(np.float32) - 128.0).reshape(h // 8, 8, w // 8, 8).transpose(0, 2, 1, 3)
    f = np.einsum("ua,yzab,vb->yzuv", _C, b, _C)
    return np.rint(f.reshape(h // 8, w // 8, 64) / q).astype(np.int32)


def _size(v: int) -> int:
    return int(abs(v)).bit_length()


def _encode_block(w: _Writer, blk: np.ndarray, pred: int, dc: _Huff, ac: _Huff) -> int:
    d = int(blk[0]) - pred
    s = _size(d)
    w.put(*dc.enc[s])
    if s:
        w.put(d if d >= 0 else d + (1 << s) - 1, s)
    run = 0
    zz = blk[ZIGZAG]
    last = int(np.max(np.nonzero(zz)[0])) if np.any(zz[1:]) else 0
    for k in range(1, last + 1):
        v = int(zz[k])
        if v == 0:
            run += 1
            continue
        while run > 15:
            w.put(*ac.enc[0xF0])
            run -= 16
        s = _size(v)
        w.put(*ac.enc[(run << 4) | s])
        w.put(v if v >= 0 else v + (1 << s) - 1, s)
        run = 0
    if last < 63:
        w.put(*ac.enc[0x00])
    return int(blk[0])


def EncodeJpeg(img: np.ndarray, quality: int = 90, subsample: bool = True, restart_interval: int = 0) -> bytes:
    """uint8 [H, W], [H, W, 1] or [H, W, 3] (RGB; an alpha channel is dropped) -> baseline JFIF stream."""
    if img.ndim == 2:
        img = img[:, :, None]
    if img.shape[2] == 4:
        img = img[:, :, :3]
    if img.shape[2] not in (1, 3) or img.dtype != np.uint8:
        raise ValueError("EncodeJpeg takes uint8 greyscale or RGB pixels")
    h, w, nc = img.shape
    ql, qc = _scaled(_QL, quality), _scaled(_QC, quality)
    if nc == 1:
        planes, samp = [img[:, :, 0].astype(np.float32)], [(1, 1)]
    else:
        r, g, b = (img[:, :, i].astype(np.float32) for i in range(3))
        planes = [0.299 * r + 0.587 * g + 0.114 * b, -0.168736 * r - 0.331264 * g + 0.5 * b + 128.0, 0.5 * r - 0.418688 * g - 0.081312 * b + 128.0]
        samp = [(2, 2), (1, 1), (1, 1)] if subsample else [(1, 1)] * 3
    hmax, vmax = max(s[0] for s in samp), max(s[1] for s in samp)
    mcux, mcuy = -(-w // (8 * hmax)), -(-h // (8 * vmax))
    coeffs = []
    for p, (sh, sv) in zip(planes, samp):
        p = np.pad(p, ((0, mcuy * 8 * vmax - h), (0, mcux * 8 * hmax - w)), mode="edge")
        fy, fx = vmax // sv, hmax // sh
        if fy > 1 or fx > 1:                                        # box filter down-sampling
            p = p.reshape(p.shape[0] // fy, fy, p.shape[1] // fx, fx).mean((1, 3))
        coeffs.append(_blocks(np.clip(p, 0, 255), ql if len(coeffs) == 0 else qc))
    out = bytearray(b"\xff\xd8\xff\xe0" + struct.pack(">H5sBBBHHBB", 16, b"JFIF\0", 1, 1, 0, 1, 1, 0, 0))
    for tq, q in ((0, ql), (1, qc))[:1 if nc == 1 else 2]:
        out += b"\xff\xdb" + struct.pack(">HB", 67, tq) + bytes(int(v) for v in q[ZIGZAG])
    out += b"\xff\xc0" + struct.pack(">HBHHB", 8 + 3 * nc, 8, h, w, nc)
    for i, (sh, sv) in enumerate(samp):
        out += bytes([i + 1, (sh << 4) | sv, 0 if i == 0 else 1])
    tables = [(0, 0, _DC_L), (1, 0, _AC_L)] + ([(0, 1, _DC_C), (1, 1, _AC_C)] if nc == 3 else [])
    for tc, th, (counts, values) in tables:
        out += b"\xff\xc4" + struct.pack(">HB", 19 + len(values), (tc << 4) | th) + bytes(counts) + bytes(values)
    if restart_interval:
        out += b"\xff\xdd" + struct.pack(">HH", 4, restart_interval)
    out += b"\xff\xda" + struct.pack(">HB", 6 + 2 * nc, nc)
    for i in range(nc):
        out += bytes([i + 1, 0x00 if i == 0 else 0x11])
    out += bytes([0, 63, 0])
    huffs = [(_Huff(*_DC_L), _Huff(*_AC_L))] + [(_Huff(*_DC_C), _Huff(*_AC_C))] * 2
    wr = _Writer()
    pred = [0] * nc
    count = rst = 0
    for my in range(mcuy):
        for mx in range(mcux):
            if restart_interval and count and count % restart_interval == 0:
                wr.flush()
                wr.out += bytes([0xFF, 0xD0 + (rst & 7)])
                rst += 1
                pred = [0] * nc
            count += 1
            for ci, (sh, sv) in enumerate(samp):
                for by in range(sv):
                    for bx in range(sh):
                        pred[ci] = _encode_block(wr, coeffs[ci][my * sv + by, mx * sh + bx], pred[ci], *huffs[ci])
    wr.flush()
    return bytes(out) + bytes(wr.out) + b"\xff\xd9"
