"""Per-chunk decode (the checker) and encode (the input writer).

Test infrastructure only.  The decode side restates what the reference does
to one chunk payload; the encode side restates the reference's choices closely
enough that, for BF16 / float / byte data, it writes the same chunk bytes the
reference's encoder writes (the test-suite holds it to that against archives
the reference itself wrote).  The encode side exists because parity and
benchmark inputs have to be produced where the reference's Python cannot go.

Reference: lmz/codec.py (decode_chunk :1149-1230, _decode_bf16c :1075-1146,
decode_delta :1045-1057, encode_chunk :914-1009, _encode_stream :307-393,
_encode_bf16_cond :456-541, encode_delta :1018-1031).
"""
from __future__ import annotations

import struct
import zlib
from math import log2

import numpy as np

from . import native

CODEC_STORED, CODEC_ZSTD, CODEC_SPLIT, CODEC_BF16, CODEC_REF = 0, 1, 2, 3, 4
CODEC_BF16C, CODEC_BLK, CODEC_GBLK, CODEC_DELTA = 5, 6, 7, 8
# Shared-table option (the format lever of docs/gpu-residency-handover.md:37-66, which the
# reference proposes but does not define; this layout is this repository's): a BF16 chunk
# whose exponent plane is coded against a 516-byte table stored ONCE in the payload region
# for a run of chunks.  Payload = <IIQ (plane 0 length, plane 1 length, file offset of the
# table), plane 0 as [8 states][words] (scratchpad/gpu/shared_enc.c:1-13), plane 1 stored.
CODEC_BF16T = 9
BF16T_HDR = struct.Struct("<IIQ")
FLAG_SHARED_TABLES = 4         # archive header flag: some chunks are CODEC_BF16T
M_STORED, M_ZSTD, M_DEFLATE, M_RANS = 0, 1, 2, 3
KIND_BYTES, KIND_BF16 = 0, 1

NOISE_BITS = 7.98              # lmz/codec.py:32
SAMPLE_BYTES = 3 * 65536       # :36
COND_BUCKETS = 8               # :43
COND_MIN_ELEMS = 1 << 20       # :44
RANS_OVERHEAD = 516 + 32       # :48
RANS_COST_SLACK = 64           # :406
BF16C_HDR = struct.Struct("<BB8BI8I")   # :50
DELTA_HDR = struct.Struct("<QB")        # :1015


class Corrupt(ValueError):
    """A payload that does not decode (the reference's CorruptArchive)."""


def _lib(lib=None):
    return lib or native.best()


# ------------------------------------------------------------------- decode

def decode_stream(raw, method: int, n: int, lib=None) -> np.ndarray:
    """One coded stream -> n bytes (lmz/entropy.py:117-136)."""
    if method == M_STORED:
        out = np.frombuffer(bytes(raw), dtype=np.uint8)
    elif method == M_RANS:
        try:
            out = _lib(lib).rans_decode(raw, n)
        except ValueError as exc:
            raise Corrupt(str(exc)) from exc
    elif method == M_DEFLATE:
        try:
            out = np.frombuffer(zlib.decompress(bytes(raw)), dtype=np.uint8)
        except zlib.error as exc:
            raise Corrupt(str(exc)) from exc
    else:
        raise Corrupt(f"method {method} is not decodable on this image")
    if out.size != n:
        raise Corrupt(f"stream decoded to {out.size} bytes, expected {n}")
    return out


def decode_bf16c(payload, nelem: int, lib=None) -> np.ndarray:
    """Exponent-conditioned BF16 chunk (lmz/codec.py:1075-1146)."""
    L = _lib(lib)
    p = native._arr(payload)
    if p.size < BF16C_HDR.size:
        raise Corrupt("conditioned bf16 chunk is truncated")
    f = BF16C_HDR.unpack_from(p, 0)
    k, exp_m, sm_m, exp_len, seg_lens = f[0], f[1], f[2:10], f[10], f[11:19]
    if k != COND_BUCKETS:
        raise Corrupt(f"conditioned bf16 chunk declares {k} buckets")
    if any(m not in (0, 1, 2, 3) for m in (exp_m, *sm_m)):
        raise Corrupt("conditioned bf16 chunk names an unknown method")
    pos = BF16C_HDR.size
    if pos + exp_len > p.size:
        raise Corrupt("conditioned bf16 chunk is truncated")
    if exp_m == M_STORED and exp_len != nelem:
        raise Corrupt("stored exponent plane has the wrong length")
    exp = decode_stream(p[pos:pos + exp_len], exp_m, nelem, L)
    pos += exp_len
    hist = L.histogram(exp)
    lut = L.bucket_lut(hist, k)
    counts = L.bucket_counts(hist, lut, k)
    segs = []
    for b in range(k):
        ln, want = seg_lens[b], int(counts[b])
        if pos + ln > p.size:
            raise Corrupt("conditioned bf16 chunk is truncated")
        if want == 0:
            if ln:
                raise Corrupt(f"bucket {b} should be empty")
            segs.append(np.zeros(0, dtype=np.uint8))
        elif sm_m[b] == M_STORED:
            if ln != want:
                raise Corrupt(f"bucket {b} holds {ln} bytes, expected {want}")
            segs.append(p[pos:pos + ln])
        else:
            segs.append(decode_stream(p[pos:pos + ln], sm_m[b], want, L))
        pos += ln
    sm = L.bucket_unpartition(exp, segs, lut, k)
    return L.merge_bf16(exp, sm)


def decode_chunk(payload, codec: int, esize: int, flags: int, rlen: int,
                 crc: int = 0, verify: bool = True, lib=None) -> np.ndarray:
    """One non-ref, non-delta chunk -> rlen bytes (lmz/codec.py:1149-1230)."""
    L = _lib(lib)
    p = native._arr(payload)
    if codec == CODEC_STORED:
        if p.size != rlen:
            raise Corrupt(f"stored chunk is {p.size} bytes, expected {rlen}")
        out = p
    elif codec == CODEC_BF16C:
        if esize != 2 or rlen % 2:
            raise Corrupt("a conditioned bf16 chunk must have 2-byte elements")
        out = decode_bf16c(p, rlen // 2, L)
    elif codec == CODEC_ZSTD:
        out = decode_stream(p, flags & 3, rlen, L)
    elif codec in (CODEC_SPLIT, CODEC_BF16):
        if esize not in (2, 4, 8) or rlen % esize or (codec == CODEC_BF16 and esize != 2):
            raise Corrupt(f"split chunk has invalid element size {esize}")
        nplanes = 2 if codec == CODEC_BF16 else esize
        nelem = rlen // nplanes
        hdr = 4 * nplanes
        if p.size < hdr:
            raise Corrupt("split chunk is truncated")
        lens = struct.unpack_from(f"<{nplanes}I", p, 0)
        pos, planes = hdr, []
        for k, ln in enumerate(lens):
            if pos + ln > p.size:
                raise Corrupt("split chunk is truncated")
            m = (flags >> (2 * k)) & 3
            if m == M_STORED and ln != nelem:
                raise Corrupt(f"plane {k} holds {ln} bytes, expected {nelem}")
            planes.append(decode_stream(p[pos:pos + ln], m, nelem, L))
            pos += ln
        if codec == CODEC_BF16:
            out = L.merge_bf16(planes[0], planes[1])
        else:
            out = native.oracle().merge_planes(planes, esize)
    else:
        raise Corrupt(f"codec {codec} is outside the decode path this checker covers")
    if verify and crc and (zlib.crc32(out) & 0xFFFFFFFF) != crc:
        raise Corrupt("chunk failed its checksum")
    return out


def decode_bf16t(payload, rlen: int, crc: int, verify: bool, lib, blob) -> np.ndarray:
    """A shared-table BF16 chunk: prepending the table makes the exponent stream an ordinary
    lmz stream again (scratchpad/gpu/prep_shared.py:101-112)."""
    L = _lib(lib)
    p = native._arr(payload)
    if rlen % 2 or p.size < BF16T_HDR.size:
        raise Corrupt("shared-table bf16 chunk is truncated")
    len0, len1, toff = BF16T_HDR.unpack_from(p, 0)
    nelem = rlen // 2
    if BF16T_HDR.size + len0 + len1 > p.size or len1 != nelem:
        raise Corrupt("shared-table bf16 chunk has inconsistent plane lengths")
    whole = native._arr(blob)
    if toff < 32 or toff + 516 > whole.size:
        raise Corrupt("shared-table bf16 chunk names a table outside the file")
    table = whole[toff:toff + 516]
    stream = np.concatenate((table, p[BF16T_HDR.size:BF16T_HDR.size + len0]))
    exp = decode_stream(stream, M_RANS, nelem, L)
    sm = p[BF16T_HDR.size + len0:BF16T_HDR.size + len0 + len1]
    out = L.merge_bf16(exp, sm)
    if verify and crc and (zlib.crc32(out) & 0xFFFFFFFF) != crc:
        raise Corrupt("chunk failed its checksum")
    return out


def delta_source(payload):
    """(src, inner codec, data offset) of a delta payload (lmz/codec.py:1034-1042)."""
    p = native._arr(payload)
    if p.size < DELTA_HDR.size:
        raise Corrupt("delta chunk is truncated")
    src, inner = DELTA_HDR.unpack_from(p, 0)
    if inner in (CODEC_REF, CODEC_DELTA):
        raise Corrupt(f"delta chunk names codec {inner} for its own difference")
    return src, inner, DELTA_HDR.size


def decode_delta(payload, esize, flags, rlen, base, crc=0, verify=True, lib=None):
    """base XOR decoded difference (lmz/codec.py:1045-1057)."""
    _src, inner, off = delta_source(payload)
    base = native._arr(base)
    if base.size != rlen:
        raise Corrupt("delta source has the wrong length")
    diff = decode_chunk(native._arr(payload)[off:], inner, esize, flags, rlen, 0, False, lib)
    out = _lib(lib).xor(base, diff)
    if verify and crc and (zlib.crc32(out) & 0xFFFFFFFF) != crc:
        raise Corrupt("chunk failed its checksum")
    return out
