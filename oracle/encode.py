"""Chunk encoder used to WRITE parity and benchmark inputs.  Test infrastructure.

Restates the choices of the reference's encoder for byte, float and BF16 data
(lmz/codec.py: encode_chunk :914-1009, _encode_stream :307-393, _rans_cost
:410-436, _encode_bf16_cond :456-541, encode_delta :1018-1031) on top of the
checker's rANS encoder, which writes the reference encoder's exact bytes.  GGUF
block codecs are not on the decode path this repository covers and are absent.
"""
from __future__ import annotations

import zlib
from math import log2

import numpy as np

from . import native
from .codec import (BF16C_HDR, CODEC_BF16, CODEC_BF16C, CODEC_DELTA, CODEC_SPLIT,
                    CODEC_STORED, CODEC_ZSTD, COND_BUCKETS, COND_MIN_ELEMS, DELTA_HDR,
                    KIND_BF16, KIND_BYTES, M_DEFLATE, M_RANS, M_STORED, NOISE_BITS,
                    RANS_COST_SLACK, RANS_OVERHEAD, SAMPLE_BYTES)


def _min_gain(n: int) -> int:                     # lmz/codec.py:396-398
    return max(1024, n >> 8)


def _sample(a: np.ndarray) -> np.ndarray:         # :192-200
    n = a.size
    if n <= SAMPLE_BYTES:
        return a
    w = SAMPLE_BYTES // 3
    mid = (n - w) // 2
    return np.concatenate((a[:w], a[mid:mid + w], a[n - w:]))


def _hist_entropy(counts, total: int) -> float:   # :439-447
    if not total:
        return 0.0
    h = 0.0
    for c in counts:
        c = int(c)
        if c:
            p = c / total
            h -= p * log2(p)
    return h


def estimate_entropy(a: np.ndarray, L) -> float:  # :203-216
    s = _sample(a)
    if not s.size:
        return 0.0
    return _hist_entropy(L.histogram(s), s.size)


def _rans_cost(hist, total: int, L):              # :410-436
    if int(np.sum(hist, dtype=np.uint64)) != total:
        return None
    freqs = L.rans_freqs(hist)
    if freqs is None:
        return None
    scale = int(freqs.astype(np.int64).sum())
    if not scale:
        return None
    bits = 0.0
    for c, f in zip(hist.tolist(), freqs.tolist()):
        if c:
            bits -= c * log2(f / scale)
    return RANS_OVERHEAD + int(bits / 8) - RANS_COST_SLACK


def _est_stream(total: int, h: float) -> int:     # :450-454
    if total == 0:
        return 0
    return min(total, int(total * h / 8) + RANS_OVERHEAD)


def encode_stream(a: np.ndarray, L, level: int = 1, plane: bool = False, hist=None):
    """(method, payload bytes-like) for one stream (lmz/codec.py:307-393).

    The general-purpose coder is deflate, as on any image without zstd
    (lmz/entropy.py:88-89)."""
    n = a.size
    if n == 0:
        return M_STORED, b""
    if hist is None and plane:
        if estimate_entropy(a, L) >= NOISE_BITS:
            return M_STORED, a
        hist = L.histogram(a)
    cost = _rans_cost(hist, n, L) if hist is not None else None
    if cost is not None:
        hopeless = cost + _min_gain(n) >= n
    else:
        hopeless = estimate_entropy(a, L) >= NOISE_BITS
    if hopeless:
        return M_STORED, a
    if plane:
        best, method = L.rans_encode(a, hist), M_RANS
    else:
        best, method = zlib.compress(a.tobytes(), min(max(level, 1), 9)), M_DEFLATE
        if len(best) > n - (n >> 5):
            alt = L.rans_encode(a, hist)
            if len(alt) < len(best):
                best, method = alt, M_RANS
    if len(best) + _min_gain(n) >= n:
        return M_STORED, a
    return method, best


def _encode_bf16_cond(exp, sm, nelem, L, level):
    """lmz/codec.py:456-541; returns the payload parts or None to decline."""
    ehist = L.histogram(exp)
    lut = L.bucket_lut(ehist, COND_BUCKETS)
    part, counts = L.bucket_partition(exp, sm, lut, COND_BUCKETS)
    est_cond, seg_hists, pos = 0, [], 0
    for c in counts.tolist():
        if not c:
            seg_hists.append(None)
            continue
        h = L.histogram(part[pos:pos + c])
        seg_hists.append(h)
        est_cond += _est_stream(c, _hist_entropy(h, c))
        pos += c
    taken = [h for h in seg_hists if h is not None]
    shist = np.sum(taken, axis=0, dtype=np.uint64) if taken else np.zeros(256, np.uint64)
    est_plain = _est_stream(nelem, _hist_entropy(shist, nelem))
    if est_cond + (BF16C_HDR.size - 8) + 512 >= est_plain:
        return None
    exp_used, exp_payload = encode_stream(exp, L, level, plane=True, hist=ehist)
    sm_methods, seg_lens, parts, pos = [], [], [], 0
    for c, h in zip(counts.tolist(), seg_hists):
        if c == 0:
            sm_methods.append(M_STORED)
            seg_lens.append(0)
            continue
        used, payload = encode_stream(part[pos:pos + c], L, level, plane=True, hist=h)
        sm_methods.append(used)
        seg_lens.append(len(payload))
        parts.append(payload)
        pos += c
    header = BF16C_HDR.pack(COND_BUCKETS, exp_used, *sm_methods, len(exp_payload), *seg_lens)
    return [header, exp_payload] + parts


def encode_chunk(data, esize: int, kind: int = KIND_BYTES, level: int = 1,
                 checksum: bool = True, lib=None):
    """(parts, codec, flags, crc) for one chunk (lmz/codec.py:914-1009)."""
    L = lib or native.best()
    O = native.oracle()
    a = native._arr(data)
    n = a.size
    crc = (zlib.crc32(a) & 0xFFFFFFFF) if checksum else 0
    nplanes = 0
    if kind == KIND_BF16 and esize == 2 and n % 2 == 0:
        nplanes, cid = 2, CODEC_BF16
        pa, pb = L.split_bf16(a)
        planes = [pa, pb]
        nelem = n // 2
        if nelem >= COND_MIN_ELEMS:
            parts = _encode_bf16_cond(pa, pb, nelem, L, level)
            if parts is not None and sum(len(p) for p in parts) + _min_gain(n) < n:
                return parts, CODEC_BF16C, 0, crc
    elif esize in (2, 4, 8) and n % esize == 0:
        nplanes, cid = esize, CODEC_SPLIT
        flat = (L if hasattr(L, "split_planes") else O).split_planes(a, esize)
        nelem = n // esize
        planes = [flat[k * nelem:(k + 1) * nelem] for k in range(esize)]
    if nplanes:
        parts, lengths, flags, total, any_coded = [], [], 0, 0, False
        for k in range(nplanes):
            used, payload = encode_stream(planes[k], L, level, plane=True)
            flags |= (used & 3) << (2 * k)
            lengths.append(len(payload))
            parts.append(payload)
            total += len(payload)
            any_coded |= used != M_STORED
        if any_coded and total + 4 * nplanes < n:
            hdr = np.asarray(lengths, dtype="<u4").tobytes()
            return [hdr] + parts, cid, flags, crc
        return [a], CODEC_STORED, 0, crc
    used, payload = encode_stream(a, L, level, plane=False)
    if used == M_STORED:
        return [a], CODEC_STORED, 0, crc
    return [payload], CODEC_ZSTD, used & 3, crc


def shared_table_for(exp_planes, own_lengths, L):
    """The table a run of exponent planes would share -- the reference's normalisation of
    their summed histogram (scratchpad/gpu/shared_enc.c:49-85), so every symbol that occurs
    anywhere can be coded -- or None when the run is cheaper with its own tables.  The choice
    is by measured cross-entropy (docs/gpu-residency-handover.md:60-63): the bits the shared
    table would spend on the run plus its 516 bytes, against the streams as they are."""
    hists = [L.histogram(p).astype(np.float64) for p in exp_planes]
    total = np.sum(hists, axis=0)
    freqs = L.rans_freqs(total.astype(np.uint64))
    if freqs is None:
        return None
    f = freqs.astype(np.float64)
    bits = float(np.sum(total[f > 0] * -np.log2(f[f > 0] / 4096.0)))
    shared = bits / 8.0 + 32 * len(exp_planes) + 516
    return freqs if shared < float(sum(own_lengths)) else None


def encode_bf16t(data, freqs, table_off: int, L, checksum: bool = True):
    """(parts, crc) of a shared-table BF16 chunk (codec.CODEC_BF16T), or None when the
    exponent plane does not pay against `freqs`."""
    from .codec import BF16T_HDR
    a = native._arr(data)
    pa, pb = L.split_bf16(a)
    stream = L.rans_encode_shared(pa, freqs)
    if BF16T_HDR.size + len(stream) + pb.size >= a.size:
        return None
    crc = (zlib.crc32(a) & 0xFFFFFFFF) if checksum else 0
    return [BF16T_HDR.pack(len(stream), pb.size, table_off), stream, pb], crc


def encode_delta(data, base, esize: int, kind: int, src: int, level: int = 1,
                 checksum: bool = True, lib=None):
    """(parts, flags, crc); the codec id is CODEC_DELTA (lmz/codec.py:1018-1031)."""
    L = lib or native.best()
    a = native._arr(data)
    crc = (zlib.crc32(a) & 0xFFFFFFFF) if checksum else 0
    diff = L.xor(a, base)
    parts, cid, flags, _ = encode_chunk(diff, esize, kind, level, False, L)
    return [DELTA_HDR.pack(src, cid)] + list(parts), flags, crc
