"""ctypes bindings for the checker libraries.  Test infrastructure only.

Two libraries with the same job:

``Oracle``  -- ``liblmzoracle.so``, this repository's scalar restatement
              (``oracle/lmz_oracle.c``), always available (built by ``make``).
``Ref``     -- ``_ref/liblmzcore.so`` + ``_ref/liblmzshared.so``, the
              reference's own C sources compiled where they lie.  Present when
              ``oracle/Makefile`` could see the reference tree (or when a
              prebuilt copy travelled with the repository).

Both expose the same Python methods so a test can run one against the other.
Buffers are numpy ``uint8`` arrays or anything exposing the buffer protocol.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_u8p = ctypes.c_void_p
_sz = ctypes.c_size_t


def _arr(buf) -> np.ndarray:
    """A contiguous uint8 view of ``buf`` (copying only when it must)."""
    if isinstance(buf, np.ndarray):
        a = buf if buf.dtype == np.uint8 else buf.view(np.uint8)
        return np.ascontiguousarray(a).reshape(-1)
    return np.frombuffer(buf, dtype=np.uint8)


def _p(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def build(force: bool = False) -> None:
    """Compile the checker libraries with ``make`` (a few hundred ms)."""
    if force or not os.path.exists(os.path.join(HERE, "liblmzoracle.so")):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)


class _Base:
    """Shared Python surface; subclasses bind symbol names."""

    name = "?"

    # -- streams -------------------------------------------------------------
    def rans_bound(self, n: int) -> int:
        return 516 + 2 * n + 32 + 64

    def rans_encode(self, src, counts=None) -> bytes:
        a = _arr(src)
        cap = self.rans_bound(a.size)
        dst = np.empty(cap, dtype=np.uint8)
        c = None
        if counts is not None:
            c = np.asarray(counts, dtype=np.uint64)
        n = self._encode(_p(a), a.size, _p(dst), cap, _p(c) if c is not None else None)
        if n < 0:
            raise ValueError("rANS encode failed")
        return dst[:n].tobytes()

    def rans_decode(self, stream, n: int) -> np.ndarray:
        s = _arr(stream)
        out = np.empty(n, dtype=np.uint8)
        if self._decode(_p(s), s.size, _p(out), n) != 0:
            raise ValueError("malformed rANS stream")
        return out

    def histogram(self, buf) -> np.ndarray:
        a = _arr(buf)
        h = np.zeros(256, dtype=np.uint64)
        if a.size:
            self._hist(_p(a), a.size, _p(h))
        return h

    def rans_freqs(self, counts) -> np.ndarray | None:
        c = np.asarray(counts, dtype=np.uint64)
        f = np.zeros(256, dtype=np.uint16)
        if self._normalize(_p(c), _p(f)) != 0:
            return None
        return f

    # -- planes --------------------------------------------------------------
    def split_bf16(self, src):
        a = _arr(src)
        n = a.size // 2
        pa = np.empty(n, dtype=np.uint8)
        pb = np.empty(n, dtype=np.uint8)
        self._split_bf16(_p(a), _p(pa), _p(pb), n)
        return pa, pb

    def merge_bf16(self, pa, pb) -> np.ndarray:
        pa, pb = _arr(pa), _arr(pb)
        out = np.empty(2 * pa.size, dtype=np.uint8)
        self._merge_bf16(_p(pa), _p(pb), _p(out), pa.size)
        return out

    def bucket_lut(self, hist, k: int = 8) -> np.ndarray:
        h = np.asarray(hist, dtype=np.uint64)
        lut = np.zeros(256, dtype=np.uint8)
        if self._bucket_lut(_p(h), k, _p(lut)) != 0:
            raise ValueError("bad bucket count")
        return lut

    def bucket_counts(self, hist, lut, k: int = 8) -> np.ndarray:
        return np.bincount(np.asarray(lut, dtype=np.int64),
                           weights=np.asarray(hist, dtype=np.float64),
                           minlength=k).astype(np.uint64)[:k]

    def bucket_unpartition(self, ctx, segs, lut, k: int = 8) -> np.ndarray:
        ctx = _arr(ctx)
        keep = [_arr(s) if len(s) else np.zeros(1, dtype=np.uint8) for s in segs]
        ptrs = (ctypes.c_void_p * k)(*[a.ctypes.data for a in keep])
        out = np.empty(ctx.size, dtype=np.uint8)
        lut = _arr(lut)
        if self._unpartition(_p(ctx), ptrs, ctx.size, _p(lut), k, _p(out)) != 0:
            raise ValueError("unpartition failed")
        return out

    def xor(self, a, b) -> np.ndarray:
        a, b = _arr(a), _arr(b)
        out = np.empty(a.size, dtype=np.uint8)
        self._xor(_p(a), _p(b), a.size, _p(out))
        return out


class Oracle(_Base):
    """This repository's restatement (oracle/lmz_oracle.c)."""

    name = "port"

    def __init__(self):
        build()
        L = ctypes.CDLL(os.path.join(HERE, "liblmzoracle.so"))
        self.lib = L
        L.orc_rans_encode.restype = ctypes.c_long
        L.orc_rans_encode.argtypes = [_u8p, _sz, _u8p, _sz, _u8p]
        L.orc_rans_encode_shared.restype = ctypes.c_long
        L.orc_rans_encode_shared.argtypes = [_u8p, _sz, _u8p, _u8p, _sz]
        L.orc_rans_decode.argtypes = [_u8p, _sz, _u8p, _sz]
        L.orc_rans_decode_ex.argtypes = [_u8p, _sz, _u8p, _sz, _u8p]
        L.orc_rans_decode_shared.argtypes = [_u8p, _u8p, _sz, _u8p, _sz]
        L.orc_hist.restype = None
        L.orc_hist.argtypes = [_u8p, _sz, _u8p]
        L.orc_rans_normalize.argtypes = [_u8p, _u8p]
        L.orc_split_bf16.restype = None
        L.orc_split_bf16.argtypes = [_u8p, _u8p, _u8p, _sz]
        L.orc_merge_bf16.restype = None
        L.orc_merge_bf16.argtypes = [_u8p, _u8p, _u8p, _sz]
        L.orc_split_planes.restype = None
        L.orc_split_planes.argtypes = [_u8p, _u8p, _sz, _sz]
        L.orc_merge_planes.restype = None
        L.orc_merge_planes.argtypes = [_u8p, _u8p, _sz, _sz]
        L.orc_bucket_lut.argtypes = [_u8p, _sz, _u8p]
        L.orc_bucket_partition.argtypes = [_u8p, _u8p, _sz, _u8p, _sz, _u8p, _u8p]
        L.orc_bucket_unpartition.argtypes = [_u8p, _u8p, _sz, _u8p, _sz, _u8p]
        L.orc_xor.restype = None
        L.orc_xor.argtypes = [_u8p, _u8p, _sz, _u8p]
        L.orc_crc32.restype = ctypes.c_uint32
        L.orc_crc32.argtypes = [ctypes.c_uint32, _u8p, _sz]
        L.orc_decode_planes.argtypes = [_u8p, _sz, _sz, _sz, ctypes.c_uint32,
                                        ctypes.c_int, _u8p, _u8p]
        self._encode = L.orc_rans_encode
        self._decode = L.orc_rans_decode
        self._hist = L.orc_hist
        self._normalize = L.orc_rans_normalize
        self._split_bf16 = L.orc_split_bf16
        self._merge_bf16 = L.orc_merge_bf16
        self._bucket_lut = L.orc_bucket_lut
        self._unpartition = L.orc_bucket_unpartition
        self._xor = L.orc_xor

    def rans_decode_ex(self, stream, n: int):
        """Decode and also return (final 8 states, final cursor offset)."""
        s = _arr(stream)
        out = np.empty(n, dtype=np.uint8)
        end = np.zeros(9, dtype=np.uint32)
        if self.lib.orc_rans_decode_ex(_p(s), s.size, _p(out), n, _p(end)) != 0:
            raise ValueError("malformed rANS stream")
        return out, end[:8].copy(), int(end[8])

    def rans_encode_shared(self, src, freqs) -> bytes:
        a = _arr(src)
        f = np.asarray(freqs, dtype=np.uint16)
        cap = 2 * a.size + 64
        dst = np.empty(cap, dtype=np.uint8)
        n = self.lib.orc_rans_encode_shared(_p(a), a.size, _p(f), _p(dst), cap)
        if n < 0:
            raise ValueError(f"shared-table encode failed ({n})")
        return dst[:n].tobytes()

    def rans_decode_shared(self, hdr, stream, n: int) -> np.ndarray:
        h, s = _arr(hdr), _arr(stream)
        out = np.empty(n, dtype=np.uint8)
        if self.lib.orc_rans_decode_shared(_p(h), _p(s), s.size, _p(out), n) != 0:
            raise ValueError("malformed rANS stream")
        return out

    def crc32(self, buf, crc: int = 0) -> int:
        a = _arr(buf)
        return int(self.lib.orc_crc32(crc, _p(a), a.size))

    def split_planes(self, src, esize: int) -> np.ndarray:
        a = _arr(src)
        out = np.empty(a.size, dtype=np.uint8)
        self.lib.orc_split_planes(_p(a), _p(out), a.size // esize, esize)
        return out

    def merge_planes(self, planes, esize: int) -> np.ndarray:
        keep = [_arr(x) for x in planes]
        n = keep[0].size
        ptrs = (ctypes.c_void_p * esize)(*[a.ctypes.data for a in keep])
        out = np.empty(n * esize, dtype=np.uint8)
        self.lib.orc_merge_planes(ptrs, _p(out), n, esize)
        return out

    def bucket_partition(self, ctx, val, lut, k: int = 8):
        ctx, val, lut = _arr(ctx), _arr(val), _arr(lut)
        out = np.empty(ctx.size, dtype=np.uint8)
        counts = np.zeros(k, dtype=np.uint64)
        self.lib.orc_bucket_partition(_p(ctx), _p(val), ctx.size, _p(lut), k,
                                      _p(out), _p(counts))
        return out, counts

    def decode_planes(self, payload, nplanes, nelem, methods, bf16) -> np.ndarray | int:
        p = _arr(payload)
        dst = np.empty(nplanes * nelem, dtype=np.uint8)
        scratch = np.empty(nplanes * nelem, dtype=np.uint8)
        rc = self.lib.orc_decode_planes(_p(p), p.size, nplanes, nelem, methods,
                                        1 if bf16 else 0, _p(dst), _p(scratch))
        return dst if rc == 0 else rc


class Ref(_Base):
    """The reference's own compiled C core (oracle/_ref/*.so)."""

    name = "reference"

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", "liblmzcore.so"))

    def __init__(self):
        L = ctypes.CDLL(os.path.join(HERE, "_ref", "liblmzcore.so"))
        self.lib = L
        L.lmz_rans_encode_h.restype = ctypes.c_long
        L.lmz_rans_encode_h.argtypes = [_u8p, _sz, _u8p, _sz, _u8p]
        L.lmz_rans_encode_portable.restype = ctypes.c_long
        L.lmz_rans_encode_portable.argtypes = [_u8p, _sz, _u8p, _sz, _u8p]
        L.lmz_rans_decode.argtypes = [_u8p, _sz, _u8p, _sz]
        L.lmz_hist.restype = None
        L.lmz_hist.argtypes = [_u8p, _sz, _u8p]
        L.lmz_rans_freqs.argtypes = [_u8p, _u8p]
        L.lmz_split_bf16.argtypes = [_u8p, _u8p, _u8p, _sz]
        L.lmz_merge_bf16.argtypes = [_u8p, _u8p, _u8p, _sz]
        L.lmz_bucket_lut.argtypes = [_u8p, _sz, _u8p]
        L.lmz_bucket_partition.argtypes = [_u8p, _u8p, _sz, _u8p, _sz, _u8p, _u8p, _u8p]
        L.lmz_bucket_unpartition.argtypes = [_u8p, _u8p, _sz, _u8p, _sz, _u8p]
        L.lmz_xor.argtypes = [_u8p, _u8p, _sz, _u8p]
        L.lmz_split.argtypes = [_u8p, _u8p, _sz, _sz, _u8p]
        L.lmz_merge_planes.argtypes = [_u8p, _u8p, _sz, _sz, _u8p]
        L.lmz_scratch_size.restype = _sz
        L.lmz_scratch_size.argtypes = [_sz, _sz]
        L.lmz_decode_planes.argtypes = [_u8p, _sz, _sz, _sz, ctypes.c_uint32,
                                        ctypes.c_int, _u8p, _u8p, _sz]
        self._encode = L.lmz_rans_encode_h
        self._decode = L.lmz_rans_decode
        self._hist = L.lmz_hist
        self._normalize = L.lmz_rans_freqs
        self._split_bf16 = L.lmz_split_bf16
        self._merge_bf16 = L.lmz_merge_bf16
        self._bucket_lut = L.lmz_bucket_lut
        self._unpartition = L.lmz_bucket_unpartition
        self._xor = L.lmz_xor
        sp = os.path.join(HERE, "_ref", "liblmzshared.so")
        self.shared = ctypes.CDLL(sp) if os.path.exists(sp) else None
        if self.shared is not None:
            self.shared.lmzx_encode_shared.restype = ctypes.c_long
            self.shared.lmzx_encode_shared.argtypes = [_u8p, _sz, _u8p, _u8p, _sz]

    def rans_encode_portable(self, src) -> bytes:
        a = _arr(src)
        cap = self.rans_bound(a.size)
        dst = np.empty(cap, dtype=np.uint8)
        n = self.lib.lmz_rans_encode_portable(_p(a), a.size, _p(dst), cap, None)
        if n < 0:
            raise ValueError("rANS encode failed")
        return dst[:n].tobytes()

    def rans_encode_shared(self, src, freqs) -> bytes:
        a = _arr(src)
        f = np.asarray(freqs, dtype=np.uint16)
        cap = 2 * a.size + 64
        dst = np.empty(cap, dtype=np.uint8)
        n = self.shared.lmzx_encode_shared(_p(a), a.size, _p(f), _p(dst), cap)
        if n < 0:
            raise ValueError(f"shared-table encode failed ({n})")
        return dst[:n].tobytes()

    def split_planes(self, src, esize: int) -> np.ndarray:
        a = _arr(src)
        nelem = a.size // esize
        out = np.empty(a.size, dtype=np.uint8)
        scratch = np.empty(max(1, self.lib.lmz_scratch_size(nelem, esize)), dtype=np.uint8)
        self.lib.lmz_split(_p(a), _p(out), nelem, esize, _p(scratch))
        return out

    def bucket_partition(self, ctx, val, lut, k: int = 8):
        ctx, val, lut = _arr(ctx), _arr(val), _arr(lut)
        out = np.empty(ctx.size, dtype=np.uint8)
        counts = np.zeros(k, dtype=np.uint64)
        self.lib.lmz_bucket_partition(_p(ctx), _p(val), ctx.size, _p(lut), k,
                                      _p(out), _p(counts), None)
        return out, counts

    def decode_planes(self, payload, nplanes, nelem, methods, bf16) -> np.ndarray | int:
        p = _arr(payload)
        dst = np.empty(nplanes * nelem, dtype=np.uint8)
        need = nplanes * nelem + self.lib.lmz_scratch_size(nelem, nplanes)
        scratch = np.empty(max(1, need), dtype=np.uint8)
        rc = self.lib.lmz_decode_planes(_p(p), p.size, nplanes, nelem, methods,
                                        1 if bf16 else 0, _p(dst), _p(scratch), scratch.size)
        return dst if rc == 0 else rc


_oracle = None
_ref = None


def oracle() -> Oracle:
    global _oracle
    if _oracle is None:
        _oracle = Oracle()
    return _oracle


def ref() -> Ref | None:
    """The compiled reference core, or None when it was never built."""
    global _ref
    if _ref is None and Ref.available():
        _ref = Ref()
    return _ref


def best():
    """The fastest checker for bulk work: the compiled reference when present."""
    return ref() or oracle()
