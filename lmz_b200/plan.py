"""Turn an archive's chunk records into device job arrays.

Host-side counterpart of the reference's per-chunk decode dispatch
(lmz/codec.py:1149-1230, lmz/api.py:867-886), restructured for the GPU: no
chunk is decoded here, the records and the small in-payload headers are only
*classified*, with numpy over all chunks at once (an archive cut into 64 KiB
blocks has hundreds of thousands of records, so nothing runs per chunk in
Python).  The result is the set of arrays `lmz_gpu_decode_chunks_dev` takes:

  stream jobs   every rANS stream whose decoded length is known from the record
  chunk jobs    how each chunk's output is assembled (copy / BF16 merge / byte
                interleave / exponent-conditioned), grouped pass 1 then pass 2
  cond jobs     framing of exponent-conditioned BF16 chunks (lmz/codec.py:1082-1142)
  pieces        64 KiB slices of chunk output, the unit the finish kernel works on

Refs and deltas (pass 2) read output that pass 1 wrote; as in the reference a
source must lie wholly on plain chunks (single hop, lmz/api.py:832-864).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field

import numpy as np

from . import archive as fmt
from .archive import CorruptArchive, FormatError

PIECE = 65536
NONE64 = np.uint64(0xFFFFFFFFFFFFFFFF)
K_COPY, K_BF16, K_SPLIT, K_COND = 0, 1, 2, 3

STREAM_JOB = np.dtype([("src_off", "<u8"), ("dst_off", "<u8"), ("src_len", "<u4"), ("n", "<u4"),
                       ("flags", "<u4"), ("aux", "<u4")])
CHUNK_JOB = np.dtype([("dst_off", "<u8"), ("base_off", "<u8"), ("plane_off", "<u8", 8),
                      ("rlen", "<u4"), ("crc", "<u4"), ("piece0", "<u4"), ("aux", "<u4"),
                      ("kind", "u1"), ("esize", "u1"), ("scratch_mask", "u1"),
                      ("src_is_out", "u1"), ("record", "<u4")])
COND_JOB = np.dtype([("exp_off", "<u8"), ("seg_src", "<u8", 8), ("seg_scratch", "<u8"),
                     ("seg_len", "<u4", 8), ("nelem", "<u4"), ("seg_job0", "<u4"),
                     ("piece0", "<u4"), ("chunk", "<u4"), ("seg_method", "u1", 8),
                     ("exp_in_scratch", "u1"), ("pad", "u1", 7)])
FUSED_JOB = np.dtype([("src_off", "<u8"), ("mant_off", "<u8"), ("dst_off", "<u8"),
                      ("src_len", "<u4"), ("n", "<u4"), ("piece0", "<u4"), ("flags", "<u4")])
COND_STATE_BYTES = 360
T_GROUP = 80                   # shared-table chunks one thread block decodes against one table (lmz_gpu_shared_group)
TABLE_STRIDE = 528             # spacing of the tables handed to the device
BF16T_HDR = np.dtype([("len0", "<u4"), ("len1", "<u4"), ("table", "<u8")])
BF16C_HDR = np.dtype([("k", "u1"), ("exp_m", "u1"), ("sm_m", "u1", 8), ("exp_len", "<u4"),
                      ("seg_len", "<u4", 8)])       # lmz/codec.py:50
assert (STREAM_JOB.itemsize, CHUNK_JOB.itemsize, COND_JOB.itemsize, BF16C_HDR.itemsize) == \
    (32, 104, 144, 46)
assert FUSED_JOB.itemsize == 40
DELTA_JOB = np.dtype([("src_a", "<u8"), ("src_b", "<u8"), ("dst_off", "<u8"), ("base_off", "<u8"),
                      ("len_a", "<u4"), ("len_b", "<u4"), ("n", "<u4"), ("piece0", "<u4")])
assert DELTA_JOB.itemsize == 48


@dataclass
class Plan:
    payload: np.ndarray            # archive bytes [0, table_off): a view, never copied
    extras: np.ndarray             # host-inflated header chunks, placed right after the payload
    total: int                     # size of the output space
    scratch_bytes: int
    stream_jobs: np.ndarray
    seg_jobs: np.ndarray
    chunks: np.ndarray
    piece_chunk: np.ndarray
    piece_split: np.ndarray        # 6 boundaries: p1 cond, p1 plain, fused, p2 cond, p2 plain
    cond_jobs: np.ndarray
    cond_pieces: np.ndarray
    fused_jobs: np.ndarray = field(default=None)   # BF16 chunks, then 4-byte-element chunks
    n_fused_small: int = 0         # leading BF16 fused jobs with at most SMALL_LIVE live symbols
    n_fused_f32: int = 0           # trailing fused jobs that are 4-byte-element chunks
    n_fused_f32_small: int = 0     # the first of those, with at most SMALL_LIVE live symbols
    stream_owner: np.ndarray = field(default=None)   # record index of each stream job
    coded_bytes: int = 0           # sum of clen: algorithmic bytes read
    device_classify: bool = False  # the fused jobs are not sorted by alphabet: the library counts on the device
    n_fused_t: int = 0             # trailing fused jobs of shared-table chunks (padded per table to T_GROUP)
    delta_jobs: np.ndarray = field(default=None)   # chunks with both BF16 planes coded: decoded, merged, a delta undone
                                                   # and checksummed by one kernel; the first n_delta_plain have no base
    n_delta_plain: int = 0
    tables: np.ndarray = field(default=None)   # the shared tables, TABLE_STRIDE bytes apart

    @property
    def n_fused(self) -> int:
        """Fused jobs that carry their own table (BF16, then 4-byte elements)."""
        return int(self.fused_jobs.size) - self.n_fused_t
    base_bytes: int = 0            # bytes of delta bases read back

    @property
    def n_pieces(self) -> int:
        return int(self.piece_chunk.size)


def _gather(blob: np.ndarray, offs: np.ndarray, width: int) -> np.ndarray:
    return blob[offs[:, None] + np.arange(width, dtype=np.int64)[None, :]]


# Fewest 4-byte-element chunks worth the fused kernel: a launch that cannot fill the SMs'
# stream slots (148 x 76) is bound by each warp's own instruction stream, and there the
# two-pass path (lean stream kernel, then the merge kernel) measured faster.
FUSE_F32_MIN = 8192
SMALL_LIVE = 104       # largest alphabet the denser fused-kernel instance takes (csrc/fused_kernel.cuh)


def _alphabet_sizes(blob: np.ndarray, offs: np.ndarray) -> np.ndarray:
    """Live symbols (non-zero frequencies) of the rANS table at each stream offset."""
    from . import gpu
    offs = np.ascontiguousarray(offs, dtype=np.uint64)
    out = np.zeros(offs.size, dtype=np.uint16)
    lib = gpu.loaded_library()
    if lib is not None and blob.flags.c_contiguous and offs.size:
        rc = lib.lmz_host_alphabet_sizes(blob.ctypes.data, offs.ctypes.data, offs.size, out.ctypes.data)
        if rc == 0:
            return out
    cols = np.arange(0, 512, 2, dtype=np.int64)[None, :]
    for i in range(0, offs.size, 8192):                # the same count, without the library
        o = offs[i:i + 8192, None].astype(np.int64) + 4 + cols
        out[i:i + 8192] = ((blob[o] | blob[o + 1]) != 0).sum(1)
    return out


def _align16(x):
    return (x + 15) & ~15


def build_plan(ar: fmt.Archive, fuse=True, select=None, payload_range=None,
               out_range=None, classify: str = "device") -> Plan:
    """`fuse` routes BF16 chunks whose exponent plane is rANS and whose sign/mantissa
    plane is stored to the fused decode+merge+checksum kernel (no scratch plane),
    4-byte-element chunks whose top byte plane alone is coded likewise when there are
    at least FUSE_F32_MIN of them (`fuse="all"`: however few), and delta chunks whose
    difference is a BF16 chunk with both planes coded to the kernel instance that decodes
    both planes, undoes the delta against the base in the output space and checksums.
    `select` (record indices) plans only those chunks -- one rank's share of a
    partitioned decode, sources of its refs and deltas included by the caller.
    `payload_range` = (lo, hi) uploads only those archive bytes (every selected chunk's
    payload must lie inside); offsets in the plan are then relative to `lo`.
    `out_range` = (lo, hi) decodes into a buffer that holds only those bytes of the
    output space (every selected chunk, and the sources of selected refs and deltas,
    must lie inside); `Plan.total` is then hi - lo.
    `classify`: which side counts the live symbols of each fused stream's table to give
    small alphabets the denser kernel instance -- "device" (a kernel, after the upload; the
    host then never touches the payload's stream headers) or "host" (here, with numpy or
    the library's host helper)."""
    ar.check_coverage()
    r = ar.records if select is None else ar.records[np.asarray(select, dtype=np.int64)]
    lo, hi = (0, int(ar.table_off)) if payload_range is None else map(int, payload_range)
    blob = ar.blob[lo:]
    N = r.size
    codec = r["codec"].astype(np.int64)
    off = r["off"].astype(np.int64) - lo
    clen = r["clen"].astype(np.int64)
    if r.size and ((off < 0).any() or (off + clen > hi - lo).any()):
        raise FormatError("a selected chunk's payload lies outside the payload range")
    rlen = r["rlen"].astype(np.int64)
    out_lo, out_hi = (0, int(ar.total)) if out_range is None else map(int, out_range)
    dst = r["dst"].astype(np.int64) - out_lo
    if r.size and ((dst < 0).any() or (dst + rlen > out_hi - out_lo).any()):
        raise FormatError("a selected chunk lies outside the output range")
    flags = r["flags"].astype(np.int64)
    esize = r["esize"].astype(np.int64)

    # ---- refs and deltas: unwrap to the inner codec, remember the source ----------
    is_delta, is_ref = codec == fmt.CODEC_DELTA, codec == fmt.CODEC_REF
    base = np.full(N, -1, dtype=np.int64)
    ref_src = np.full(N, -1, dtype=np.int64)
    ecodec, eoff, eclen = codec.copy(), off.copy(), clen.copy()
    di = np.nonzero(is_delta)[0]
    if di.size:
        if (clen[di] < 9).any():
            raise CorruptArchive("delta chunk is truncated")           # lmz/codec.py:1036
        h = _gather(blob, off[di], 9)
        base[di] = np.ascontiguousarray(h[:, :8]).view("<u8")[:, 0].astype(np.int64) - out_lo
        inner = h[:, 8].astype(np.int64)
        if np.isin(inner, (fmt.CODEC_REF, fmt.CODEC_DELTA)).any():
            raise CorruptArchive("delta chunk names a ref or delta for its own difference")
        ecodec[di], eoff[di], eclen[di] = inner, off[di] + 9, clen[di] - 9
    ri = np.nonzero(is_ref)[0]
    if ri.size:
        if (clen[ri] != 8).any():
            raise CorruptArchive("ref chunk payload must be 8 bytes")  # lmz/api.py:873
        ref_src[ri] = np.ascontiguousarray(_gather(blob, off[ri], 8)).view("<u8")[:, 0].astype(np.int64) - out_lo
    pass2 = is_delta | is_ref
    src = np.where(is_ref, ref_src, base)
    si = np.nonzero(pass2)[0]
    if si.size:
        s, e = src[si], src[si] + rlen[si]
        if (s < 0).any() or (e > out_hi - out_lo).any():
            raise CorruptArchive("a ref or delta source lies outside the output")
        o2 = si[np.argsort(dst[si], kind="stable")]
        d2, e2 = dst[o2], dst[o2] + rlen[o2]
        hits = np.searchsorted(d2, e, "left") - np.searchsorted(e2, s, "right")
        if (hits[rlen[si] > 0] > 0).any():
            raise CorruptArchive("a ref or delta chunk points at another one")   # lmz/api.py:851

    kind = np.zeros(N, dtype=np.uint8)
    plane_off = np.zeros((N, 8), dtype=np.uint64)
    scratch_mask = np.zeros(N, dtype=np.uint8)
    src_is_out = np.zeros(N, dtype=np.uint8)
    extras, extra_pos = [], hi - lo
    # stream jobs, collected as columns; dst assigned once all are known
    sj_src, sj_len, sj_n, sj_owner, sj_plane = [], [], [], [], []

    def add_streams(src_off, src_len, n, owner, plane):
        sj_src.append(src_off); sj_len.append(src_len); sj_n.append(n)
        sj_owner.append(owner); sj_plane.append(np.broadcast_to(plane, owner.shape))

    known = np.zeros(N, dtype=bool)
    fused = np.zeros(N, dtype=bool)
    f_src = np.zeros(N, dtype=np.int64)
    f_len = np.zeros(N, dtype=np.int64)
    f_mant = np.zeros(N, dtype=np.int64)
    fused_d = np.zeros(N, dtype=bool)               # delta chunks for the two-plane instance
    f_len_b = np.zeros(N, dtype=np.int64)

    # stored, and refs (a copy out of the output space)
    i = np.nonzero((ecodec == fmt.CODEC_STORED) & ~is_ref)[0]
    if (eclen[i] != rlen[i]).any():
        raise CorruptArchive("stored chunk length differs from its record")
    plane_off[i, 0] = eoff[i]
    known[i] = True
    plane_off[ri, 0] = ref_src[ri]
    src_is_out[ri] = 1
    known[ri] = True

    # one coded stream (header chunks, esize-1 data)
    i = np.nonzero((ecodec == fmt.CODEC_ZSTD) & ~is_ref)[0]
    if i.size:
        m = flags[i] & 3
        st = i[m == fmt.METHOD_STORED]
        if (eclen[st] != rlen[st]).any():
            raise CorruptArchive("stored chunk length differs from its record")
        plane_off[st, 0] = eoff[st]
        ra = i[m == fmt.METHOD_RANS]
        add_streams(eoff[ra], eclen[ra], rlen[ra], ra, 0)
        scratch_mask[ra] = 1
        for j in i[(m == fmt.METHOD_ZSTD) | (m == fmt.METHOD_DEFLATE)]:
            # General-purpose streams are tiny container headers; they are inflated
            # here and travel to the device as stored bytes.
            raw = blob[eoff[j]:eoff[j] + eclen[j]].tobytes()
            data = fmt.inflate_tail(raw) if (flags[j] & 3) == fmt.METHOD_ZSTD else _inflate(raw)
            if len(data) != rlen[j]:
                raise CorruptArchive(f"chunk decoded to {len(data)} bytes, expected {rlen[j]}")
            plane_off[j, 0] = extra_pos
            extras.append(np.frombuffer(data, dtype=np.uint8))
            extra_pos += len(data)
        known[i] = True

    # byte-plane and BF16 field splits (lmz/codec.py:1176-1223, lmzcore.c:1553-1598)
    for cid in (fmt.CODEC_SPLIT, fmt.CODEC_BF16):
        sel = (ecodec == cid) & ~is_ref
        if not sel.any():
            continue
        if cid == fmt.CODEC_BF16 and (esize[sel] != 2).any():
            raise CorruptArchive("a bf16 chunk must have 2-byte elements")
        if (~np.isin(esize[sel], (2, 4, 8))).any() or (rlen[sel] % esize[sel]).any():
            raise CorruptArchive("split chunk has an invalid element size")
        kind[sel] = K_BF16 if cid == fmt.CODEC_BF16 else K_SPLIT
        for npl in (2, 4, 8):
            i = np.nonzero(sel & (esize == npl))[0]
            if not i.size:
                continue
            if (eclen[i] < 4 * npl).any():
                raise CorruptArchive("split chunk is truncated")
            lens = np.ascontiguousarray(_gather(blob, eoff[i], 4 * npl)).view("<u4").astype(np.int64)
            meth = (flags[i][:, None] >> (2 * np.arange(npl))[None, :]) & 3
            nelem = rlen[i] // npl
            starts = eoff[i][:, None] + 4 * npl + np.cumsum(lens, axis=1) - lens
            if (4 * npl + lens.sum(axis=1) > eclen[i]).any():
                raise CorruptArchive("split chunk is truncated")
            if (~np.isin(meth, (fmt.METHOD_STORED, fmt.METHOD_RANS))).any():
                raise FormatError("a plane is coded with a general-purpose compressor; "
                                  "the GPU path decodes stored and rANS planes only")
            stored = meth == fmt.METHOD_STORED
            if (stored & (lens != nelem[:, None])).any():
                raise CorruptArchive("a stored plane's length differs from the element count")
            plane_off[i[:, None], np.arange(npl)[None, :]] = starts
            if fuse and cid == fmt.CODEC_BF16:
                fz = ~pass2[i] & ~stored[:, 0] & stored[:, 1] & (nelem > 0)
                fi = i[fz]
                fused[fi] = True
                f_src[fi], f_len[fi], f_mant[fi] = starts[fz, 0], lens[fz, 0], starts[fz, 1]
                stored = stored | fz[:, None]          # no scratch stream for these
                # both planes coded: a delta's difference (mostly zero bytes, so both pay), or a plain
                # chunk whose sign/mantissa bytes compress; the same kernel, with or without a base
                dz = ~is_ref[i] & ~stored[:, 0] & ~stored[:, 1] & (nelem > 0)
                di2 = i[dz]
                fused_d[di2] = True
                f_src[di2], f_len[di2] = starts[dz, 0], lens[dz, 0]
                f_mant[di2], f_len_b[di2] = starts[dz, 1], lens[dz, 1]
                stored = stored | dz[:, None]
            if fuse and cid == fmt.CODEC_SPLIT and npl == 4:
                # top byte plane coded, the three lower planes stored (and then back to back)
                fz = ~pass2[i] & ~stored[:, 3] & stored[:, :3].all(axis=1) & (nelem > 0)
                if fuse != "all" and int(fz.sum()) < FUSE_F32_MIN:
                    fz[:] = False
                fi = i[fz]
                fused[fi] = True
                f_src[fi], f_len[fi], f_mant[fi] = starts[fz, 3], lens[fz, 3], starts[fz, 0]
                stored = stored | fz[:, None]
            rr, pp = np.nonzero(~stored)
            add_streams(starts[rr, pp], lens[rr, pp], nelem[rr], i[rr], pp)
            np.bitwise_or.at(scratch_mask, i[rr], (1 << pp).astype(np.uint8))
            known[i] = True

    # BF16 against a shared table (this repository's format option, archive.CODEC_BF16T)
    is_t = np.zeros(N, dtype=bool)
    table_of = np.zeros(N, dtype=np.int64)
    tables = np.zeros((0, TABLE_STRIDE), dtype=np.uint8)
    ti = np.nonzero((ecodec == fmt.CODEC_BF16T) & ~is_ref)[0]
    if ti.size:
        if pass2[ti].any():
            raise FormatError("a delta whose difference is shared-table coded is not something any writer produces")
        if (esize[ti] != 2).any() or (rlen[ti] % 2).any() or (eclen[ti] < 16).any():
            raise CorruptArchive("a shared-table bf16 chunk is malformed")
        h = np.ascontiguousarray(_gather(blob, eoff[ti], 16)).view(BF16T_HDR)[:, 0]
        len0, len1 = h["len0"].astype(np.int64), h["len1"].astype(np.int64)
        nelem = rlen[ti] // 2
        if (16 + len0 + len1 > eclen[ti]).any() or (len1 != nelem).any():
            raise CorruptArchive("a shared-table bf16 chunk has inconsistent plane lengths")
        toff = h["table"].astype(np.int64)
        if (h["table"] < fmt.HEADER.size).any() or (h["table"] > np.uint64(int(ar.table_off) - fmt.TABLE_BYTES)).any():
            raise CorruptArchive("a shared-table bf16 chunk names a table outside the payload region")
        uniq, inv = np.unique(toff, return_inverse=True)
        tables = np.zeros((uniq.size, TABLE_STRIDE), dtype=np.uint8)
        tables[:, :fmt.TABLE_BYTES] = _gather(ar.blob, uniq, fmt.TABLE_BYTES)      # read from the file itself: a
        table_of[ti] = inv                                                         # table may lie outside this plan's payload range
        kind[ti] = K_BF16
        plane_off[ti, 0], plane_off[ti, 1] = eoff[ti] + 16, eoff[ti] + 16 + len0
        nz = nelem > 0
        fused[ti[nz]] = is_t[ti[nz]] = True
        f_src[ti], f_len[ti], f_mant[ti] = eoff[ti] + 16, len0, eoff[ti] + 16 + len0
        if (~nz).any():
            raise CorruptArchive("a shared-table bf16 chunk is empty")
        known[ti] = True

    # exponent-conditioned BF16 (lmz/codec.py:1075-1146)
    ci = np.nonzero((ecodec == fmt.CODEC_BF16C) & ~is_ref)[0]
    cond = np.zeros(ci.size, dtype=COND_JOB)
    seg_rans_total = np.zeros(ci.size, dtype=np.int64)
    if ci.size:
        if (esize[ci] != 2).any() or (rlen[ci] % 2).any():
            raise CorruptArchive("a conditioned bf16 chunk must have 2-byte elements")
        if (eclen[ci] < 46).any():
            raise CorruptArchive("conditioned bf16 chunk is truncated")
        h = np.ascontiguousarray(_gather(blob, eoff[ci], 46)).view(BF16C_HDR)[:, 0]
        if (h["k"] != 8).any():
            raise CorruptArchive("conditioned bf16 chunk does not declare 8 buckets")
        nelem = rlen[ci] // 2
        exp_len = h["exp_len"].astype(np.int64)
        seg_len = h["seg_len"].astype(np.int64)
        if (46 + exp_len + seg_len.sum(axis=1) > eclen[ci]).any():
            raise CorruptArchive("conditioned bf16 chunk is truncated")
        meths = np.concatenate((h["exp_m"][:, None], h["sm_m"]), axis=1)
        if (meths > 3).any():
            raise CorruptArchive("conditioned bf16 chunk names an unknown method")
        live = np.concatenate((np.ones((ci.size, 1), bool), seg_len > 0), axis=1)
        if (live & ~np.isin(meths, (fmt.METHOD_STORED, fmt.METHOD_RANS))).any():
            raise FormatError("a conditioned plane is coded with a general-purpose compressor")
        exp_src = eoff[ci] + 46
        st = h["exp_m"] == fmt.METHOD_STORED
        if (st & (exp_len != nelem)).any():
            raise CorruptArchive("stored exponent plane has the wrong length")
        cond["exp_off"] = exp_src
        cond["exp_in_scratch"] = (~st).astype(np.uint8)
        ce = np.nonzero(~st)[0]
        add_streams(exp_src[ce], exp_len[ce], nelem[ce], ci[ce], -1)
        cond["seg_src"] = (exp_src + exp_len)[:, None] + np.cumsum(seg_len, axis=1) - seg_len
        cond["seg_len"] = seg_len
        cond["seg_method"] = h["sm_m"]
        cond["nelem"] = nelem
        seg_rans_total = nelem - np.where(h["sm_m"] == fmt.METHOD_STORED, seg_len, 0).sum(axis=1)
        if (seg_rans_total < 0).any():
            raise CorruptArchive("stored buckets hold more bytes than the chunk has elements")
        kind[ci] = K_COND
        known[ci] = True

    if not known.all():
        bad = int(ecodec[np.nonzero(~known)[0][0]])
        raise FormatError(f"codec {bad} is outside the decode path this library covers")

    # ---- scratch: decoded planes, then decoded segments --------------------------
    if sj_src:
        s_src = np.concatenate(sj_src).astype(np.int64)
        s_len = np.concatenate(sj_len).astype(np.int64)
        s_n = np.concatenate(sj_n).astype(np.int64)
        s_owner = np.concatenate(sj_owner).astype(np.int64)
        s_plane = np.concatenate(sj_plane).astype(np.int64)
    else:
        s_src = s_len = s_n = s_owner = s_plane = np.zeros(0, dtype=np.int64)
    sizes = _align16(s_n)
    s_dst = np.cumsum(sizes) - sizes
    scratch_pos = int(sizes.sum())
    pl = s_plane >= 0
    plane_off[s_owner[pl], s_plane[pl]] = s_dst[pl]
    if ci.size:
        cond_of = np.full(N, -1, dtype=np.int64)
        cond_of[ci] = np.arange(ci.size)
        ex = ~pl
        cond["exp_off"][cond_of[s_owner[ex]]] = s_dst[ex]
        seg_sizes = _align16(seg_rans_total)
        cond["seg_scratch"] = scratch_pos + np.cumsum(seg_sizes) - seg_sizes
        scratch_pos += int(seg_sizes.sum())
        is_job = (cond["seg_method"] == fmt.METHOD_RANS) & (cond["seg_len"] > 0)
        per = is_job.sum(axis=1)
        cond["seg_job0"] = np.cumsum(per) - per
    order = np.argsort(-s_n, kind="stable")         # long streams first
    stream_jobs = np.zeros(s_n.size, dtype=STREAM_JOB)
    stream_jobs["src_off"], stream_jobs["dst_off"] = s_src[order], s_dst[order]
    stream_jobs["src_len"], stream_jobs["n"] = s_len[order], s_n[order]
    if ci.size:
        seg_jobs = np.zeros(int(is_job.sum()), dtype=STREAM_JOB)
        seg_jobs["src_off"] = cond["seg_src"][is_job]        # row-major: chunk, then bucket
        seg_jobs["src_len"] = cond["seg_len"][is_job]
    else:
        seg_jobs = np.zeros(0, dtype=STREAM_JOB)

    # ---- chunk jobs in launch order ----------------------------------------------
    group = np.where(pass2, 3, 0) + (kind != K_COND) + (fused & ~pass2)
    group[fused_d] = 2                              # written by their own kernel, like the fused chunks
    corder = np.argsort(group, kind="stable")
    chunks = np.zeros(N, dtype=CHUNK_JOB)
    chunks["dst_off"] = dst[corder]
    chunks["base_off"] = np.where(base[corder] >= 0, base[corder].astype(np.uint64), NONE64)
    chunks["plane_off"] = plane_off[corder]
    chunks["rlen"], chunks["crc"] = rlen[corder], r["crc"][corder]
    chunks["kind"], chunks["esize"] = kind[corder], esize[corder]
    chunks["scratch_mask"], chunks["src_is_out"] = scratch_mask[corder], src_is_out[corder]
    chunks["record"] = corder
    npieces = (rlen[corder] + PIECE - 1) // PIECE
    piece0 = np.cumsum(npieces) - npieces
    chunks["piece0"] = piece0
    piece_chunk = np.repeat(np.arange(N, dtype=np.uint32), npieces)
    g = group[corder]
    split = np.array([0] + [int(npieces[g <= k].sum()) for k in range(5)], dtype=np.uint32)
    if ci.size:
        pos_of = np.empty(N, dtype=np.int64)
        pos_of[corder] = np.arange(N)
        cond["chunk"] = pos_of[ci]
        cond["piece0"] = piece0[pos_of[ci]]
        chunks["aux"][pos_of[ci]] = np.arange(ci.size)
    cond_pieces = np.nonzero(chunks["kind"][piece_chunk] == K_COND)[0].astype(np.uint32)
    fall = np.nonzero(g == 2)[0]
    tpos = fall[is_t[corder[fall]]]                 # shared-table chunks: jobs of their own, below
    dpos = fall[fused_d[corder[fall]]]              # two-plane delta chunks: jobs of their own, too
    fpos = fall[~is_t[corder[fall]] & ~fused_d[corder[fall]]]      # fused chunks, in launch order ...
    whole = f_len[corder[fpos]] >= 548              # table + states present (else the kernel rejects it)
    small = np.zeros(fpos.size, dtype=bool)
    if classify == "host":
        small[whole] = _alphabet_sizes(blob, f_src[corder[fpos]][whole]) <= SMALL_LIVE
    wide4 = esize[corder[fpos]] == 4                # ... BF16 before 4-byte elements,
    fpos = np.concatenate([fpos[~wide4 & small], fpos[~wide4 & ~small],     # small alphabets first
                           fpos[wide4 & small], fpos[wide4 & ~small]])
    fused_jobs = np.zeros(fpos.size, dtype=FUSED_JOB)
    frec = corder[fpos]
    fused_jobs["src_off"], fused_jobs["src_len"] = f_src[frec], f_len[frec]
    fused_jobs["mant_off"], fused_jobs["dst_off"] = f_mant[frec], dst[frec]
    fused_jobs["n"], fused_jobs["piece0"] = rlen[frec] // esize[frec], piece0[fpos]
    n_fused_t = 0
    if tpos.size:
        # table by table, each table's run padded with empty jobs to whole thread blocks
        tid = table_of[corder[tpos]]
        o = np.argsort(tid, kind="stable")
        tpos, tid = tpos[o], tid[o]
        per = np.bincount(tid, minlength=tables.shape[0])
        padded = -(-per // T_GROUP) * T_GROUP
        n_fused_t = int(padded.sum())
        first = np.cumsum(padded) - padded
        slot = first[tid] + (np.arange(tpos.size) - (np.cumsum(per) - per)[tid])
        tj = np.zeros(n_fused_t, dtype=FUSED_JOB)
        tj["flags"] = np.repeat(np.arange(tables.shape[0]), padded)
        trec = corder[tpos]
        tj["src_off"][slot], tj["src_len"][slot] = f_src[trec], f_len[trec]
        tj["mant_off"][slot], tj["dst_off"][slot] = f_mant[trec], dst[trec]
        tj["n"][slot], tj["piece0"][slot] = rlen[trec] // 2, piece0[tpos]
        fused_jobs = np.concatenate((fused_jobs, tj))

    dpos = np.concatenate([dpos[~pass2[corder[dpos]]], dpos[pass2[corder[dpos]]]])   # plain chunks first: the first pass
    n_delta_plain = int((~pass2[corder[dpos]]).sum())
    delta_jobs = np.zeros(dpos.size, dtype=DELTA_JOB)
    drec = corder[dpos]
    delta_jobs["src_a"], delta_jobs["len_a"] = f_src[drec], f_len[drec]
    delta_jobs["src_b"], delta_jobs["len_b"] = f_mant[drec], f_len_b[drec]
    delta_jobs["dst_off"] = dst[drec]
    delta_jobs["base_off"] = np.where(base[drec] >= 0, base[drec].astype(np.uint64), NONE64)
    delta_jobs["n"], delta_jobs["piece0"] = rlen[drec] // 2, piece0[dpos]

    payload = blob[:hi - lo]
    extra = np.concatenate(extras) if extras else np.zeros(0, dtype=np.uint8)
    return Plan(payload=payload, extras=extra, total=out_hi - out_lo, scratch_bytes=scratch_pos + 64,
                stream_jobs=stream_jobs, seg_jobs=seg_jobs, chunks=chunks,
                piece_chunk=piece_chunk, piece_split=split, cond_jobs=cond,
                cond_pieces=cond_pieces, stream_owner=s_owner[order], fused_jobs=fused_jobs,
                n_fused_small=int((~wide4 & small).sum()), n_fused_f32=int(wide4.sum()),
                n_fused_f32_small=int((wide4 & small).sum()),
                coded_bytes=int(clen.sum()), base_bytes=int(rlen[is_delta].sum()),
                device_classify=classify != "host", n_fused_t=n_fused_t, tables=tables,
                delta_jobs=delta_jobs, n_delta_plain=n_delta_plain)


def _inflate(raw: bytes) -> bytes:
    try:
        return zlib.decompress(raw)
    except zlib.error as exc:
        raise CorruptArchive(f"chunk failed to decode: {exc}") from exc
