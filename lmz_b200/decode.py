"""Whole-archive decode on one GPU.

The reference decodes an archive on CPU threads (lmz/api.py:889-975
`decompress`, :1061-1143 `verify`); this is the same job on the device: the
archive's payload is uploaded once, `ArchiveDecoder.run()` decodes every chunk
into one device buffer laid out like the reference's concatenated output space
(members end to end, lmz/format.py:17-19), and per-chunk crc32 verdicts come
back with it.  PyTorch only owns the device buffers and the stream.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _chunks, archive as fmt, gpu, plan as planner
from .archive import CorruptArchive

_ST_NAMES = {1: "bad stream header", 2: "truncated stream", 3: "input copy timed out",
             4: "lengths disagree with the record", 5: "checksum mismatch"}

_TORCH_DTYPES = {"BF16": "bfloat16", "F16": "float16", "F32": "float32", "F64": "float64",
                 "I8": "int8", "U8": "uint8", "I16": "int16", "I32": "int32", "I64": "int64",
                 "BOOL": "bool"}


def _dev(arr: np.ndarray, device):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1).copy())
    return t.to(device, non_blocking=False)


_tables = {}


def _crc_tables(lib, device):
    """The CRC tables, uploaded once per device."""
    import torch
    key = str(device)
    if key not in _tables:
        n = lib.lmz_gpu_crc_tables(None, 0)
        host = np.zeros(n, dtype=np.uint8)
        lib.lmz_gpu_crc_tables(host.ctypes.data, n)
        _tables[key] = torch.from_numpy(host).to(device)
    return _tables[key]


class ArchiveDecoder:
    """An archive planned and resident on `device`, ready to decode repeatedly.

    `ar` is an `archive.Archive`, a path, or the archive's bytes.  With
    `checksum=False` the per-chunk crc32 is skipped (the reference's
    `verify_checksums=False`).  `payload` may be given as a CUDA uint8 tensor with room
    for `plan.payload`, the plan's host-inflated header chunks and `gpu.pad_bytes()` of
    slack; the caller then brings the payload bytes there itself (`upload`, or copies of
    its own) before `run`."""

    def __init__(self, ar, device=None, checksum: bool = True, out=None, plan=None,
                 fuse=True, payload=None):
        import torch

        lib = gpu.library()
        self.lib = lib
        sizes = (ctypes.c_uint * 5)()
        lib.lmz_gpu_struct_sizes(ctypes.byref(sizes))
        want = (planner.STREAM_JOB.itemsize, planner.CHUNK_JOB.itemsize,
                planner.COND_JOB.itemsize, planner.COND_STATE_BYTES, planner.FUSED_JOB.itemsize)
        if tuple(sizes) != want or lib.lmz_gpu_piece_bytes() != planner.PIECE or \
                lib.lmz_gpu_shared_group() != planner.T_GROUP or \
                lib.lmz_gpu_delta_job_bytes() != planner.DELTA_JOB.itemsize:
            raise RuntimeError("the CUDA library and the planner disagree on job layouts")
        self.archive = ar if isinstance(ar, fmt.Archive) else fmt.Archive(ar)
        self.plan = p = plan if plan is not None else planner.build_plan(self.archive, fuse=fuse)
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        self.checksum = checksum
        d = self.device
        with torch.cuda.device(d):
            pad = gpu.pad_bytes()
            nbytes = p.payload.size + p.extras.size
            if payload is not None and payload.numel() < nbytes + pad:
                raise ValueError("the payload buffer is smaller than the plan's payload, header chunks and slack")
            self.d_payload = payload if payload is not None else \
                torch.empty(nbytes + pad, dtype=torch.uint8, device=d)
            self.h2d_bytes = int(nbytes)
            self.d_payload[nbytes:].zero_()
            if p.extras.size:
                self.d_payload[p.payload.size:nbytes].copy_(torch.from_numpy(p.extras.copy()))
            if payload is None:
                self.upload()
            self.d_scratch = torch.empty(max(p.scratch_bytes, 64), dtype=torch.uint8, device=d)
            self.d_out = out if out is not None else \
                torch.empty(p.total + 64, dtype=torch.uint8, device=d)
            if self.d_out.numel() < p.total + 64:
                raise ValueError("the output buffer needs total + 64 bytes")
            self.d_stream_jobs = _dev(p.stream_jobs, d)
            self.d_seg_jobs = _dev(p.seg_jobs, d)
            self.d_fused_jobs = _dev(p.fused_jobs, d)
            self.d_delta_jobs = _dev(p.delta_jobs, d)
            self.d_chunks = _dev(p.chunks, d)
            self.d_piece_chunk = _dev(p.piece_chunk, d)
            self.d_cond_jobs = _dev(p.cond_jobs, d)
            self.d_cond_pieces = _dev(p.cond_pieces, d)
            ncond = p.cond_jobs.size
            u32 = dict(dtype=torch.int32, device=d)
            self.d_cond_state = torch.zeros(max(1, ncond * planner.COND_STATE_BYTES),
                                            dtype=torch.uint8, device=d)
            self.d_hist = torch.zeros(max(1, ncond * 256), **u32)
            self.d_piece_cnt = torch.zeros(max(1, p.n_pieces * 16), **u32)
            self.d_piece_wcnt = torch.zeros(max(1, p.n_pieces * 64 if ncond else 1), dtype=torch.int16, device=d)
            self.d_piece_lcnt = torch.empty(max(1, p.cond_pieces.size * 2048), **u32)
            self.d_piece_crc = torch.zeros(max(1, p.n_pieces), **u32)
            self.d_stream_status = torch.zeros(max(1, p.stream_jobs.size), **u32)
            self.d_seg_status = torch.zeros(max(1, p.seg_jobs.size), **u32)
            self.d_fused_status = torch.zeros(max(1, p.fused_jobs.size), **u32)
            self.d_delta_status = torch.zeros(max(1, 2 * p.delta_jobs.size), **u32)
            self.d_delta_order = torch.zeros(p.delta_jobs.size + 4, **u32)
            self.d_chunk_status = torch.zeros(max(1, p.chunks.size), **u32)
            self.d_chunk_crc = torch.zeros(max(1, p.chunks.size), **u32)
            self.d_any_bad = torch.zeros(1, **u32)
            self.d_fused_order = torch.zeros(p.n_fused + 4, **u32) if p.device_classify else None
            self.d_tables = _dev(p.tables, d) if p.n_fused_t else None
            self.d_tabs = _crc_tables(lib, d)
        c = _chunks.DecodePlan()
        c.d_payload, c.d_scratch = self.d_payload.data_ptr(), self.d_scratch.data_ptr()
        c.d_out = self.d_out.data_ptr()
        c.d_stream_jobs, c.d_seg_jobs = self.d_stream_jobs.data_ptr(), self.d_seg_jobs.data_ptr()
        c.d_stream_status, c.d_seg_status = self.d_stream_status.data_ptr(), self.d_seg_status.data_ptr()
        c.d_fused_jobs, c.d_fused_status = self.d_fused_jobs.data_ptr(), self.d_fused_status.data_ptr()
        c.n_fused, c.n_fused_t = p.n_fused, p.n_fused_t
        c.d_delta_jobs, c.d_delta_status = self.d_delta_jobs.data_ptr(), self.d_delta_status.data_ptr()
        c.n_delta, c.n_delta_plain = p.delta_jobs.size, p.n_delta_plain
        c.d_delta_order = self.d_delta_order.data_ptr()
        c.d_tables = self.d_tables.data_ptr() if self.d_tables is not None else None
        c.n_fused_small = p.n_fused_small
        c.n_fused_f32, c.n_fused_f32_small = p.n_fused_f32, p.n_fused_f32_small
        c.d_chunks, c.d_piece_chunk = self.d_chunks.data_ptr(), self.d_piece_chunk.data_ptr()
        c.d_cond_jobs, c.d_cond_state = self.d_cond_jobs.data_ptr(), self.d_cond_state.data_ptr()
        c.d_cond_pieces = self.d_cond_pieces.data_ptr()
        c.d_hist, c.d_piece_cnt = self.d_hist.data_ptr(), self.d_piece_cnt.data_ptr()
        c.d_piece_wcnt = self.d_piece_wcnt.data_ptr()
        c.d_piece_lcnt = self.d_piece_lcnt.data_ptr()
        c.d_piece_crc = self.d_piece_crc.data_ptr() if checksum else None
        c.d_crc_tables = self.d_tabs.data_ptr()
        c.d_chunk_status, c.d_chunk_crc = self.d_chunk_status.data_ptr(), self.d_chunk_crc.data_ptr()
        c.d_any_bad = self.d_any_bad.data_ptr()
        c.d_fused_order = self.d_fused_order.data_ptr() if self.d_fused_order is not None else None
        c.n_stream_jobs, c.n_seg_jobs = p.stream_jobs.size, p.seg_jobs.size
        c.n_chunks, c.n_pieces = p.chunks.size, p.n_pieces
        c.n_cond, c.n_cond_pieces = ncond, p.cond_pieces.size
        for i in range(6):
            c.piece_split[i] = int(p.piece_split[i])
        self._c = c
        # kernels launched by one run(): stream decode; histogram, bucket map, counting, running
        # totals and the segment decode of conditioned chunks; up to four finish launches; the
        # verdict kernel
        nbf = p.n_fused - p.n_fused_f32
        if p.device_classify:                # per group: the count kernel and both instances
            fused_launches = 3 * ((1 if nbf else 0) + (1 if p.n_fused_f32 else 0))
        else:
            fused_launches = (1 if p.n_fused_small else 0) + (1 if nbf > p.n_fused_small else 0) + \
                (1 if p.n_fused_f32_small else 0) + (1 if p.n_fused_f32 > p.n_fused_f32_small else 0)
        fused_launches += (1 if p.n_fused_t else 0) + (3 if p.n_delta_plain else 0) + \
            (3 if p.delta_jobs.size > p.n_delta_plain else 0)
        self.launches_per_run = (1 if p.stream_jobs.size else 0) + \
            ((4 + (1 if p.seg_jobs.size else 0)) if ncond else 0) + fused_launches + \
            int(sum(p.piece_split[i + 1] > p.piece_split[i] for i in (0, 1, 3, 4))) + 1

    def upload(self, pinned=None, non_blocking: bool = False):
        """Copy the archive's payload region host -> device (from `pinned`, a host
        uint8 tensor of `plan.payload.size` bytes, if given)."""
        import warnings

        import torch
        if pinned is None:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")          # read-only numpy views are fine to read
                pinned = torch.from_numpy(self.plan.payload)
        self.d_payload[:self.plan.payload.size].copy_(pinned, non_blocking=non_blocking)

    def run(self, stream=None, phases: int = 0):
        """Launch the decode on `stream` (default: torch's current). Asynchronous.
        `phases` restricts the launch sequence (bit 0 stream decode, 1 conditioned-chunk
        kernels, 2 finish, 3 verdicts, 4 fused BF16 chunks) so one phase can be timed
        alone; 0 runs all."""
        import torch
        self._c.phases = phases
        with torch.cuda.device(self.device):
            s = stream if stream is not None else torch.cuda.current_stream(self.device)
            rc = self.lib.lmz_gpu_decode_chunks_dev(ctypes.byref(self._c), s.cuda_stream)
        if rc != gpu.OK:
            raise RuntimeError(f"decode launch failed ({rc}): {gpu.last_error()}")
        return self.output

    @property
    def output(self):
        """The decoded output space (device uint8 tensor of `total` bytes)."""
        return self.d_out[:self.plan.total]

    def check(self) -> None:
        """Synchronise and raise CorruptArchive if any stream or chunk failed."""
        import torch
        torch.cuda.synchronize(self.device)
        if int(self.d_any_bad.item()) == 0:
            return
        p = self.plan
        st = self.d_chunk_status.cpu().numpy()[:p.chunks.size]
        bad = np.nonzero(st)[0]
        if bad.size:
            rec = int(p.chunks["record"][bad[0]])
            raise CorruptArchive(f"chunk {rec} ({bad.size} in all): "
                                 f"{_ST_NAMES.get(int(st[bad[0]]), st[bad[0]])}")
        ss = self.d_stream_status.cpu().numpy()[:p.stream_jobs.size]
        hard = np.nonzero((ss != 0) & (ss != 0x100))[0]
        if hard.size:
            rec = int(p.stream_owner[hard[0]])
            raise CorruptArchive(f"a plane of chunk {rec}: {_ST_NAMES.get(int(ss[hard[0]]), '?')}")
        fs = self.d_fused_status.cpu().numpy()[:p.fused_jobs.size]
        hard = np.nonzero((fs != 0) & (fs != 0x100))[0]
        if hard.size:
            raise CorruptArchive(f"the exponent plane of a bf16 chunk: "
                                 f"{_ST_NAMES.get(int(fs[hard[0]]), '?')}")
        ds = self.d_delta_status.cpu().numpy()[:2 * p.delta_jobs.size]
        hard = np.nonzero((ds != 0) & (ds != 0x100))[0]
        if hard.size:
            raise CorruptArchive(f"a plane of a delta chunk's difference: {_ST_NAMES.get(int(ds[hard[0]]), '?')}")
        raise CorruptArchive("a bucket segment of a conditioned chunk failed to decode")

    def chunk_crcs(self) -> np.ndarray:
        """crc32 of every decoded chunk, in archive record order."""
        p = self.plan
        crc = self.d_chunk_crc.cpu().numpy().view(np.uint32)[:p.chunks.size]
        out = np.zeros(p.chunks.size, dtype=np.uint32)
        out[p.chunks["record"]] = crc
        return out

    def tensors(self):
        """{(member path, tensor name): device tensor view} for safetensors members,
        typed and shaped from the manifest; views into the output buffer."""
        import torch
        out = {}
        for key, (dt, shape, s, e) in self.archive.tensor_index().items():
            name = _TORCH_DTYPES.get(dt)
            raw = self.d_out[s:e]
            if name is None or s % 2:
                out[key] = raw
                continue
            try:
                out[key] = raw.view(getattr(torch, name)).reshape(shape)
            except RuntimeError:
                out[key] = raw
        return out


class PipelinedDecoder:
    """Host-to-HBM decode with the upload overlapped: the archive's chunks are cut
    into `nslices` runs of consecutive payload bytes, each with its own plan, and
    slice i decodes on the compute stream while slice i+1 is still crossing PCIe on
    the copy stream.  All slices write into one output buffer.  Archives with refs
    or deltas (which read other chunks' output) use a single slice.

    `nslices=None` chooses: 8 for archives of small chunks; for chunks of a megabyte or
    more, whose decode time is the latency of one long stream whatever their number,
    one slice per ~1900 such chunks (a slice of fewer costs as much as a full one)."""

    def __init__(self, ar, nslices=None, device=None, checksum: bool = True):
        import torch
        self.archive = ar if isinstance(ar, fmt.Archive) else fmt.Archive(ar)
        r = self.archive.records
        groups = _slice_groups(self.archive, nslices)
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        out = torch.empty(self.archive.total + 64, dtype=torch.uint8, device=self.device)
        self.slices, self.ranges = [], []
        for g in groups:
            lo = int(r["off"][g].min())
            hi = int((r["off"][g].astype(np.int64) + r["clen"][g]).max())
            p = planner.build_plan(self.archive, select=g, payload_range=(lo, hi))
            self.slices.append(ArchiveDecoder(self.archive, device=self.device, checksum=checksum,
                                              out=out, plan=p))
            self.ranges.append((lo, hi))
        self.d_out = out
        self.copy_stream = torch.cuda.Stream(self.device)
        self.h2d_bytes = sum(hi - lo for lo, hi in self.ranges)
        self.launches_per_run = sum(s.launches_per_run for s in self.slices)

    def run_from_host(self, pinned, stream=None):
        """`pinned`: a pinned uint8 host tensor over the archive's bytes (offset 0 =
        file start).  Uploads and decodes slice by slice; asynchronous."""
        import torch
        compute = stream if stream is not None else torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(compute)
        for dec, (lo, hi) in zip(self.slices, self.ranges):
            with torch.cuda.stream(self.copy_stream):
                dec.upload(pinned[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
            compute.wait_event(ev)
            dec.run(stream=compute)
        return self.d_out[:self.archive.total]

    def run_from_file(self, stream=None, staging=None):
        """The same from the archive's own bytes wherever they are (a mapped file, the page
        cache, ordinary memory): see `load_archive`, which also plans under the copies."""
        import torch
        compute = stream if stream is not None else torch.cuda.current_stream(self.device)
        up = _Uploader(self.archive.blob, self.device, staging)
        up.copy_stream.wait_stream(compute)
        for dec, (lo, hi) in zip(self.slices, self.ranges):
            up.send(lo, hi, dec.d_payload)
        for si, dec in enumerate(self.slices):
            compute.wait_event(up.wait(si))
            dec.run(stream=compute)
        up.close()
        return self.d_out[:self.archive.total]

    def check(self):
        for dec in self.slices:
            dec.check()


class Staging:
    """Page-locked staging between a file and the device: `depth` buffers of `block`
    bytes and the threads that fill and send them.  (Six threads: on a 16-core host four
    leave the link idle at times and eight or more slow the planning that runs beside them.)"""

    _shared = None

    def __init__(self, block: int = 32 << 20, depth: int = 8, threads: int = 6):
        import concurrent.futures

        import torch
        if threads >= depth:
            raise ValueError("staging needs more buffers than threads")
        self.block, self.depth = block, depth
        self.buffers = [torch.empty(block, dtype=torch.uint8).pin_memory() for _ in range(depth)]
        self.views = [b.numpy() for b in self.buffers]
        self.pool = concurrent.futures.ThreadPoolExecutor(threads)

    @classmethod
    def shared(cls):
        if cls._shared is None:
            cls._shared = cls()
        return cls._shared


class _Uploader:
    """Byte ranges of a host array -> device tensors through `Staging`, in the background.

    `send(lo, hi, dst)` queues one range ("a slice"); worker threads copy it block by
    block into page-locked buffers and start each block's host -> device copy themselves on
    one copy stream, so the caller is free to plan and launch meanwhile.  `wait(i)` blocks
    until every block of the i-th range has been issued and returns a CUDA event that
    completes when they have all arrived."""

    def __init__(self, blob, device, staging=None):
        import threading

        import torch
        self.blob, self.device = blob, device
        self.st = staging if staging is not None else Staging.shared()
        self.copy_stream = torch.cuda.Stream(device)
        self.lock = threading.Lock()
        self.turn = threading.Condition()
        self.slot_free = [None] * self.st.depth        # CUDA event: the slot's last copy has left it
        self.slot_round = [0] * self.st.depth          # blocks that have been through each buffer
        self.nblocks = 0
        self.failed = False
        self.left, self.ready, self.events, self.tasks = [], [], [], []

    def send(self, lo: int, hi: int, dst):
        import threading
        si = len(self.left)
        spans = [(b, min(b + self.st.block, hi)) for b in range(lo, hi, self.st.block)]
        self.left.append(len(spans))
        self.ready.append(threading.Event())
        self.events.append(None)
        if not spans:
            self._finish(si)
        for b, e in spans:
            self.tasks.append(self.st.pool.submit(self._block, si, self.nblocks, b, e, dst[b - lo:e - lo]))
            self.nblocks += 1
        return si

    def _finish(self, si):
        import torch
        with torch.cuda.stream(self.copy_stream):
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self.events[si] = ev
        self.ready[si].set()

    def _block(self, si, index, lo, hi, dst):
        import torch
        try:
            slot, rnd = index % self.st.depth, index // self.st.depth
            with torch.cuda.device(self.device):
                # a buffer takes its blocks strictly in turn: block `index` may fill it only after
                # block `index - depth` has issued its copy (tasks start in order but may finish in
                # any) and that copy has left the buffer
                with self.turn:
                    self.turn.wait_for(lambda: self.slot_round[slot] == rnd or self.failed)
                if self.failed:
                    raise RuntimeError("an earlier upload block failed")
                if self.slot_free[slot] is not None:
                    self.slot_free[slot].synchronize()
                np.copyto(self.st.views[slot][:hi - lo], self.blob[lo:hi])
                with self.lock:                      # one issuer at a time keeps stream order = event order
                    with torch.cuda.stream(self.copy_stream):
                        dst.copy_(self.st.buffers[slot][:hi - lo], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(self.copy_stream)
                    self.slot_free[slot] = ev
                    self.left[si] -= 1
                    if self.left[si] == 0:
                        self._finish(si)
                with self.turn:
                    self.slot_round[slot] = rnd + 1
                    self.turn.notify_all()
        except BaseException:
            self.failed = True
            with self.turn:
                self.turn.notify_all()
            self.ready[si].set()                     # wake the waiter; result() re-raises below
            raise

    def wait(self, si):
        self.ready[si].wait()
        if self.events[si] is None:
            for t in self.tasks:
                t.result()                           # surfaces the worker's exception
            raise RuntimeError("an upload block failed")
        return self.events[si]

    def close(self):
        for t in self.tasks:
            t.result()


def _slice_groups(ar, nslices):
    """Record indices of an archive cut into runs of consecutive payload bytes of about
    equal size (refs and deltas read other chunks' output: one run then)."""
    r = ar.records
    if nslices is None:
        big = int((r["rlen"] >= (1 << 20)).sum())
        nslices = 8 if big == 0 else max(1, min(8, big // 1900))
    sourced = np.isin(r["codec"], (fmt.CODEC_REF, fmt.CODEC_DELTA)).any()
    order = np.argsort(r["off"], kind="stable")
    nslices = 1 if sourced or r.size < nslices else nslices
    cum = np.cumsum(r["clen"][order].astype(np.int64))
    cuts = np.searchsorted(cum, cum[-1] * np.arange(1, nslices) / nslices) if r.size else []
    return [g for g in np.split(order, cuts) if g.size]


def load_archive(path, device=None, checksum: bool = True, nslices=None, stats=None, staging=None):
    """File on disk -> verified plaintext in HBM (the load the reference times as "cold
    disk -> VRAM", README.md:79-84).  The archive is mapped and its index read; its chunks
    are cut into slices of consecutive payload bytes; background threads stream slice
    after slice through page-locked staging to the device; each slice is planned while it
    is on its way (after the copy has brought its pages in, so the planner's reads of the
    in-payload headers cost nothing) and decoded as soon as it has arrived, under the
    copies of the next; every chunk's verdict is checked at the end.  Returns the decoded
    output space as a device tensor.  `stats`, a dict, receives `open_s` (map + index),
    `run_s` (everything else), `plan_s` (planning inside run_s), `h2d_bytes`, `slices`."""
    import time

    import torch
    t0 = time.perf_counter()
    ar = fmt.Archive(path)
    ar.check_coverage()
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    r = ar.records
    groups = _slice_groups(ar, nslices)
    t1 = time.perf_counter()
    with torch.cuda.device(dev):
        out = torch.empty(ar.total + 64, dtype=torch.uint8, device=dev)
        compute = torch.cuda.current_stream(dev)
        up = _Uploader(ar.blob, dev, staging)
        pad = gpu.pad_bytes()
        spans, payloads = [], []
        for g in groups:
            lo = int(r["off"][g].min())
            hi = int((r["off"][g].astype(np.int64) + r["clen"][g]).max())
            # room behind the payload for header chunks the planner inflates on the host
            general = (r["codec"][g] == fmt.CODEC_ZSTD) & np.isin(r["flags"][g] & 3, (fmt.METHOD_ZSTD, fmt.METHOD_DEFLATE))
            extra = int(r["rlen"][g][general].sum())
            d = torch.empty(hi - lo + extra + pad, dtype=torch.uint8, device=dev)
            spans.append((lo, hi))
            payloads.append(d)
            up.send(lo, hi, d)
        decs, plan_s = [], 0.0
        for si, g in enumerate(groups):
            arrived = up.wait(si)                    # every block of the slice has been read and issued
            tp = time.perf_counter()
            p = planner.build_plan(ar, select=g, payload_range=spans[si])
            dec = ArchiveDecoder(ar, device=dev, checksum=checksum, out=out, plan=p, payload=payloads[si])
            plan_s += time.perf_counter() - tp
            compute.wait_event(arrived)
            dec.run(stream=compute)
            decs.append(dec)
        up.close()
        for dec in decs:
            dec.check()
        torch.cuda.synchronize(dev)
    if stats is not None:
        stats.update(open_s=t1 - t0, run_s=time.perf_counter() - t1, plan_s=plan_s,
                     h2d_bytes=sum(hi - lo for lo, hi in spans), slices=len(groups))
    return out[:ar.total]


def decode_tensors(ar, names, device=None, checksum: bool = True):
    """Decode only what the named tensors need.  `names`: (member path, tensor name)
    keys of `Archive.tensor_index()`, or bare tensor names when they are unambiguous.
    Uploads the payload bytes of the chunks that overlap those tensors (and of the
    sources of any ref or delta among them), decodes them into a buffer that spans
    just their part of the output space, verifies, and returns {key: device tensor}."""
    import torch
    from . import multi

    ar = ar if isinstance(ar, fmt.Archive) else fmt.Archive(ar)
    index = ar.tensor_index()
    by_name = {}
    for key in index:
        by_name.setdefault(key[1], []).append(key)
    keys = []
    for n in names:
        if isinstance(n, tuple):
            if n not in index:
                raise KeyError(n)
            keys.append(n)
        else:
            hits = by_name.get(n, [])
            if len(hits) != 1:
                raise KeyError(f"{n!r} names {len(hits)} tensors; give (member path, name)")
            keys.append(hits[0])
    if not keys:
        return {}
    select = multi.cover(ar, [(index[k][2], index[k][3]) for k in keys])
    r = ar.records[select]
    out_lo = int(r["dst"].min()) & ~15                     # keep the output's 16-byte phase
    out_hi = int((r["dst"].astype(np.int64) + r["rlen"]).max())
    pay_lo = int(r["off"].min()) & ~15
    pay_hi = int((r["off"].astype(np.int64) + r["clen"]).max())
    p = planner.build_plan(ar, select=select, payload_range=(pay_lo, pay_hi), out_range=(out_lo, out_hi))
    dec = ArchiveDecoder(ar, device=device, checksum=checksum, plan=p)
    dec.run()
    dec.check()
    out = {}
    for k in keys:
        dt, shape, s, e = index[k]
        raw = dec.d_out[s - out_lo:e - out_lo]
        name = _TORCH_DTYPES.get(dt)
        if name is not None and (s - out_lo) % 2 == 0:
            try:
                raw = raw.view(getattr(torch, name)).reshape(shape)
            except RuntimeError:
                pass
        out[k] = raw
    return out


def decode_archive(ar, device=None, checksum: bool = True):
    """Decode a whole archive to a device tensor and verify it (the reference's
    `decompress` + `verify`, lmz/api.py:889, :1061, without the files)."""
    dec = ArchiveDecoder(ar, device=device, checksum=checksum)
    dec.run()
    dec.check()
    return dec.output
