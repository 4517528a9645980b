"""Write a large synthetic-model archive with many processes.  Test infrastructure.

Each worker generates the bytes of the chunks it is given from the shard's
seed, encodes them with the reference's compiled encoder (or the checker's),
and parks the payloads in a temporary file; the parent stitches payloads, chunk
table, manifest and footer together in the reference's layout
(lmz/format.py:279-322).  Chunk boundaries are those the reference's planner
produces for a safetensors file whose tensors all share one dtype: the header
is one byte-chunk, the data area is sliced every `chunk_size` bytes
(lmz/planner.py:582-652).
"""
from __future__ import annotations

import json
import multiprocessing as mp
import os
import tempfile
import zlib

import numpy as np

from . import archive, codec, encode, native, synth


def _tasks(layouts, chunk_size):
    """(member, start, end, esize, kind) for every chunk, in archive order."""
    out = []
    for m, lay in enumerate(layouts):
        es = synth._ESZ[lay.dtype]
        kind = codec.KIND_BF16 if lay.dtype == "BF16" else codec.KIND_BYTES
        p = 0
        while p < lay.data_start:
            q = min(p + chunk_size, lay.data_start)
            out.append((m, p, q, 1, codec.KIND_BYTES))
            p = q
        step = max(chunk_size - chunk_size % es, es)
        p = lay.data_start
        while p < lay.size:
            q = min(p + step, lay.size)
            out.append((m, p, q, es, kind))
            p = q
    return out


_G = {}


def _work(span):
    lo, hi = span
    layouts, tasks, tmpdir, run_len = _G["layouts"], _G["tasks"], _G["tmpdir"], _G.get("shared_tables", 0)
    L = native.best()
    recs, pos = [], 0
    path = os.path.join(tmpdir, f"part-{lo}.bin")
    with open(path, "wb", buffering=1 << 22) as f:
        def put(parts, rlen, crc, cid, es, flags, table_pos=-1):
            nonlocal pos
            clen = 0
            for p in parts:
                b = p.tobytes() if isinstance(p, np.ndarray) else bytes(p)
                f.write(b)
                clen += len(b)
            recs.append((pos, clen, rlen, crc, cid, es, flags, table_pos))
            pos += clen

        def flush(run):
            """A run of BF16 chunks with a coded exponent plane and a stored mantissa plane:
            one table for all of them where that is measured to be smaller."""
            nonlocal pos
            freqs = None
            if len(run) > 1:
                exps = [L.split_bf16(d)[0] for d, *_ in run]
                freqs = encode.shared_table_for(exps, [len(parts[1]) for _d, parts, *_ in run], L)
            table_pos = -1
            if freqs is not None:
                f.write(b"R1\0\0" + freqs.astype("<u2").tobytes())
                table_pos, pos = pos, pos + 516
            for data, parts, cid, flags, crc, es in run:
                shared = encode.encode_bf16t(data, freqs, 0, L) if freqs is not None else None
                if shared is not None:               # the table's file offset is patched in by the parent
                    put(shared[0], data.size, crc, codec.CODEC_BF16T, es, flags, table_pos)
                else:
                    put(parts, data.size, crc, cid, es, flags)
            run.clear()

        run, run_member = [], -1
        for t in range(lo, hi):
            m, s, e, es, kind = tasks[t]
            data = layouts[m].bytes(s, e)
            parts, cid, flags, crc = encode.encode_chunk(data, es, kind, 1, True, L)
            if run_len > 0 and cid == codec.CODEC_BF16 and flags == 3:
                if run and (m != run_member or len(run) >= run_len):
                    flush(run)
                run.append((data, parts, cid, flags, crc, es))
                run_member = m
                continue
            flush(run)
            put(parts, e - s, crc, cid, es, flags)
        flush(run)
    return lo, hi, path, recs, pos


def write_model_archive(spec, seed: int = 1, chunk_size: int | None = None, mapped: bool = False,
                        nproc: int | None = None, sigma: float = 0.02, shared_tables: int = 0):
    """Returns (archive bytes as a numpy array, layouts).  `spec` is a list of
    shards, each a list of (name, dtype, shape).  `shared_tables` = N > 0: the shared-table
    option of `archive.write_archive`, in runs of up to N chunks (a run never crosses from
    one worker's stretch of chunks into the next)."""
    if chunk_size is None:
        chunk_size = (64 << 10) if mapped else (8 << 20)
    chunk_size = max(chunk_size, 1 << 16)
    layouts = [synth.ShardLayout(t, seed * 1000 + i, sigma) for i, t in enumerate(spec)]
    tasks = _tasks(layouts, chunk_size)
    nproc = nproc or os.cpu_count() or 1
    # spans of roughly equal plaintext, several per process for balance
    target = max(1, sum(t[2] - t[1] for t in tasks) // (nproc * 6))
    spans, lo, acc = [], 0, 0
    for i, t in enumerate(tasks):
        acc += t[2] - t[1]
        if acc >= target:
            spans.append((lo, i + 1))
            lo, acc = i + 1, 0
    if lo < len(tasks):
        spans.append((lo, len(tasks)))
    tmpdir = tempfile.mkdtemp(prefix="lmzgen-", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    _G.update(layouts=layouts, tasks=tasks, tmpdir=tmpdir, shared_tables=int(shared_tables))
    try:
        if nproc > 1:
            with mp.get_context("fork").Pool(nproc) as pool:
                results = pool.map(_work, spans, chunksize=1)
        else:
            results = [_work(s) for s in spans]
        results.sort()
        total_payload = sum(r[4] for r in results)
        recs = np.zeros(len(tasks), dtype=archive.RECORD)
        bases, base = [], 0
        for m, lay in enumerate(layouts):
            bases.append(base)
            base += lay.size
        members = [{"path": f"model-{m + 1:05d}-of-{len(layouts):05d}.safetensors", "size": lay.size,
                    "dst": bases[m], "kind": "safetensors", "mode": 0o644, "crc": 0,
                    "tensors": lay.tensors} for m, lay in enumerate(layouts)]
        manifest = {"version": 1, "tool": "lmz-b200 oracle writer", "level": 1,
                    "chunk_size": chunk_size, "mapped": bool(mapped), "aligned": False,
                    "entropy": "deflate", "checksum": "crc32", "total_size": base,
                    "members": members, "chunks": len(tasks), "table_raw_len": recs.nbytes}
        off = 32
        patch_at, patch_to = [], []          # shared-table chunks: where their table ended up
        for lo, hi, path, rr, size in results:
            for j, (pos, clen, rlen, crc, cid, es, flags, table_pos) in enumerate(rr):
                m, s, _e, _es, _k = tasks[lo + j]
                recs[lo + j] = (off + pos, bases[m] + s, clen, rlen, crc, cid, es, flags)
                if table_pos >= 0:
                    patch_at.append(off + pos + 8)
                    patch_to.append(off + table_pos)
            off += size
        if patch_at:
            manifest["shared_tables"] = {"count": len(set(patch_to)), "run": int(shared_tables), "table_bytes": 516}
        table_c = zlib.compress(recs.tobytes(), 3)
        man_c = zlib.compress(json.dumps(manifest, separators=(",", ":")).encode(), 3)
        tail = table_c + man_c + archive.FOOTER.pack(off, len(table_c), off + len(table_c),
                                                      len(man_c), archive.TAIL)
        blob = np.empty(32 + total_payload + len(tail), dtype=np.uint8)
        hflags = (1 if mapped else 0) | (codec.FLAG_SHARED_TABLES if patch_at else 0)
        blob[:32] = np.frombuffer(archive.HEADER.pack(archive.MAGIC, 6, hflags, base, 0, 0), dtype=np.uint8)
        p = 32
        for lo, hi, path, rr, size in results:
            if size:
                blob[p:p + size] = np.fromfile(path, dtype=np.uint8)
            p += size
            os.unlink(path)
        blob[p:] = np.frombuffer(tail, dtype=np.uint8)
        if patch_at:
            at = np.asarray(patch_at, dtype=np.int64)[:, None] + np.arange(8, dtype=np.int64)[None, :]
            blob[at] = np.asarray(patch_to, dtype="<u8").view(np.uint8).reshape(-1, 8)
        return blob, layouts
    finally:
        for f in os.listdir(tmpdir):
            os.unlink(os.path.join(tmpdir, f))
        os.rmdir(tmpdir)
