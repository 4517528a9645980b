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
    layouts, tasks, tmpdir = _G["layouts"], _G["tasks"], _G["tmpdir"]
    L = native.best()
    recs, pos = [], 0
    path = os.path.join(tmpdir, f"part-{lo}.bin")
    with open(path, "wb", buffering=1 << 22) as f:
        for t in range(lo, hi):
            m, s, e, es, kind = tasks[t]
            data = layouts[m].bytes(s, e)
            parts, cid, flags, crc = encode.encode_chunk(data, es, kind, 1, True, L)
            clen = 0
            for p in parts:
                b = p.tobytes() if isinstance(p, np.ndarray) else bytes(p)
                f.write(b)
                clen += len(b)
            recs.append((pos, clen, e - s, crc, cid, es, flags))
            pos += clen
    return lo, hi, path, recs, pos


def write_model_archive(spec, seed: int = 1, chunk_size: int | None = None, mapped: bool = False,
                        nproc: int | None = None, sigma: float = 0.02):
    """Returns (archive bytes as a numpy array, layouts).  `spec` is a list of
    shards, each a list of (name, dtype, shape)."""
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
    _G.update(layouts=layouts, tasks=tasks, tmpdir=tmpdir)
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
        for lo, hi, path, rr, size in results:
            for j, (pos, clen, rlen, crc, cid, es, flags) in enumerate(rr):
                m, s, _e, _es, _k = tasks[lo + j]
                recs[lo + j] = (off + pos, bases[m] + s, clen, rlen, crc, cid, es, flags)
            off += size
        table_c = zlib.compress(recs.tobytes(), 3)
        man_c = zlib.compress(json.dumps(manifest, separators=(",", ":")).encode(), 3)
        tail = table_c + man_c + archive.FOOTER.pack(off, len(table_c), off + len(table_c),
                                                      len(man_c), archive.TAIL)
        blob = np.empty(32 + total_payload + len(tail), dtype=np.uint8)
        blob[:32] = np.frombuffer(archive.HEADER.pack(archive.MAGIC, 6, 1 if mapped else 0,
                                                      base, 0, 0), dtype=np.uint8)
        p = 32
        for lo, hi, path, rr, size in results:
            if size:
                blob[p:p + size] = np.fromfile(path, dtype=np.uint8)
            p += size
            os.unlink(path)
        blob[p:] = np.frombuffer(tail, dtype=np.uint8)
        return blob, layouts
    finally:
        for f in os.listdir(tmpdir):
            os.unlink(os.path.join(tmpdir, f))
        os.rmdir(tmpdir)
