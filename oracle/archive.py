"""Read, decode and WRITE .lmz archives on the CPU.  Test infrastructure only.

Layout per lmz/format.py:32-66 (header, 32-byte chunk records, compressed
table + manifest, 40-byte footer).  `decode_archive` is the checker the CUDA
path is compared with and the timed CPU baseline; it follows the reference's
decode driver (lmz/api.py:832-886: refs and deltas resolve through a single
hop onto plain chunks).  `write_archive` produces inputs where the reference's
own Python cannot travel; it plans safetensors members the way the reference
does (lmz/planner.py:196-237 regions, :582-652 coalesce-then-slice).
"""
from __future__ import annotations

import json
import os
import struct
import zlib
from bisect import bisect_right
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import codec, encode, native

MAGIC, TAIL = b"LMZ\x01", b"LMZTAIL\x01"
HEADER = struct.Struct("<4sHHQQQ")
FOOTER = struct.Struct("<QQQQ8s")
RECORD = np.dtype([("off", "<u8"), ("dst", "<u8"), ("clen", "<u4"), ("rlen", "<u4"),
                   ("crc", "<u4"), ("codec", "u1"), ("esize", "u1"), ("flags", "<u2")])
assert RECORD.itemsize == 32
ST_ESIZE = {"BOOL": 1, "U8": 1, "I8": 1, "I16": 2, "U16": 2, "F16": 2, "BF16": 2,
            "I32": 4, "U32": 4, "F32": 4, "I64": 8, "U64": 8, "F64": 8}


def _inflate(raw: bytes) -> bytes:
    """Tail streams are zstd where the writer had it and deflate otherwise
    (lmz/entropy.py:88-89); this image has only deflate."""
    if raw[:4] == b"\x28\xb5\x2f\xfd":
        raise codec.Corrupt("archive tail is zstd-coded; no zstd on this image")
    return zlib.decompress(raw)


class Archive:
    """Header, manifest and the flat record table of one archive in memory."""

    def __init__(self, blob):
        self.blob = native._arr(blob)
        b = self.blob
        if b.size < 72:
            raise codec.Corrupt("file is too small to be an lmz archive")
        magic, self.version, self.flags, self.original_size, _, _ = HEADER.unpack_from(b, 0)
        if magic != MAGIC:
            raise codec.Corrupt("not an lmz archive (bad magic)")
        toff, tlen, moff, mlen, tail = FOOTER.unpack_from(b, b.size - 40)
        if tail != TAIL:
            raise codec.Corrupt("archive is truncated or corrupt (bad footer)")
        self.manifest = json.loads(_inflate(b[moff:moff + mlen].tobytes()))
        table = _inflate(b[toff:toff + tlen].tobytes())
        if len(table) % 32:
            raise codec.Corrupt("chunk table has a partial record")
        self.records = np.frombuffer(table, dtype=RECORD)
        self.members = self.manifest.get("members", [])
        self.total = sum(m["size"] for m in self.members)

    def payload(self, r) -> np.ndarray:
        return self.blob[int(r["off"]):int(r["off"]) + int(r["clen"])]


def _decode_plain(ar, c, verify, lib):
    if int(c["codec"]) == codec.CODEC_BF16T:
        return codec.decode_bf16t(ar.payload(c), int(c["rlen"]), int(c["crc"]), verify, lib, ar.blob)
    return codec.decode_chunk(ar.payload(c), int(c["codec"]), int(c["esize"]), int(c["flags"]),
                              int(c["rlen"]), int(c["crc"]), verify, lib)


def decode_archive(blob, workers: int = 1, verify: bool = True, lib=None) -> np.ndarray:
    """Every chunk decoded into one output buffer (lmz/api.py:889-975 without
    the file writes; coverage check :1038-1055)."""
    ar = blob if isinstance(blob, Archive) else Archive(blob)
    recs = ar.records
    order = np.argsort(recs["dst"], kind="stable")
    pos = 0
    for i in order:
        if int(recs["dst"][i]) != pos:
            raise codec.Corrupt(f"archive does not cover its output at byte {pos}")
        pos += int(recs["rlen"][i])
    if pos != ar.total:
        raise codec.Corrupt(f"archive covers {pos} bytes but declares {ar.total}")
    out = np.empty(ar.total, dtype=np.uint8)
    starts = recs["dst"][order].tolist()

    def resolve(src: int, rlen: int) -> np.ndarray:       # lmz/api.py:844-862
        buf = np.empty(rlen, dtype=np.uint8)
        p, end = src, src + rlen
        i = bisect_right(starts, p) - 1
        while p < end:
            if not 0 <= i < len(order):
                raise codec.Corrupt(f"source at byte {p} is not covered")
            c = recs[order[i]]
            d, rl = int(c["dst"]), int(c["rlen"])
            if not d <= p < d + rl:
                raise codec.Corrupt(f"source at byte {p} is not covered")
            if c["codec"] in (codec.CODEC_REF, codec.CODEC_DELTA):
                raise codec.Corrupt("a ref or delta chunk points at another one")
            data = _decode_plain(ar, c, verify, lib)
            a, b = p - d, min(end - d, rl)
            buf[p - src:p - src + (b - a)] = data[a:b]
            p = d + b
            i += 1
        return buf

    def work(i: int) -> None:
        c = recs[i]
        d, rl, cid = int(c["dst"]), int(c["rlen"]), int(c["codec"])
        pl = ar.payload(c)
        if cid == codec.CODEC_REF:
            if pl.size != 8:
                raise codec.Corrupt("ref chunk payload must be 8 bytes")
            data = resolve(struct.unpack("<Q", pl.tobytes())[0], rl)
        elif cid == codec.CODEC_DELTA:
            src, _inner, _off = codec.delta_source(pl)
            data = codec.decode_delta(pl, int(c["esize"]), int(c["flags"]), rl,
                                      resolve(src, rl), int(c["crc"]), verify, lib)
        else:
            data = _decode_plain(ar, c, verify, lib)
        out[d:d + rl] = data

    if workers <= 1:
        for i in range(recs.size):
            work(i)
    else:
        with ThreadPoolExecutor(workers) as ex:
            list(ex.map(work, range(recs.size), chunksize=max(1, recs.size // (workers * 8))))
    return out


# --------------------------------------------------------------------- writer

def parse_safetensors(a: np.ndarray):
    """(regions, tensors) of one safetensors member (lmz/planner.py:196-237)."""
    if a.size < 8:
        return None
    hlen = int.from_bytes(a[:8].tobytes(), "little")
    if hlen <= 0 or 8 + hlen > a.size:
        return None
    try:
        meta = json.loads(a[8:8 + hlen].tobytes())
    except ValueError:
        return None
    base, regions, tensors = 8 + hlen, [], {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        s, e = info["data_offsets"]
        dt = info.get("dtype", "")
        if e > s:
            regions.append((base + s, base + e, ST_ESIZE.get(dt, 1),
                            codec.KIND_BF16 if dt == "BF16" else codec.KIND_BYTES))
        tensors[name] = {"dtype": dt, "shape": info.get("shape", []),
                         "offsets": [base + s, base + e]}
    return (regions, tensors) if tensors else None


KIND_REF = 2     # lmz/planner.py:146


def _chunkify(regions, size: int, chunk_size: int, deltas):
    """(start, end, esize, kind, src) tasks covering [0, size)
    (lmz/planner.py:582-652; `deltas` = {(start, end): src} whole regions)."""
    regions = sorted(regions)
    covered, pos = [], 0
    for s, e, es, kind in regions:
        if s > pos:
            covered.append([pos, s, 1, codec.KIND_BYTES, -1])
        src = deltas.get((s, e), -1)
        if isinstance(src, tuple):          # an exact duplicate: a ref, not a delta
            covered.append([s, e, es, KIND_REF, src[0]])
        else:
            covered.append([s, e, es, kind, src])
        pos = e
    if pos < size:
        covered.append([pos, size, 1, codec.KIND_BYTES, -1])
    merged = []
    for r in covered:
        p = merged[-1] if merged else None
        if (p is not None and p[1] == r[0] and (p[2] == r[2] or r[3] == KIND_REF) and p[3] == r[3]
                and (p[4] >= 0) == (r[4] >= 0)
                and (p[4] < 0 or p[4] + (p[1] - p[0]) == r[4])):
            p[1] = r[1]
        else:
            merged.append(list(r))
    out = []
    for s, e, es, kind, src in merged:
        step = max(chunk_size - chunk_size % es, es)
        p = s
        while p < e:
            stop = min(p + step, e)
            if kind != KIND_REF and (stop - p) % es and stop == e:
                out.append((p, stop, 1, codec.KIND_BYTES, -1))
            else:
                out.append((p, stop, es, kind, src + (p - s) if src >= 0 else -1))
            p = stop
    return out


def write_archive(members, chunk_size: int | None = None, mapped: bool = False,
                  delta: bool = True, workers: int = 1, level: int = 1, lib=None,
                  shared_tables: int = 0) -> bytes:
    """An archive of `members` = [(path, bytes-like)], laid out as the
    reference's `compress` lays it out (lmz/api.py:651-815, format.py:279-322).

    Delta candidates are chosen by a simpler rule than the reference's sampled
    search (lmz/api.py:592-598 keeps the earliest member holding a tensor as
    the source): a tensor of >= 64 KiB whose name, dtype and shape also appear
    in member 0 is coded as a delta against member 0's bytes.

    `shared_tables` = N > 0 turns on the shared-table option (codec.CODEC_BF16T): runs of
    up to N consecutive BF16 chunks of one member whose exponent plane is rANS-coded and
    whose sign/mantissa plane is stored share one frequency table, stored once before the
    run, wherever that is measured to be smaller than their own tables."""
    if chunk_size is None:
        chunk_size = (64 << 10) if mapped else (8 << 20)
    chunk_size = max(chunk_size, 1 << 16)
    L = lib or native.best()
    datas = [native._arr(d) for _p, d in members]
    metas, base, first = [], 0, None
    plan = []
    for idx, ((path, _d), a) in enumerate(zip(members, datas)):
        parsed = parse_safetensors(a)
        regions, tensors = parsed if parsed else ([], None)
        deltas = {}
        if idx == 0:
            first = tensors or {}
        elif delta and tensors:
            for name, t in tensors.items():
                t0 = first.get(name)
                s, e = t["offsets"]
                if not (t0 and t0["dtype"] == t["dtype"] and t0["shape"] == t["shape"]):
                    continue
                s0 = t0["offsets"][0]                      # member 0 sits at dst 0
                if e - s < (64 << 10):                     # DEDUP_MIN_TENSOR / DELTA_MIN_TENSOR, lmz/api.py:47,59
                    continue
                if np.array_equal(a[s:e], datas[0][s0:s0 + (e - s)]):
                    deltas[(s, e)] = (s0,)                 # dedup: lmz/api.py:748-753
                else:
                    deltas[(s, e)] = s0
        m = {"path": path, "size": int(a.size), "dst": base,
             "kind": "safetensors" if parsed else "raw", "mode": 0o644, "crc": 0}
        if tensors:
            m["tensors"] = tensors
        metas.append(m)
        for s, e, es, kind, src in _chunkify(regions, a.size, chunk_size, deltas):
            plan.append((idx, base, s, e, es, kind, src))
        base += a.size
    total = base

    def work(task):
        idx, mbase, s, e, es, kind, src = task
        data = datas[idx][s:e]
        if kind == KIND_REF:
            return mbase + s, e - s, [struct.pack("<Q", src)], codec.CODEC_REF, 1, 0, 0
        if src >= 0:
            parts, flags, crc = encode.encode_delta(data, datas[0][src:src + (e - s)], es,
                                                    kind, src, level, True, L)
            return mbase + s, e - s, parts, codec.CODEC_DELTA, es, flags, crc
        parts, cid, flags, crc = encode.encode_chunk(data, es, kind, level, True, L)
        return mbase + s, e - s, parts, cid, es, flags, crc

    if workers > 1:
        with ThreadPoolExecutor(workers) as ex:
            results = list(ex.map(work, plan))
    else:
        results = [work(t) for t in plan]

    # shared-table runs: (first result, table) for every run that pays
    run_table, run_of = {}, {}
    if shared_tables > 0:
        fits = [r[3] == codec.CODEC_BF16 and r[5] == 3 for r in results]
        i = 0
        while i < len(results):
            if not fits[i]:
                i += 1
                continue
            j = i
            while j < len(results) and fits[j] and plan[j][0] == plan[i][0] and j - i < shared_tables:
                j += 1
            exps = [L.split_bf16(datas[plan[t][0]][plan[t][2]:plan[t][3]])[0] for t in range(i, j)]
            own = [len(results[t][2][1]) for t in range(i, j)]          # parts = [header, plane 0, plane 1]
            freqs = encode.shared_table_for(exps, own, L) if j - i > 1 else None
            if freqs is not None:
                run_table[i] = freqs
                for t in range(i, j):
                    run_of[t] = i
            i = j

    body, recs, off = [b"\0" * 32], np.zeros(len(results), dtype=RECORD), 32
    table_at = {}
    for i, (dst, rlen, parts, cid, es, flags, crc) in enumerate(results):
        if i in run_table:
            body.append(b"R1\0\0" + run_table[i].astype("<u2").tobytes())
            table_at[i] = off
            off += 516
        if i in run_of:
            first = run_of[i]
            shared = encode.encode_bf16t(datas[plan[i][0]][plan[i][2]:plan[i][3]], run_table[first],
                                         table_at[first], L)
            if shared is not None:
                parts, cid = shared[0], codec.CODEC_BF16T
        clen = 0
        for p in parts:
            p = p.tobytes() if isinstance(p, np.ndarray) else bytes(p)
            body.append(p)
            clen += len(p)
        recs[i] = (off, dst, clen, rlen, crc, cid, es, flags)
        off += clen
    manifest = {"version": 1, "tool": "lmz-b200 oracle writer", "level": level,
                "chunk_size": chunk_size, "mapped": bool(mapped), "aligned": False,
                "entropy": "deflate", "checksum": "crc32", "total_size": total,
                "members": metas, "chunks": len(results), "table_raw_len": recs.nbytes}
    table_c = zlib.compress(recs.tobytes(), 3)
    man_c = zlib.compress(json.dumps(manifest, separators=(",", ":")).encode(), 3)
    body += [table_c, man_c, FOOTER.pack(off, len(table_c), off + len(table_c), len(man_c), TAIL)]
    if table_at:
        manifest["shared_tables"] = {"count": len(table_at), "run": int(shared_tables), "table_bytes": 516}
        body[-2] = zlib.compress(json.dumps(manifest, separators=(",", ":")).encode(), 3)
        body[-1] = FOOTER.pack(off, len(table_c), off + len(table_c), len(body[-2]), TAIL)
    body[0] = HEADER.pack(MAGIC, 6, (1 if mapped else 0) | (codec.FLAG_SHARED_TABLES if table_at else 0), total, 0, 0)
    return b"".join(body)
