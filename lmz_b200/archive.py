"""Reader for the reference's .lmz container (lmz/format.py:32-66, 325-366).

    [32 B header "LMZ\\x01", version, flags, original_size]
    [chunk payloads, each addressed by its record]
    [chunk table: N x 32 B records, zstd or deflate]
    [manifest JSON, zstd or deflate]
    [40 B footer: table off/len, manifest off/len, "LMZTAIL\\x01"]

The record table is kept as one flat numpy structured array -- it is already
the struct-of-records the planner wants -- and is never expanded into objects.
"""
from __future__ import annotations

import json
import os
import struct
import zlib

import numpy as np

MAGIC, TAIL = b"LMZ\x01", b"LMZTAIL\x01"
HEADER = struct.Struct("<4sHHQQQ")     # lmz/format.py:45
FOOTER = struct.Struct("<QQQQ8s")      # lmz/format.py:49
READABLE_VERSIONS = (1, 2, 3, 4, 5, 6)  # lmz/format.py:43
RECORD = np.dtype([("off", "<u8"), ("dst", "<u8"), ("clen", "<u4"), ("rlen", "<u4"),
                   ("crc", "<u4"), ("codec", "u1"), ("esize", "u1"), ("flags", "<u2")])

CODEC_STORED, CODEC_ZSTD, CODEC_SPLIT, CODEC_BF16, CODEC_REF = 0, 1, 2, 3, 4   # lmz/format.py:58-66
CODEC_BF16C, CODEC_BLK, CODEC_GBLK, CODEC_DELTA = 5, 6, 7, 8
# Shared-table option -- the format lever the reference proposes without defining a layout
# (docs/gpu-residency-handover.md:37-66); this one is this repository's.  A BF16 chunk whose
# exponent plane is coded against a 516-byte table stored once, in the payload region, for a
# run of chunks: payload = <IIQ (plane 0 length, plane 1 length, file offset of the table),
# plane 0 as [8 states][words] (scratchpad/gpu/shared_enc.c:1-13), plane 1 stored.
CODEC_BF16T = 9
FLAG_SHARED_TABLES = 4
TABLE_BYTES = 516
METHOD_STORED, METHOD_ZSTD, METHOD_DEFLATE, METHOD_RANS = 0, 1, 2, 3          # lmz/entropy.py:17-22
FLAG_PAGE_MAPPED = 1


class FormatError(ValueError):
    """Malformed, truncated, or not an archive (lmz/format.py:82-83)."""


class CorruptArchive(FormatError):
    """Data that fails to decode or to match its checksum (lmz/format.py:86-87)."""


def inflate_tail(raw: bytes) -> bytes:
    """The table, the manifest and header chunks are zstd where the writer had
    zstd and deflate otherwise (lmz/entropy.py:79-89); tell them apart by magic."""
    if raw[:4] == b"\x28\xb5\x2f\xfd":
        try:
            try:
                from compression import zstd as _z          # Python 3.14+
                return _z.decompress(raw)
            except ImportError:
                import zstandard as _zs
                return _zs.ZstdDecompressor().decompress(raw)
        except ImportError as exc:
            raise FormatError("this archive's index is zstd-coded and no zstd binding "
                              "is installed") from exc
    try:
        return zlib.decompress(raw)
    except zlib.error as exc:
        raise CorruptArchive(f"archive index failed to inflate: {exc}") from exc


class Archive:
    """Header, manifest and chunk records of one archive held in host memory."""

    def __init__(self, blob):
        if isinstance(blob, (str, os.PathLike)):
            # a file is mapped, not read: only the index at its end is touched here, and the
            # payload pages are read when they are uploaded
            blob = np.memmap(blob, dtype=np.uint8, mode="r")
        self.blob = blob if isinstance(blob, np.ndarray) else np.frombuffer(blob, dtype=np.uint8)
        b = self.blob
        if b.size < HEADER.size + FOOTER.size:
            raise FormatError("file is too small to be an lmz archive")
        magic, self.version, self.flags, self.original_size, _, _ = HEADER.unpack_from(b, 0)
        if magic != MAGIC:
            raise FormatError("not an lmz archive (bad magic)")
        if self.version not in READABLE_VERSIONS:
            raise FormatError(f"archive format v{self.version} is not understood")
        toff, tlen, moff, mlen, tail = FOOTER.unpack_from(b, b.size - FOOTER.size)
        if tail != TAIL:
            raise FormatError("archive is truncated or corrupt (bad footer)")
        for off, ln, what in ((toff, tlen, "chunk table"), (moff, mlen, "manifest")):
            if off < HEADER.size or off + ln > b.size:
                raise FormatError(f"{what} points outside the file")
        self.table_off = toff
        self.manifest = json.loads(inflate_tail(b[moff:moff + mlen].tobytes()))
        table = inflate_tail(b[toff:toff + tlen].tobytes())
        if len(table) % RECORD.itemsize:
            raise FormatError("chunk table has a partial record")
        self.records = np.frombuffer(table, dtype=RECORD)
        self.members = self.manifest.get("members", [])
        self.total = int(sum(m["size"] for m in self.members))
        r = self.records
        if r.size:
            # every payload inside [header, table), compared without forming off + clen
            # (an offset near 2^64 must not wrap into range)
            off, room = r["off"], np.uint64(self.table_off)
            inside = (off >= HEADER.size) & (off <= room)
            inside &= r["clen"].astype(np.uint64) <= room - np.minimum(off, room)
            if not inside.all():
                raise FormatError("a chunk payload points outside the payload region")

    @property
    def page_mapped(self) -> bool:
        return bool(self.flags & FLAG_PAGE_MAPPED)

    def check_coverage(self) -> None:
        """Chunks must tile [0, total) exactly (lmz/api.py:1038-1055).  Checked once."""
        if getattr(self, "_covered", False):
            return
        r = self.records
        order = np.argsort(r["dst"], kind="stable")
        dst = r["dst"][order].astype(np.int64)
        end = dst + r["rlen"][order]
        pos = np.concatenate(([0], end[:-1])) if r.size else np.zeros(0, np.int64)
        bad = np.nonzero(dst != pos)[0]
        if bad.size:
            raise FormatError(
                f"archive does not cover its output: gap or overlap at byte {int(pos[bad[0]])}")
        covered = int(end[-1]) if r.size else 0
        if covered != self.total:
            raise FormatError(f"archive covers {covered} bytes but declares {self.total}")
        self._covered = True

    def tensor_index(self):
        """{(member path, tensor name): (dtype string, shape, start, end)} in the
        concatenated output space (manifest layout: lmz/format.py:216-239)."""
        out = {}
        for m in self.members:
            for name, t in (m.get("tensors") or {}).items():
                s, e = t["offsets"]
                out[(m["path"], name)] = (t["dtype"], t["shape"], m["dst"] + s, m["dst"] + e)
        return out
