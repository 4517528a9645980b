"""Partition an archive's chunks over the GPUs of one node.

The reference has no multi-device path; its chunks are independent writes at
known destinations (lmz/format.py:11-15), which is what makes this a plain
partition: every rank decodes a contiguous run of chunks (in destination order,
balanced by coded + decoded bytes) from its own copy of those payloads into its
own HBM, with no collective on the data path.  A ref or delta chunk needs the
output range it names; when that range belongs to another rank, this rank
decodes the covering plain chunks as well (one hop, as in lmz/api.py:832-864)
rather than waiting for a peer.  For a full replica on every rank the output space is
cut into equal slices instead and one in-place NCCL all-gather rebuilds it.
"""
from __future__ import annotations

import numpy as np

from . import archive as fmt


def sources(ar: fmt.Archive) -> np.ndarray:
    """Per record: the output offset a ref/delta chunk reads from, or -1."""
    r, blob = ar.records, ar.blob
    src = np.full(r.size, -1, dtype=np.int64)
    idx = np.nonzero((r["codec"] == fmt.CODEC_REF) | (r["codec"] == fmt.CODEC_DELTA))[0]
    if idx.size:
        # a ref payload is the 8-byte source; a delta payload starts with it and an inner codec id
        short = r["clen"][idx] < np.where(r["codec"][idx] == fmt.CODEC_REF, 8, 9)
        if short.any():
            raise fmt.CorruptArchive("a ref or delta chunk is too short to name its source")
        off = r["off"][idx].astype(np.int64)
        raw = blob[off[:, None] + np.arange(8, dtype=np.int64)[None, :]]
        src[idx] = np.ascontiguousarray(raw).view("<u8")[:, 0].astype(np.int64)
    return src


def cover(ar: fmt.Archive, ranges) -> np.ndarray:
    """Record indices needed to produce the bytes [lo, hi) of the output space for
    every (lo, hi) in `ranges`: the chunks that overlap them, plus the plain chunks
    that cover the sources of any ref or delta among those (one hop)."""
    r = ar.records
    order = np.argsort(r["dst"], kind="stable")
    dst_sorted = r["dst"][order].astype(np.int64)

    def overlapping(pairs):
        got = [order[max(int(np.searchsorted(dst_sorted, lo, "right")) - 1, 0):
                     int(np.searchsorted(dst_sorted, hi, "left"))] for lo, hi in pairs if hi > lo]
        return np.unique(np.concatenate(got)) if got else np.zeros(0, dtype=np.int64)

    mine = overlapping(ranges)
    src = sources(ar)
    need = mine[src[mine] >= 0]
    extra = overlapping([(int(src[i]), int(src[i]) + int(r["rlen"][i])) for i in need])
    return np.union1d(mine, extra).astype(np.int64)


def shard(ar: fmt.Archive, rank: int, world: int):
    """(select, (lo, hi)): record indices rank `rank` must decode, and the byte
    range of the output space it owns.  The owned ranges of all ranks tile the
    output; `select` is the owned chunks plus the plain chunks that cover the
    sources of owned refs and deltas."""
    r = ar.records
    order = np.argsort(r["dst"], kind="stable")
    cost = (r["clen"].astype(np.int64) + r["rlen"])[order]
    cum = np.cumsum(cost)
    total = int(cum[-1]) if cum.size else 0
    # chunk i goes to the rank whose cost interval holds the chunk's midpoint
    mid = cum - cost // 2
    owner = np.minimum((mid * world) // max(total, 1), world - 1)
    mine = order[owner == rank]
    if mine.size:
        lo = int(r["dst"][mine[0]])
        hi = int(r["dst"][mine[-1]]) + int(r["rlen"][mine[-1]])
    else:
        lo = hi = int(ar.total) if rank else 0
    src = sources(ar)
    need = mine[src[mine] >= 0]
    extra = np.zeros(0, dtype=np.int64)
    if need.size:
        dst_sorted = r["dst"][order].astype(np.int64)
        s, e = src[need], src[need] + r["rlen"][need].astype(np.int64)
        first = np.searchsorted(dst_sorted, s, "right") - 1
        last = np.searchsorted(dst_sorted, e, "left")           # exclusive
        cover = np.concatenate([order[a:b] for a, b in zip(first, last)]) if need.size else extra
        extra = np.setdiff1d(np.unique(cover), mine)
    select = np.concatenate((mine, extra)).astype(np.int64)
    return select, (lo, hi)


def slice_width(total: int, world: int) -> int:
    """Bytes of the output space each rank holds when a full replica is rebuilt by an
    in-place all-gather: equal slices, a multiple of 256 bytes."""
    return ((-(-max(total, 1) // world)) + 255) & ~255


def slice_shard(ar: fmt.Archive, rank: int, world: int):
    """(select, (lo, hi)) for the replica layout: rank `rank` produces the output bytes
    [rank * w, (rank + 1) * w) clipped to the total, w = slice_width().  A chunk that
    straddles a slice boundary is decoded by both neighbours, so every rank's slice is
    complete without talking to a peer."""
    w = slice_width(int(ar.total), world)
    lo, hi = min(rank * w, int(ar.total)), min((rank + 1) * w, int(ar.total))
    return cover(ar, [(lo, hi)]), (lo, hi)


def gather_replica(buf, rank: int, world: int, width: int, group=None):
    """All-gather in place: `buf` holds at least world * width bytes and this rank's slice
    [rank * width, (rank + 1) * width) is filled; afterwards every slice is.  One
    collective, no staging buffer: NCCL is given the slice as a view of the buffer it
    gathers into (its in-place form).  On CPU tensors (gloo) the slice is cloned first,
    because that backend does not take aliased arguments."""
    import torch.distributed as dist
    whole = buf[:world * width]
    mine = whole[rank * width:(rank + 1) * width]
    if not buf.is_cuda:
        mine = mine.clone()
    dist.all_gather_into_tensor(whole, mine, group=group)
    return whole


class ShardedDecoder:
    """Rank `rank`'s share of an archive on its GPU.

    `replica=False` (default): the chunks are partitioned by coded + decoded bytes (see
    `shard`) and the rank's buffer holds only the stretch of the output space its chunks
    and their sources span -- 1/world of it for an archive without refs or deltas.
    `owned()` is the decoded range the rank is responsible for.

    `replica=True`: the output space is cut into equal slices (see `slice_shard`), every
    rank allocates the whole of it, decodes its slice, and `all_gather()` fills in the
    rest with one in-place NCCL all-gather over NVLink."""

    def __init__(self, ar, rank: int, world: int, device=None, checksum: bool = True,
                 replica: bool = False):
        import torch

        from . import decode, plan
        self.archive = ar if isinstance(ar, fmt.Archive) else fmt.Archive(ar)
        self.rank, self.world, self.replica = rank, world, replica
        self.select, self.range = (slice_shard if replica else shard)(self.archive, rank, world)
        r = self.archive.records
        sel = self.select
        pay = out_range = out = None
        self.width = slice_width(int(self.archive.total), world)
        dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if sel.size:                 # upload only the stretch of the payload this rank reads
            off = r["off"][sel].astype(np.int64)
            pay = (int(off.min()) & ~15, int((off + r["clen"][sel]).max()))
        if replica:
            out = torch.empty(self.width * world + 64, dtype=torch.uint8, device=dev)
        elif sel.size:
            dst = r["dst"][sel].astype(np.int64)
            out_range = (int(dst.min()) & ~15, int((dst + r["rlen"][sel]).max()))
        else:
            out_range = (0, 0)
        self.out_lo = out_range[0] if out_range else 0
        p = plan.build_plan(self.archive, select=sel, payload_range=pay, out_range=out_range)
        self.decoder = decode.ArchiveDecoder(self.archive, device=dev, checksum=checksum, plan=p, out=out)
        own = sel[(r["dst"][sel] >= self.range[0]) & (r["dst"][sel] < max(self.range[1], self.range[0] + 1))]
        self.owned_plain = int(r["rlen"][own].sum())
        self.owned_coded = int(r["clen"][own].sum())
        self.h2d_bytes = int(pay[1] - pay[0]) if pay else 0
        self.payload_range = pay

    def run(self, stream=None):
        return self.decoder.run(stream)

    def upload(self, pinned, non_blocking: bool = True):
        """Host -> device copy of just this rank's payload stretch; `pinned` is a host
        uint8 tensor over the archive file from byte 0."""
        if self.payload_range:
            lo, hi = self.payload_range
            self.decoder.upload(pinned[lo:hi], non_blocking=non_blocking)

    def check(self):
        self.decoder.check()

    def owned(self):
        """Device view of the output bytes [range[0], range[1]) this rank is responsible for."""
        lo, hi = self.range
        return self.decoder.d_out[lo - self.out_lo:hi - self.out_lo]

    def all_gather(self, group=None):
        """Every rank's slice into every rank's buffer (replica mode): one in-place NCCL
        all-gather.  Returns the full output."""
        if not self.replica:
            raise RuntimeError("all_gather needs ShardedDecoder(..., replica=True)")
        gather_replica(self.decoder.d_out, self.rank, self.world, self.width, group=group)
        return self.decoder.d_out[:self.archive.total]
