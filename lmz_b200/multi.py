"""Partition an archive's chunks over the GPUs of one node.

The reference has no multi-device path; its chunks are independent writes at
known destinations (lmz/format.py:11-15), which is what makes this a plain
partition: every rank decodes a contiguous run of chunks (in destination order,
balanced by coded + decoded bytes) from its own copy of those payloads into its
own HBM, with no collective on the data path.  A ref or delta chunk needs the
output range it names; when that range belongs to another rank, this rank
decodes the covering plain chunks as well (one hop, as in lmz/api.py:832-864)
rather than waiting for a peer.  `all_gather` optionally rebuilds the full
output on every rank with one NCCL all-gather of equal, padded shards.
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


class ShardedDecoder:
    """Rank `rank`'s share of an archive on its GPU (see `shard`)."""

    def __init__(self, ar, rank: int, world: int, device=None, checksum: bool = True):
        from . import decode, plan
        self.archive = ar if isinstance(ar, fmt.Archive) else fmt.Archive(ar)
        self.rank, self.world = rank, world
        self.select, self.range = shard(self.archive, rank, world)
        r = self.archive.records
        pay = None
        if self.select.size:                 # upload only the stretch of the payload this rank reads
            off = r["off"][self.select].astype(np.int64)
            pay = (int(off.min()) & ~15, int((off + r["clen"][self.select]).max()))
        p = plan.build_plan(self.archive, select=self.select, payload_range=pay)
        self.decoder = decode.ArchiveDecoder(self.archive, device=device, checksum=checksum, plan=p)
        own = self.select[(r["dst"][self.select] >= self.range[0]) &
                          (r["dst"][self.select] < max(self.range[1], self.range[0] + 1))]
        self.owned_plain = int(r["rlen"][own].sum())
        self.owned_coded = int(r["clen"][own].sum())

    def run(self, stream=None):
        return self.decoder.run(stream)

    def check(self):
        self.decoder.check()

    def all_gather(self, group=None):
        """Every rank's owned range into every rank's output buffer (NCCL)."""
        import torch
        import torch.distributed as dist
        out = self.decoder.d_out
        ranges = [None] * self.world
        dist.all_gather_object(ranges, self.range, group=group)
        width = max(hi - lo for lo, hi in ranges)
        width = (width + 15) & ~15
        lo, hi = self.range
        mine = torch.zeros(width, dtype=torch.uint8, device=out.device)
        mine[:hi - lo] = out[lo:hi]
        gathered = torch.empty(width * self.world, dtype=torch.uint8, device=out.device)
        dist.all_gather_into_tensor(gathered, mine, group=group)
        for rk, (a, b) in enumerate(ranges):
            if rk != self.rank:
                out[a:b] = gathered[rk * width:rk * width + (b - a)]
        return self.decoder.output
