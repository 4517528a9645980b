"""The partition across ranks, on the CPU: shard() over several world sizes, and
a two-process gloo run in which each rank decodes only its share (with the CPU
oracle standing in for the GPU) and an all-gather rebuilds the full output."""
import os
import socket

import numpy as np
import pytest

from oracle import archive as oa, codec, synth


def _delta_archive():
    c0 = synth.llama_shard([0, 1], 9, scale=0.125)
    info = oa.parse_safetensors(c0)[1]
    c1 = c0.copy()
    for i, (name, t) in enumerate(info.items()):
        s, e = t["offsets"]
        if i % 3 == 0 and e - s > 70000:
            c1[s:e] = synth.perturbed_bf16(c0[s:e], i)
    files = [c0, c1]
    return oa.write_archive([(f"ck/{i}.safetensors", f) for i, f in enumerate(files)],
                            chunk_size=1 << 18), np.concatenate(files)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_shards_tile_the_output_and_carry_their_sources(world):
    from lmz_b200 import archive, multi, plan
    blob, _src = _delta_archive()
    ar = archive.Archive(blob)
    r = ar.records
    src = multi.sources(ar)
    assert (src >= 0).sum() == ((r["codec"] == 4) | (r["codec"] == 8)).sum() > 0
    pos, owned_all = 0, []
    for rank in range(world):
        select, (lo, hi) = multi.shard(ar, rank, world)
        assert lo == pos and hi >= lo
        pos = hi
        own = select[(r["dst"][select] >= lo) & (r["dst"][select] < hi)]
        owned_all.append(own)
        # every source range of an owned ref/delta is covered by selected plain chunks
        have = np.zeros(ar.total, dtype=bool)
        for i in select:
            if src[i] < 0:
                have[int(r["dst"][i]):int(r["dst"][i]) + int(r["rlen"][i])] = True
        for i in own:
            if src[i] >= 0:
                assert have[src[i]:src[i] + int(r["rlen"][i])].all()
        p = plan.build_plan(ar, select=select)
        assert sorted(p.chunks["record"].tolist()) == list(range(select.size))
    assert pos == ar.total
    assert sorted(np.concatenate(owned_all).tolist()) == list(range(r.size))
    costs = [int((r["clen"][o].astype(np.int64) + r["rlen"][o]).sum()) for o in owned_all]
    assert max(costs) <= 1.6 * (sum(costs) / world) + int(r["rlen"].max()) * 2


def _rank_main(rank, world, port, blob_path, out_path):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lmz_b200 import archive, multi
    blob = np.fromfile(blob_path, dtype=np.uint8)
    ar = archive.Archive(blob)
    select, (lo, hi) = multi.shard(ar, rank, world)
    # decode the share with the CPU oracle: plain chunks first, then refs and deltas
    out = np.zeros(ar.total, dtype=np.uint8)
    oar = oa.Archive(blob)
    src = multi.sources(ar)
    for phase in (0, 1):
        for i in select:
            c = oar.records[i]
            d, n = int(c["dst"]), int(c["rlen"])
            if (src[i] >= 0) != bool(phase):
                continue
            pl = oar.payload(c)
            if c["codec"] == codec.CODEC_REF:
                out[d:d + n] = out[src[i]:src[i] + n]
            elif c["codec"] == codec.CODEC_DELTA:
                out[d:d + n] = codec.decode_delta(pl, int(c["esize"]), int(c["flags"]), n,
                                                  out[src[i]:src[i] + n], int(c["crc"]))
            else:
                out[d:d + n] = codec.decode_chunk(pl, int(c["codec"]), int(c["esize"]),
                                                  int(c["flags"]), n, int(c["crc"]))
    # all-gather of equal padded shards, as ShardedDecoder.all_gather does on NCCL
    ranges = [None] * world
    dist.all_gather_object(ranges, (lo, hi))
    width = (max(b - a for a, b in ranges) + 15) & ~15
    mine = torch.zeros(width, dtype=torch.uint8)
    mine[:hi - lo] = torch.from_numpy(out[lo:hi].copy())
    parts = [torch.empty(width, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(parts, mine)
    full = np.zeros(ar.total, dtype=np.uint8)
    for rk, (a, b) in enumerate(ranges):
        full[a:b] = parts[rk][:b - a].numpy()
    if rank == 0:
        full.tofile(out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_decode_their_shares_and_gather(tmp_path):
    import torch.multiprocessing as mp
    blob, source = _delta_archive()
    bp, op = str(tmp_path / "a.lmz"), str(tmp_path / "out.bin")
    np.frombuffer(blob, dtype=np.uint8).tofile(bp)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, bp, op), nprocs=2, join=True)
    got = np.fromfile(op, dtype=np.uint8)
    assert (got == source).all()
