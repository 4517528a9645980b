"""The partition across ranks, on the CPU: shard() over several world sizes, and
a two-process gloo run in which each rank decodes only its slice (with the CPU
oracle standing in for the GPU) and the library's in-place all-gather rebuilds the
full output."""
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


@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_slices_tile_the_output_and_are_self_contained(world):
    """Replica layout: equal slices; a rank's selection covers its slice and the sources of
    every ref or delta in it."""
    from lmz_b200 import archive, multi
    blob, _src = _delta_archive()
    ar = archive.Archive(blob)
    r = ar.records
    src = multi.sources(ar)
    w = multi.slice_width(ar.total, world)
    assert w % 256 == 0 and w * world >= ar.total
    pos = 0
    for rank in range(world):
        select, (lo, hi) = multi.slice_shard(ar, rank, world)
        assert lo == pos and hi - lo <= w
        pos = hi
        have = np.zeros(ar.total, dtype=bool)
        plain = np.zeros(ar.total, dtype=bool)
        for i in select:
            have[int(r["dst"][i]):int(r["dst"][i]) + int(r["rlen"][i])] = True
            if src[i] < 0:
                plain[int(r["dst"][i]):int(r["dst"][i]) + int(r["rlen"][i])] = True
        assert have[lo:hi].all()
        for i in select:
            if src[i] >= 0 and int(r["dst"][i]) < hi and int(r["dst"][i]) + int(r["rlen"][i]) > lo:
                assert plain[src[i]:src[i] + int(r["rlen"][i])].all()
    assert pos == ar.total
    # an empty share plans to nothing
    from lmz_b200 import plan
    p = plan.build_plan(ar, select=np.zeros(0, dtype=np.int64), out_range=(0, 0))
    assert p.chunks.size == 0 and p.total == 0


def _rank_main(rank, world, port, blob_path, out_path):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lmz_b200 import archive, multi
    blob = np.fromfile(blob_path, dtype=np.uint8)
    ar = archive.Archive(blob)
    select, (lo, hi) = multi.slice_shard(ar, rank, world)
    width = multi.slice_width(ar.total, world)
    # decode the share with the CPU oracle: plain chunks first, then refs and deltas
    out = np.zeros(width * world, dtype=np.uint8)
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
    # what lies outside this rank's slice must come from its peers: wipe it, then run the
    # library's own in-place all-gather (the call ShardedDecoder.all_gather makes on NCCL)
    out[:lo] = 0xEE
    out[hi:] = 0xEE
    buf = torch.from_numpy(out)
    multi.gather_replica(buf, rank, world, width)
    full = buf.numpy()[:ar.total]
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
