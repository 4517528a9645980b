"""ShardedDecoder on one GPU, rank by rank: what every rank of a partitioned decode
produces, stitched together, must be the oracle's output -- for the cost-balanced
partition (each rank's buffer holding only its own stretch) and for the equal-slice
replica layout (the in-place all-gather is emulated here by copying the slices, since
one process has one rank; the collective itself runs in tests/test_multi_rank.py on
gloo and in the benchmark on NCCL)."""
import numpy as np
import pytest

from oracle import archive as oa, synth

pytestmark = pytest.mark.gpu


def _delta_archive():
    c0 = synth.llama_shard([0, 1], 9, scale=0.125)
    info = oa.parse_safetensors(c0)[1]
    c1 = c0.copy()
    for i, (name, t) in enumerate(info.items()):
        s, e = t["offsets"]
        if i % 3 == 0 and e - s > 70000:
            c1[s:e] = synth.perturbed_bf16(c0[s:e], i)
    files = [c0, c1]
    return oa.write_archive([(f"ck/{i}.safetensors", f) for i, f in enumerate(files)], chunk_size=1 << 18)


def _plain_archive():
    return oa.write_archive([("m.safetensors", synth.llama_shard([0], 5, scale=0.25, vocab=2000, embed=True))],
                            mapped=True)


@pytest.fixture(scope="module", params=["delta", "plain"])
def case(request, orc):
    blob = _delta_archive() if request.param == "delta" else _plain_archive()
    return request.param, blob, oa.decode_archive(blob, lib=orc)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_partitioned_ranks_stitch_to_the_oracle_output(gpu, case, world):
    from lmz_b200 import archive, multi
    kind, blob, want = case
    ar = archive.Archive(blob)
    got = np.zeros(ar.total, dtype=np.uint8)
    pos, spans = 0, []
    for rank in range(world):
        sd = multi.ShardedDecoder(ar, rank, world)
        sd.run()
        sd.check()
        lo, hi = sd.range
        assert lo == pos
        pos = hi
        got[lo:hi] = sd.owned().cpu().numpy()
        spans.append(sd.decoder.d_out.numel())
    assert pos == ar.total
    assert (got == want).all()
    if kind == "plain":
        # without refs or deltas a rank's buffer is its own stretch, not the whole output
        assert max(spans) <= ar.total // world + int(ar.records["rlen"].max()) * 2 + 128


@pytest.mark.parametrize("world", [2, 3, 8])
def test_replica_slices_gathered_give_the_oracle_output(gpu, case, world):
    import torch
    from lmz_b200 import archive, multi
    _kind, blob, want = case
    ar = archive.Archive(blob)
    width = multi.slice_width(ar.total, world)
    full = torch.zeros(width * world, dtype=torch.uint8, device="cuda")
    for rank in range(world):
        sd = multi.ShardedDecoder(ar, rank, world, replica=True)
        assert sd.decoder.d_out.numel() >= width * world
        sd.run()
        sd.check()
        # what the all-gather would carry: exactly this rank's slice
        full[rank * width:(rank + 1) * width] = sd.decoder.d_out[rank * width:(rank + 1) * width]
    assert (full[:ar.total].cpu().numpy() == want).all()
    with pytest.raises(RuntimeError):
        multi.ShardedDecoder(ar, 0, world).all_gather()
