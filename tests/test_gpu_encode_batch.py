"""GPU batch encoder against the CPU oracle's encoder (itself held byte-identical to the
reference's, tests/test_oracle_golden.py): the streams must be the same bytes, and they
must decode back through the GPU decoder."""
import numpy as np
import pytest

from helpers import DISTRIBUTIONS, distribution, shaped, SHAPES

pytestmark = pytest.mark.gpu


def _check(gpu, orc, plains):
    nstr, plane = len(plains), plains[0].size
    got = gpu.encode_batch(b"".join(p.tobytes() for p in plains), nstr, plane)
    assert got is not None, gpu.last_error()
    streams, offsets = got
    offs = np.frombuffer(offsets, dtype="<u8").reshape(nstr, 2)
    pos = 0
    for i, p in enumerate(plains):
        want = orc.rans_encode(p)
        o, n = int(offs[i, 0]), int(offs[i, 1])
        assert o == pos, f"stream {i} is not packed behind its predecessor"
        assert n == len(want), f"stream {i}: {n} bytes, the reference writes {len(want)}"
        assert streams[o:o + n] == want, f"stream {i} differs from the reference's bytes"
        pos += n
    assert pos == len(streams)
    back = gpu.decode_batch(streams, offsets, nstr, plane)
    assert bytes(back) == b"".join(p.tobytes() for p in plains)


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("plane", [1, 7, 8, 9, 127, 128, 129, 4096, 4097, 65537])
def test_shapes_and_ragged_planes(gpu, orc, name, plane):
    for nstr in (1, 5, 33):
        if plane > 4097 and nstr > 5:
            continue
        _check(gpu, orc, [shaped(name, plane, hash((name, plane, nstr, i)) & 0xFFFF) for i in range(nstr)])


@pytest.mark.parametrize("dist", DISTRIBUTIONS)
@pytest.mark.parametrize("n", [1, 17, 4096, 65536, 1 << 20])
def test_stress_distributions(gpu, orc, dist, n):
    nstr = 3 if n >= 65536 else 40
    _check(gpu, orc, [distribution(dist, n, 7 * i + n) for i in range(nstr)])


def test_device_tensors_round_trip(gpu, orc):
    import torch
    plains = [distribution("exponent", 32768, i) for i in range(200)]
    t = torch.from_numpy(np.concatenate(plains)).cuda()
    streams, offs = gpu.encode_batch(t, 200, 32768)
    assert streams.is_cuda and offs.is_cuda and offs.numel() == 400
    back = gpu.decode_batch(streams, offs, 200, 32768)
    assert torch.equal(back, t)
    o = offs.cpu().numpy().reshape(200, 2)
    s = streams.cpu().numpy()
    assert s[o[17, 0]:o[17, 0] + o[17, 1]].tobytes() == orc.rans_encode(plains[17])


def test_arguments(gpu):
    assert gpu.encode_batch(b"", 0, 16) == (b"", b"")
    with pytest.raises(ValueError):
        gpu.encode_batch(b"abc", 2, 16)
    with pytest.raises(ValueError):
        gpu.encode_batch(b"abc", 1, 0)


def test_random_round_trips(gpu, orc):
    """Seeded random planes - alphabet size, skew, length and batch size all drawn - through
    encode_batch and back through decode_batch in every table mode; the first stream of
    every batch is also held to the oracle's encoder."""
    rng = np.random.default_rng(20261125)
    lib = gpu.library()
    try:
        for trial in range(60):
            plane = int(rng.choice([1, 3, 64, 129, 1000, 4096, 20000, 70001]))
            nstr = int(rng.choice([1, 2, 9, 33, 130])) if plane <= 4096 else int(rng.choice([1, 3, 7]))
            live = int(rng.integers(1, 257))
            syms = rng.choice(256, live, replace=False)
            weights = rng.random(live) ** rng.integers(1, 8)
            weights /= weights.sum()
            data = syms[rng.choice(live, size=nstr * plane, p=weights)].astype(np.uint8)
            streams, offsets = gpu.encode_batch(data.tobytes(), nstr, plane)
            o = np.frombuffer(offsets, dtype="<u8").reshape(nstr, 2)
            assert streams[:int(o[0, 1])] == orc.rans_encode(data[:plane])
            lib.lmz_gpu_set_table_mode([0, 2, 3, -1][trial % 4])
            assert bytes(gpu.decode_batch(streams, offsets, nstr, plane)) == data.tobytes(), (trial, plane, nstr, live)
    finally:
        lib.lmz_gpu_set_table_mode(-1)
