"""decode_batch on the GPU against the CPU oracle (mirrors the reference's own
GPU tests, tests/test_lmz.py:2272-2390 and :2538-2570 in the reference tree)."""
import numpy as np
import pytest

from helpers import DISTRIBUTIONS, SHAPES, distribution, pack_streams, shaped

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[0, 2, 3, 4, -1], ids=["narrow", "compact", "wide1", "wide13", "auto"])
def table_mode(request, gpu):
    """Every test runs with both per-stream table layouts forced."""
    lib = gpu.library()
    assert lib.lmz_gpu_set_table_mode(request.param) == 0
    yield request.param
    lib.lmz_gpu_set_table_mode(-1)


def _check(gpu, orc, plains, header=None, freqs=None):
    nstr, plane = len(plains), plains[0].size
    if header is None:
        streams = [orc.rans_encode(p) for p in plains]
    else:
        streams = [orc.rans_encode_shared(p, freqs) for p in plains]
    blob, offs = pack_streams(streams)
    out = gpu.decode_batch(blob, offs, nstr, plane, header=header)
    assert out is not None, gpu.last_error()
    out = np.frombuffer(out, dtype=np.uint8).reshape(nstr, plane)
    for i, p in enumerate(plains):
        assert (out[i] == p).all(), f"stream {i} differs"
        if header is None:
            assert (orc.rans_decode(streams[i], plane) == p).all()


def test_matches_cpu_64x4096(gpu, orc):
    plains = [shaped("skewed", 4096, 100 + i) for i in range(64)]
    _check(gpu, orc, plains)


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("plane", [1, 2, 7, 8, 9, 17, 127, 128, 129, 4096, 4097, 65537])
def test_shapes_and_ragged_planes(gpu, orc, name, plane):
    for nstr in (1, 17, 129):
        if plane > 4097 and nstr > 17:
            continue
        plains = [shaped(name, plane, hash((name, plane, nstr, i)) & 0xFFFF) for i in range(nstr)]
        _check(gpu, orc, plains)


@pytest.mark.parametrize("dist", DISTRIBUTIONS)
@pytest.mark.parametrize("n", [1, 17, 4096, 65536, 1 << 20])
def test_stress_distributions_per_stream_and_shared(gpu, orc, dist, n):
    nstr = 7 if n >= 65536 else 64
    plains = [distribution(dist, n, 7 * i + n) for i in range(nstr)]
    _check(gpu, orc, plains)
    counts = np.sum([np.bincount(p, minlength=256) for p in plains], axis=0)
    freqs = orc.rans_freqs(counts)
    header = b"R1\0\0" + freqs.astype("<u2").tobytes()
    _check(gpu, orc, plains, header=header, freqs=freqs)


def test_large_batches_are_sorted_by_alphabet_on_the_device(gpu, orc, table_mode):
    """12 000 short streams, every seventh with more live symbols than the dense instance
    of the throughput kernel holds: in automatic mode the library counts alphabets on the
    device and splits the launch; results must not depend on it."""
    if table_mode not in (-1, 2):
        pytest.skip("only the throughput kernel takes batches this large")
    pool = [distribution("uniform" if i % 7 == 0 else "exponent", 640, 900 + i) for i in range(70)]
    streams = [orc.rans_encode(p) for p in pool]
    n = 12000
    blob, offs = pack_streams([streams[i % 70] for i in range(n)])
    out = np.frombuffer(gpu.decode_batch(blob, offs, n, 640), dtype=np.uint8).reshape(n, 640)
    assert (out == np.stack([pool[i % 70] for i in range(n)])).all()
    bad = bytearray(blob)
    bad[int(np.frombuffer(offs, dtype="<u8")[2 * 777])] = ord("X")      # one stream's magic
    with pytest.raises(ValueError):
        gpu.decode_batch(bytes(bad), offs, n, 640)


def test_declines_and_errors(gpu, orc):
    plains = [shaped("skewed", 4096, i) for i in range(2)]
    blob, offs = pack_streams([orc.rans_encode(p) for p in plains])
    assert bytes(gpu.decode_batch(blob, offs, 0, 4096)) == b""
    with pytest.raises(ValueError):
        gpu.decode_batch(blob, offs, -1, 4096)
    with pytest.raises(ValueError):
        gpu.decode_batch(blob, offs[:16], 2, 4096)
    with pytest.raises(ValueError):
        gpu.decode_batch(blob, offs, 2, 4096, header=b"x" * 10)
    broken = bytearray(blob)
    broken[0] = ord("X")
    with pytest.raises(ValueError):
        gpu.decode_batch(bytes(broken), offs, 2, 4096)
    broken = bytearray(blob)
    broken[4] ^= 1                      # frequencies no longer sum to 4096
    with pytest.raises(ValueError):
        gpu.decode_batch(bytes(broken), offs, 2, 4096)
    # the superset: a plane that is not a multiple of 128 decodes
    out = gpu.decode_batch(blob, offs, 2, 4095)
    assert bytes(out[:4095]) == plains[0][:4095].tobytes()
    # truncated stream: the reference CPU decoder rejects it, so does this
    short = orc.rans_encode(shaped("flat", 4096, 9))
    cut = short[:len(short) - 200]
    b2, o2 = pack_streams([cut])
    with pytest.raises(ValueError):
        orc.rans_decode(cut, 4096)
    with pytest.raises(ValueError):
        gpu.decode_batch(b2, o2, 1, 4096)


def test_cuda_tensor_path(gpu, orc):
    import torch
    plains = [shaped("tail", 4099, i) for i in range(33)]
    blob, offs = pack_streams([orc.rans_encode(p) for p in plains])
    t = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    out = gpu.decode_batch(t, offs, 33, 4099)
    assert out.is_cuda
    assert out.cpu().numpy().tobytes() == b"".join(p.tobytes() for p in plains)


def test_verify_reports_ok(gpu):
    r = gpu.verify(quick=True)
    assert r["ok"], r
    assert r["checked"] >= 5 and r["gbps"] > 0


@pytest.mark.parametrize("dist", ["exponent", "uniform", "two"])
def test_stress_extremes_long_streams_and_wide_batches(gpu, orc, dist, table_mode):
    """The corners of the decoder stress matrix: 4 MiB streams (batch 1 and 7) and a
    4096-stream batch, per-stream and shared tables.  The wide batch cycles a pool of
    256 distinct streams so the CPU encoder stays out of the way."""
    if table_mode in (0, 3, -1) and dist != "exponent":
        pytest.skip("one distribution is enough for the narrow and wide-per-stream kernels")
    big = [distribution(dist, 4 << 20, 1000 + i) for i in range(7)]
    _check(gpu, orc, big[:1])
    _check(gpu, orc, big)
    pool = [distribution(dist, 4096, 50 + i) for i in range(256)]
    plains = [pool[i % 256] for i in range(4096)]
    streams = [orc.rans_encode(p) for p in pool]
    blob, offs = pack_streams([streams[i % 256] for i in range(4096)])
    out = np.frombuffer(gpu.decode_batch(blob, offs, 4096, 4096), dtype=np.uint8).reshape(4096, 4096)
    assert (out == np.stack(plains)).all()
    counts = np.sum([np.bincount(p, minlength=256) for p in pool], axis=0)
    freqs = orc.rans_freqs(counts)
    header = b"R1\0\0" + freqs.astype("<u2").tobytes()
    shared = [orc.rans_encode_shared(p, freqs) for p in pool]
    blob, offs = pack_streams([shared[i % 256] for i in range(4096)])
    out = np.frombuffer(gpu.decode_batch(blob, offs, 4096, 4096, header=header),
                        dtype=np.uint8).reshape(4096, 4096)
    assert (out == np.stack(plains)).all()
