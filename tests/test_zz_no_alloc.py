"""The allocation-free checked decode, through the C ABI, against the existing
device entry point.

`lmz_gpu_decode_batch_dev_noalloc` is for hosts that cannot let this library call
cudaMalloc (their own pool owns the device's memory): its per-stream verdicts sit
in a fixed array inside the library, shared by every call, so the test makes
several calls in a row -- a failing batch first -- to show nothing leaks from one
call into the next, and compares the decoded bytes with `lmz_gpu_decode_batch_dev`.
The file name sorts last so a run that stops at the first failure has already
run every other test.
"""
import ctypes

import numpy as np
import pytest

from helpers import pack_streams, shaped

pytestmark = pytest.mark.gpu


def _upload(blob, offs, pad):
    import torch
    d = torch.zeros(len(blob) + pad, dtype=torch.uint8, device="cuda")
    d[:len(blob)] = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
    o = torch.frombuffer(bytearray(offs), dtype=torch.int64).cuda()
    return d, o


def _entry(gpu):
    lib = gpu.library()
    v, u = ctypes.c_void_p, ctypes.c_uint
    fn = lib.lmz_gpu_decode_batch_dev_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [v, v, v, u, u, v, v, v]
    return lib, fn


def test_noalloc_matches_the_device_entry_point_on_calls_in_a_row(gpu, orc):
    import torch
    lib, fn = _entry(gpu)
    cs = torch.cuda.current_stream().cuda_stream
    pad = gpu.pad_bytes()

    def both(plains, streams, plane):
        nstr = len(streams)
        blob, offs = pack_streams(streams)
        d, o = _upload(blob, offs, pad)
        want = torch.full((nstr * plane,), 0xAA, dtype=torch.uint8, device="cuda")
        got = torch.full((nstr * plane,), 0x55, dtype=torch.uint8, device="cuda")
        assert lib.lmz_gpu_decode_batch_dev(None, d.data_ptr(), o.data_ptr(), nstr, plane,
                                            want.data_ptr(), cs, 0) == 0
        status = np.full(nstr, 0xFFFFFFFF, dtype=np.uint32)
        rc = fn(None, d.data_ptr(), o.data_ptr(), nstr, plane, got.data_ptr(), cs,
                status.ctypes.data)
        torch.cuda.synchronize()
        return rc, got.cpu().numpy(), want.cpu().numpy(), status

    # call 1: one stream of the batch is truncated -> reported, the others still decode
    plains = [shaped("flat", 4096, 10 + i) for i in range(5)]
    streams = [orc.rans_encode(p) for p in plains]
    streams[3] = streams[3][:len(streams[3]) - 300]
    rc, got, want, status = both(plains, streams, 4096)
    assert rc == gpu.EBADSTREAM and "truncated" in gpu.last_error()
    assert status[3] == 2 and (status[[0, 1, 2, 4]] == 0).all()
    for i in (0, 1, 2, 4):
        assert (got[i * 4096:(i + 1) * 4096] == plains[i]).all()

    # calls 2 and 3: clean batches of other shapes; the earlier failure must not linger
    for seed, (name, plane, nstr) in enumerate((("skewed", 4099, 37), ("tail", 65537, 9))):
        plains = [shaped(name, plane, 100 * seed + i) for i in range(nstr)]
        streams = [orc.rans_encode(p) for p in plains]
        rc, got, want, status = both(plains, streams, plane)
        assert rc == 0, gpu.last_error()
        assert (status == 0).all()
        assert (got == want).all()
        assert got.tobytes() == b"".join(p.tobytes() for p in plains)

    # beyond the fixed array's capacity: refused with a message, nothing launched
    rc = fn(None, None, None, 65537, 128, None, cs, None)
    assert rc == gpu.EUNSUPPORTED and "65536" in gpu.last_error()


@pytest.mark.parametrize("nstr,plane,shared", [
    (2000, 256, False),      # narrow per-stream tables
    (12000, 64, False),      # compact tables; no index list may be allocated to sort them
    (65536, 64, False),      # the fixed array's last word
    (300, 512, True),        # one shared table, the plain kernel
    (20000, 64, True),       # one shared table, the throughput kernel
], ids=["narrow", "compact-unsorted", "capacity", "shared-plain", "shared-throughput"])
def test_noalloc_every_launch_path_reports_its_own_stream(gpu, orc, nstr, plane, shared):
    """Each launch path the entry point can take writes verdicts into the library's fixed
    array: one truncated stream (cut on the host) must come back as status 2 with its
    neighbours 0 and their bytes equal to the allocating entry point's, and the call must
    leave the device's free memory where it was."""
    import torch
    lib, fn = _entry(gpu)
    cs = torch.cuda.current_stream().cuda_stream
    pool_n = 61
    pool = [shaped("flat" if i % 5 else "skewed", plane, 3000 + i) for i in range(pool_n)]
    hdr = None
    if shared:
        counts = np.sum([np.bincount(p, minlength=256) for p in pool], axis=0)
        freqs = orc.rans_freqs(counts)
        coded = [orc.rans_encode_shared(p, freqs) for p in pool]
        hdr = torch.frombuffer(bytearray(b"R1\0\0" + freqs.astype("<u2").tobytes()), dtype=torch.uint8).cuda()
    else:
        coded = [orc.rans_encode(p) for p in pool]
    victim = nstr // 2 + 1
    streams = [coded[i % pool_n] for i in range(nstr)]
    assert len(streams[victim]) > (32 if shared else 548) + 8, "the victim needs coded words to lose"
    streams[victim] = streams[victim][:-6]
    blob, offs = pack_streams(streams)
    d, o = _upload(blob, offs, gpu.pad_bytes())
    want = torch.zeros(nstr * plane, dtype=torch.uint8, device="cuda")
    got = torch.zeros(nstr * plane, dtype=torch.uint8, device="cuda")
    h = hdr.data_ptr() if hdr is not None else None
    assert lib.lmz_gpu_decode_batch_dev(h, d.data_ptr(), o.data_ptr(), nstr, plane, want.data_ptr(), cs, 0) == 0
    status = np.full(nstr, 0xFFFFFFFF, dtype=np.uint32)
    fn(h, d.data_ptr(), o.data_ptr(), nstr, plane, got.data_ptr(), cs, status.ctypes.data)   # loads the kernels
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status[:] = 0xFFFFFFFF
    got.zero_()
    rc = fn(h, d.data_ptr(), o.data_ptr(), nstr, plane, got.data_ptr(), cs, status.ctypes.data)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
    assert rc == gpu.EBADSTREAM, gpu.last_error()
    assert status[victim] == 2, status[victim]
    others = np.delete(status, victim)
    assert (others == 0).all(), np.unique(others)
    g = got.cpu().numpy().reshape(nstr, plane)
    w = want.cpu().numpy().reshape(nstr, plane)
    keep = np.arange(nstr) != victim
    assert (g[keep] == w[keep]).all()
    assert (g[keep] == np.stack([pool[i % pool_n] for i in range(nstr)])[keep]).all()
