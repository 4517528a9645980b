"""The CUDA decoder behind the reference's `lmz.gpu` interface.

Same module-level functions, arguments and error behaviour as
lmz/gpu/__init__.py:26-27,210-428 -- `available`, `backend`, `state`,
`last_error`, `grain`, `header_bytes`, `pad_bytes`, `verify`, `decode_batch` --
backed by this repository's sm_100a library.  Differences, all supersets:

* `grain()` is 1: any `plane >= 1` decodes, ragged tails included, so the
  reference's "not a multiple of the grain" decline never happens.
* a truncated stream raises ValueError instead of returning garbage.
* `decode_batch` also takes CUDA `torch.uint8` tensors and then returns one,
  decoding device to device with no host copy.

There is no CPU decoder here: when the library is unavailable `decode_batch`
returns None exactly as the reference does and the caller decides what to do.
"""
from __future__ import annotations

import ctypes
import json
import os
import subprocess
import sys
import threading

__all__ = ["available", "backend", "decode_batch", "grain", "header_bytes",
           "last_error", "pad_bytes", "state", "verify"]

ABI_VERSION = 1                      # lmz/gpu/__init__.py:31
OK, ENODEV, EUNSUPPORTED, EBADSTREAM, ECUDA, EMISMATCH = 0, -1, -2, -3, -4, -5

_C = ctypes
_SIGNATURES = {
    # name: (restype, argtypes)
    "lmz_gpu_abi_version": (_C.c_int, []),
    "lmz_gpu_grain": (_C.c_int, []),
    "lmz_gpu_header_bytes": (_C.c_int, []),
    "lmz_gpu_pad_bytes": (_C.c_int, []),
    "lmz_gpu_last_error": (_C.c_char_p, []),
    "lmz_gpu_device_name": (_C.c_int, [_C.c_char_p, _C.c_int]),
    "lmz_gpu_validate": (_C.c_int, [_C.c_void_p, _C.c_void_p, _C.c_uint]),
    "lmz_gpu_decode_batch": (_C.c_int, [_C.c_void_p, _C.c_void_p, _C.c_size_t, _C.c_void_p,
                                        _C.c_uint, _C.c_uint, _C.c_void_p]),
    "lmz_gpu_decode_batch_dev": (_C.c_int, [_C.c_void_p] * 3 + [_C.c_uint, _C.c_uint, _C.c_void_p,
                                                                 _C.c_void_p, _C.c_uint]),
    "lmz_gpu_decode_batch_dev_noalloc": (_C.c_int, [_C.c_void_p] * 3 + [_C.c_uint, _C.c_uint, _C.c_void_p,
                                                                         _C.c_void_p, _C.c_void_p]),
    "lmz_gpu_set_device": (_C.c_int, [_C.c_int]),
    "lmz_gpu_set_table_mode": (_C.c_int, [_C.c_int]),
    "lmz_gpu_decode_streams_dev": (_C.c_int, [_C.c_void_p, _C.c_uint] + [_C.c_void_p] * 6),
    "lmz_gpu_encode_slot_bytes": (_C.c_int, [_C.c_uint]),
    "lmz_gpu_encode_batch_dev": (_C.c_int, [_C.c_void_p, _C.c_uint, _C.c_uint] + [_C.c_void_p] * 3),
    "lmz_gpu_pack_streams_dev": (_C.c_int, [_C.c_void_p, _C.c_uint, _C.c_void_p, _C.c_uint,
                                            _C.c_void_p, _C.c_void_p]),
    "lmz_gpu_split_bf16_dev": (_C.c_int, [_C.c_void_p, _C.c_uint64, _C.c_uint, _C.c_void_p, _C.c_void_p]),
    "lmz_gpu_frame_bf16_dev": (_C.c_int, [_C.c_void_p, _C.c_uint64, _C.c_uint] + [_C.c_void_p] * 7),
    "lmz_gpu_crc32_chunks_dev": (_C.c_int, [_C.c_void_p, _C.c_uint64, _C.c_uint] + [_C.c_void_p] * 3),
}


class _Loader:
    """Finds, vets and opens the library once per process.

    The steps, each of which can end the attempt with a reason: LMZ_NO_GPU set ->
    build (or find) the library -> load it in a child process first, because a driver
    that is half installed can fault inside dlopen and that must not take the caller
    down (lmz/gpu/__init__.py:39-95) -> open it here and compare ABI versions ->
    decode a batch whose plaintext is known (lmz/gpu/__init__.py:164-207)."""

    def __init__(self):
        self.lock = threading.Lock()
        self.lib = None
        self.status = "unloaded"          # unloaded | disabled | unavailable | abi-mismatch | cuda:<device>
        self.reason = "not probed"

    def get(self):
        if self.status == "unloaded":
            with self.lock:
                if self.status == "unloaded":
                    try:
                        self._attempt()
                    except Exception as exc:          # nothing here may reach the caller
                        self._give_up("unavailable", f"{type(exc).__name__}: {exc}")
        return self.lib

    def _give_up(self, status: str, reason: str) -> None:
        self.lib, self.status, self.reason = None, status, reason

    def _attempt(self) -> None:
        if os.environ.get("LMZ_NO_GPU"):
            return self._give_up("disabled", "disabled by LMZ_NO_GPU")
        from . import build
        path = build.build()
        if not path:
            return self._give_up("unavailable", build.last_error or "the CUDA decoder did not build")
        device, problem = _ask_child(path)
        if problem:
            return self._give_up("unavailable", problem)
        lib = ctypes.CDLL(path)
        lib.lmz_gpu_abi_version.restype = ctypes.c_int
        if lib.lmz_gpu_abi_version() != ABI_VERSION:
            return self._give_up("abi-mismatch", "the built CUDA decoder is from another source")
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        from . import _chunks
        _chunks.bind(lib)
        if not _known_answer(lib):
            return self._give_up("unavailable", f"the CUDA decoder did not reproduce the known "
                                                f"plaintext on {device}; refusing to use it")
        self.lib, self.status, self.reason = lib, "cuda:" + device, ""


def _ask_child(path: str):
    """(device name, None), or (None, why the library must not be loaded here)."""
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_probe.py")
    try:
        child = subprocess.run([sys.executable, script, path], capture_output=True, text=True,
                               timeout=120)
    except subprocess.TimeoutExpired:
        return None, "the CUDA driver did not answer within 120s"
    except OSError as exc:
        return None, f"could not probe the CUDA driver: {exc}"
    if child.returncode != 0:
        how = f"signal {-child.returncode}" if child.returncode < 0 else f"status {child.returncode:#x}"
        return None, f"the CUDA driver crashed while loading ({how})"
    try:
        said = json.loads(child.stdout.strip().splitlines()[-1])
    except (ValueError, IndexError):
        return None, "the probe process gave no answer"
    if said.get("abi") is None:
        return None, said.get("error") or "the library did not load"
    if said["abi"] != ABI_VERSION:
        return None, "the built CUDA decoder is from another source"
    if said.get("rc") != OK:
        return None, "no CUDA device" if said.get("rc") == ENODEV else (said.get("error") or "no CUDA device")
    return said["device"], None


_loader = _Loader()


def library():
    """The loaded ctypes library, or raise: for callers that cannot go on without it."""
    lib = _loader.get()
    if lib is None:
        raise RuntimeError(f"the lmz_b200 CUDA library is unavailable: {_loader.reason}")
    return lib


def loaded_library():
    """The library if an earlier call has loaded it, else None.  Never probes."""
    return _loader.lib


def _host_view(buf, writable: bool = False):
    """A numpy uint8 view of a host buffer (bytes, bytearray, memoryview, array) whose
    `.ctypes.data` is the buffer's address; the view keeps the buffer alive."""
    import numpy as np
    if buf is None:
        return None
    arr = np.frombuffer(buf, dtype=np.uint8)
    if writable and not arr.flags.writeable:
        raise ValueError("the output buffer is read-only")
    return arr


def _addr(view):
    return view.ctypes.data if view is not None and view.size else None


# The load-time check: five ragged planes of 203 bytes (not a multiple of the 8 lanes),
# one of them a single repeated symbol, whose plaintext is a closed formula.
def _known_planes():
    import numpy as np
    i = np.arange(203, dtype=np.uint32)
    rows = [((i * 37 + r * 11) % 23).astype(np.uint8) if r != 2 else np.full(203, 0x40, np.uint8)
            for r in range(5)]
    rows[4] = np.where(i % 3 == 0, 0x40, rows[4]).astype(np.uint8)
    return np.stack(rows)


def _known_answer(lib) -> bool:
    import numpy as np

    from . import _streams
    planes = _known_planes()
    blob, table = _streams.pack(_streams.encode_batch(planes))
    src, offs = _host_view(blob), _host_view(table)
    got = np.zeros(planes.size, dtype=np.uint8)
    rc = lib.lmz_gpu_decode_batch(None, _addr(src), src.size, _addr(offs), planes.shape[0],
                                  planes.shape[1], _addr(got))
    if rc in (ENODEV, EUNSUPPORTED, ECUDA):
        return True                  # the device declined; nothing wrong was decoded
    return rc == OK and np.array_equal(got, planes.reshape(-1))


def available() -> tuple[bool, str]:
    """Whether the GPU decoder can run, and if not, the reason."""
    return (_loader.get() is not None), _loader.reason


def state() -> str:
    """What is known without probing (lmz/gpu/__init__.py:220-226)."""
    return "not probed" if _loader.status == "unloaded" else _loader.status


def backend() -> str:
    return _loader.status if _loader.get() is not None else "unavailable"


def last_error() -> str:
    lib = _loader.get()
    return _loader.reason if lib is None else (lib.lmz_gpu_last_error() or b"").decode(errors="replace")


def grain() -> int:
    """A plane must be a multiple of this; 1 here (the reference's is 128)."""
    lib = _loader.get()
    return lib.lmz_gpu_grain() if lib is not None else 1


def header_bytes() -> int:
    lib = _loader.get()
    return lib.lmz_gpu_header_bytes() if lib is not None else 516


def pad_bytes() -> int:
    lib = _loader.get()
    return lib.lmz_gpu_pad_bytes() if lib is not None else 576


def _is_cuda_tensor(x) -> bool:
    return type(x).__module__.startswith("torch") and getattr(x, "is_cuda", False)


def decode_batch(streams, offsets, nstr: int, plane: int, out=None, header=None):
    """Decode `nstr` lmz rANS streams to `plane` bytes each. None if unavailable.

    Arguments as lmz/gpu/__init__.py:380-428: `streams` are the streams back
    to back exactly as an archive stores them, `offsets` is 2*nstr
    little-endian uint64 (byte offset, byte length), `header` an optional
    516-byte table shared by the batch.  Returns nstr*plane bytes
    (memoryview), None when there is no usable GPU decoder, and raises
    ValueError for arguments that make no sense or a stream that is not valid
    lmz rANS (bad magic, frequencies that do not sum to 4096, truncated, or
    lying outside `streams`).

    With a CUDA uint8 tensor for `streams` the decode runs device to device
    and a CUDA tensor comes back; `offsets` may then be bytes or a CUDA int64
    tensor of 2*nstr values."""
    lib = _loader.get()
    if lib is None:
        return None
    if nstr == 0:
        return memoryview(b"")
    if nstr < 0:
        raise ValueError("nstr is negative")
    if plane < 1:
        raise ValueError("plane must be at least 1")
    if header is not None and len(header) != header_bytes():
        raise ValueError(f"a shared table is {header_bytes()} bytes, not {len(header)}")
    if _is_cuda_tensor(streams):
        return _decode_batch_cuda(lib, streams, offsets, nstr, plane, out, header)
    table = _host_view(offsets)
    if table.size < 16 * nstr:
        raise ValueError(f"offsets holds {table.size} bytes, need {nstr * 16}")
    src, shared = _host_view(streams), _host_view(header)
    size = nstr * plane
    if out is not None and len(out) >= size:
        held, dst = out, _host_view(out, writable=True)
    else:
        held = bytearray(size)
        dst = _host_view(held)
    rc = lib.lmz_gpu_decode_batch(_addr(shared), _addr(src), src.size, _addr(table), nstr, plane,
                                  _addr(dst))
    if rc == EBADSTREAM:
        raise ValueError("malformed rANS stream")
    return memoryview(held)[:size] if rc == OK else None


def _decode_batch_cuda(lib, streams, offsets, nstr, plane, out, header):
    """Device-to-device decode with per-stream verdicts.  The offset table is checked
    against the buffer before anything is launched, and the kernels report bad magic, bad
    frequency sums and truncation per stream, so hostile input ends in ValueError."""
    import torch

    dev = streams.device
    with torch.cuda.device(dev):
        flat = streams.reshape(-1)
        pad = pad_bytes()
        if _is_cuda_tensor(offsets):
            offs = offsets.reshape(-1).view(torch.int64)
        else:
            table = _host_view(offsets)
            if table.size < 16 * nstr:
                raise ValueError(f"offsets holds {table.size} bytes, need {nstr * 16}")
            offs = torch.frombuffer(bytearray(table[:16 * nstr]), dtype=torch.int64).to(dev)
        if offs.numel() < 2 * nstr:
            raise ValueError("offsets is too short")
        pairs = offs[:2 * nstr].reshape(nstr, 2)
        start, length = pairs[:, 0], pairs[:, 1]
        inside = (start >= 0) & (length >= 0) & (length < (1 << 32)) & (start <= flat.numel()) & \
                 (length <= flat.numel() - start)
        if not bool(inside.all()):
            raise ValueError("a stream lies outside the buffer")
        buf = torch.empty(flat.numel() + pad, dtype=torch.uint8, device=dev)
        buf[:flat.numel()].copy_(flat)
        buf[flat.numel():].zero_()
        hdr = None
        if header is not None:
            hdr = header if _is_cuda_tensor(header) else \
                torch.frombuffer(bytearray(header), dtype=torch.uint8).to(dev)
        size = nstr * plane
        dst = out if (out is not None and _is_cuda_tensor(out) and out.numel() >= size) \
            else torch.empty(size, dtype=torch.uint8, device=dev)
        # one 32-byte job per stream (include/lmz_b200.h, lmz_stream_job): source offset,
        # destination offset, then length and symbol count packed into the third word
        jobs = torch.zeros((nstr, 4), dtype=torch.int64, device=dev)
        jobs[:, 0] = start
        jobs[:, 1] = torch.arange(nstr, dtype=torch.int64, device=dev) * plane
        jobs[:, 2] = length | (plane << 32)
        verdicts = torch.zeros(nstr + 1, dtype=torch.int32, device=dev)      # [nstr] = any bad
        cs = torch.cuda.current_stream(dev)
        rc = lib.lmz_gpu_decode_streams_dev(jobs.data_ptr(), nstr, buf.data_ptr(), dst.data_ptr(),
                                            hdr.data_ptr() if hdr is not None else None,
                                            verdicts.data_ptr(), verdicts[nstr:].data_ptr(),
                                            cs.cuda_stream)
        if rc != OK:
            return None
        cs.synchronize()             # also keeps the inputs alive until the kernels have read them
        if int(verdicts[nstr].item()) != 0:
            raise ValueError("malformed rANS stream")
        return dst[:size]


def encode_batch(planes, nstr: int, plane: int):
    """The inverse of `decode_batch` (the reference has no GPU encoder; its CPU one is
    lmz/kernels.py rans_encode over lmz/native/lmzcore.c:1318-1383): code `nstr` planes
    of `plane` bytes, each with its own histogram.  Returns (streams, offsets) in the
    layout `decode_batch` takes - the streams back to back and 2*nstr little-endian
    uint64 (byte offset, byte length) - and every stream is byte-identical to what the
    reference's encoder writes for that plane.  Host bytes in, bytes out; a CUDA uint8
    tensor in, CUDA tensors out (uint8 streams with pad_bytes() of zeroed slack after
    them, int64 offsets).  None if there is no usable GPU library."""
    lib = _loader.get()
    if lib is None:
        return None
    if nstr < 0 or plane < 1:
        raise ValueError("nstr must not be negative and plane must be at least 1")
    import torch

    on_device = _is_cuda_tensor(planes)
    if not on_device and len(planes) < nstr * plane:
        raise ValueError(f"planes holds {len(planes)} bytes, need {nstr * plane}")
    if nstr == 0:
        return (torch.empty(0, dtype=torch.uint8, device=planes.device),
                torch.empty(0, dtype=torch.int64, device=planes.device)) if on_device else (b"", b"")
    dev = planes.device if on_device else torch.device(f"cuda:{torch.cuda.current_device()}")
    with torch.cuda.device(dev):
        src = planes.reshape(-1) if on_device else \
            torch.frombuffer(bytearray(planes[:nstr * plane]), dtype=torch.uint8).to(dev)
        if src.numel() < nstr * plane:
            raise ValueError("planes is too short")
        slot = lib.lmz_gpu_encode_slot_bytes(plane)
        if slot <= 0:
            raise ValueError("plane must be at most 2^29 bytes")
        slots = torch.empty(nstr * slot, dtype=torch.uint8, device=dev)       # the allocator aligns to 512
        lens = torch.zeros(nstr, dtype=torch.int32, device=dev)
        cs = torch.cuda.current_stream(dev).cuda_stream
        rc = lib.lmz_gpu_encode_batch_dev(src.data_ptr(), nstr, plane, slots.data_ptr(), lens.data_ptr(), cs)
        if rc != OK:
            return None
        lens64 = lens.to(torch.int64)
        if bool((lens64 == 0).any()):
            raise ValueError("a plane could not be coded")
        offs = torch.stack((torch.cumsum(lens64, 0) - lens64, lens64), dim=1).reshape(-1).contiguous()
        total = int(lens64.sum())
        out = torch.zeros(total + pad_bytes(), dtype=torch.uint8, device=dev)
        rc = lib.lmz_gpu_pack_streams_dev(slots.data_ptr(), plane, offs.data_ptr(), nstr, out.data_ptr(), cs)
        if rc != OK:
            return None
        torch.cuda.current_stream(dev).synchronize()
        if on_device:
            return out[:total], offs
        return out[:total].cpu().numpy().tobytes(), offs.cpu().numpy().astype("<u8").tobytes()


# Byte-value distributions that break frequency tables, as 256-entry translate() tables
# over uniform random bytes (the five of lmz/gpu/__init__.py:272-278).
def _runs(*pieces) -> bytes:
    """Concatenate (value or range of values, repeat count) pieces into a byte table."""
    return b"".join(bytes([v] if isinstance(v, int) else v) * n for v, n in pieces)


_AWKWARD = {
    "single symbol": _runs((0x5A, 256)),
    "two symbols": _runs((0x01, 128), (0xFE, 128)),
    "near uniform": _runs((range(256), 1)),
    "dominant + tail": _runs((0x20, 250), (range(6), 1)),
    "skewed": _runs((0x40, 170), (range(16), 5), (0x7F, 6)),
}
assert all(len(t) == 256 for t in _AWKWARD.values())


def _shaped_batch(name: str, plane: int, nstr: int, seed: int):
    """`nstr` planes of `plane` bytes drawn from the named distribution, and their streams."""
    import numpy as np

    from . import _streams
    raw = np.random.default_rng(seed).integers(0, 256, plane * nstr, dtype=np.uint8)
    lut = np.frombuffer(_AWKWARD[name], dtype=np.uint8)
    planes = lut[raw].reshape(nstr, plane)
    blob, table = _streams.pack(_streams.encode_batch(planes))
    return planes, blob, table


def verify(quick: bool = False) -> dict:
    """Decode every awkward shape on this device and check the plaintext comes
    back (lmz/gpu/__init__.py:281-361).  Streams are built by this package's
    own encoder, so the check needs no data files.  Keys: lmz, device, ok,
    checked, failures, gbps, why."""
    import itertools
    import time

    from . import __version__

    usable, why = available()
    report = {"lmz": __version__, "device": backend().removeprefix("cuda:") if usable else None,
              "ok": False, "checked": 0, "failures": [], "gbps": None, "why": "" if usable else why}
    if not usable:
        return report

    def trial(name, plane, nstr, seed):
        """None when the batch decodes to its plaintext, else what went wrong."""
        planes, blob, table = _shaped_batch(name, plane, nstr, seed)
        try:
            got = decode_batch(blob, table, nstr, plane)
        except ValueError as exc:
            return str(exc)
        if got is None:
            return f"declined -- {last_error()}"
        return None if bytes(got) == planes.tobytes() else "output differs"

    sizes = (4096,) if quick else (1, 17, 128, 4096)
    for seed, (name, plane, nstr) in enumerate(itertools.product(_AWKWARD, sizes, (1, 17, 129))):
        problem = trial(name, plane, nstr, 7000 + seed)
        if problem is None:
            report["checked"] += 1
        else:
            report["failures"].append(f"{name} plane={plane} n={nstr}: {problem}")

    # a host round trip of one larger batch, timed on its second run
    plane, nstr = (4096, 256) if quick else (32768, 512)
    planes, blob, table = _shaped_batch("skewed", plane, nstr, 4242)
    sink = bytearray(nstr * plane)
    decode_batch(blob, table, nstr, plane, out=sink)
    t0 = time.perf_counter()
    got = decode_batch(blob, table, nstr, plane, out=sink)
    elapsed = time.perf_counter() - t0
    if got is None or bytes(sink) != planes.tobytes():
        report["failures"].append("throughput batch did not decode correctly")
    elif elapsed > 0:
        report["gbps"] = round(nstr * plane / elapsed / 1e9, 2)
    report["ok"] = report["checked"] > 0 and not report["failures"]
    return report
