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
import os
import subprocess
import sys
import threading

__all__ = ["available", "backend", "decode_batch", "grain", "header_bytes",
           "last_error", "pad_bytes", "state", "verify"]

ABI_VERSION = 1                      # lmz/gpu/__init__.py:31
OK, ENODEV, EUNSUPPORTED, EBADSTREAM, ECUDA, EMISMATCH = 0, -1, -2, -3, -4, -5

# The first touch of the driver happens in a child that is allowed to die
# (lmz/gpu/__init__.py:39-95): a half-installed driver can fault inside
# dlopen, and that must not take the caller's process with it.
_PROBE_SOURCE = """
import ctypes, sys
try:
    lib = ctypes.CDLL(sys.argv[1])
    lib.lmz_gpu_abi_version.restype = ctypes.c_int
    if lib.lmz_gpu_abi_version() != ABI:
        sys.exit(2)
    lib.lmz_gpu_device_name.restype = ctypes.c_int
    lib.lmz_gpu_device_name.argtypes = [ctypes.c_char_p, ctypes.c_int]
    buf = ctypes.create_string_buffer(256)
    if lib.lmz_gpu_device_name(buf, 256) != 0:
        sys.exit(3)
    sys.stdout.write(buf.value.decode())
except Exception as exc:
    sys.stderr.write(f"{type(exc).__name__}: {exc}")
    sys.exit(4)
"""


def _probe_elsewhere(path: str) -> tuple[bool, str]:
    src = _PROBE_SOURCE.replace("ABI", str(ABI_VERSION))
    try:
        p = subprocess.run([sys.executable, "-c", src, path], capture_output=True,
                           text=True, timeout=120)
    except subprocess.TimeoutExpired:
        return False, "the CUDA driver did not answer within 120s"
    except Exception as exc:
        return False, f"could not probe the CUDA driver: {exc}"
    if p.returncode == 0:
        return True, p.stdout.strip()
    if p.returncode == 2:
        return False, "the built CUDA decoder is from another source"
    if p.returncode == 3:
        return False, "no CUDA device"
    if p.returncode == 4:
        return False, (p.stderr.strip().splitlines() or ["the library did not load"])[-1]
    sig = f"signal {-p.returncode}" if p.returncode < 0 else f"status {p.returncode:#x}"
    return False, f"the CUDA driver crashed while loading ({sig})"


_lock = threading.Lock()
_lib = None
_state = "unloaded"
_why = "not probed"


def _bind(lib) -> None:
    v, c_int, c_uint = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
    for name in ("lmz_gpu_abi_version", "lmz_gpu_grain", "lmz_gpu_header_bytes",
                 "lmz_gpu_pad_bytes"):
        getattr(lib, name).restype = c_int
    lib.lmz_gpu_device_name.restype = c_int
    lib.lmz_gpu_device_name.argtypes = [ctypes.c_char_p, c_int]
    lib.lmz_gpu_last_error.restype = ctypes.c_char_p
    lib.lmz_gpu_validate.restype = c_int
    lib.lmz_gpu_validate.argtypes = [v, v, c_uint]
    lib.lmz_gpu_decode_batch.restype = c_int
    lib.lmz_gpu_decode_batch.argtypes = [v, v, ctypes.c_size_t, v, c_uint, c_uint, v]
    lib.lmz_gpu_decode_batch_dev.restype = c_int
    lib.lmz_gpu_decode_batch_dev.argtypes = [v, v, v, c_uint, c_uint, v, v, c_uint]
    lib.lmz_gpu_set_device.restype = c_int
    lib.lmz_gpu_set_device.argtypes = [c_int]
    lib.lmz_gpu_set_table_mode.restype = c_int
    lib.lmz_gpu_set_table_mode.argtypes = [c_int]
    lib.lmz_gpu_decode_streams_dev.restype = c_int
    lib.lmz_gpu_decode_streams_dev.argtypes = [v, c_uint, v, v, v, v, v, v]
    lib.lmz_gpu_encode_slot_bytes.restype = c_int
    lib.lmz_gpu_encode_slot_bytes.argtypes = [c_uint]
    lib.lmz_gpu_encode_batch_dev.restype = c_int
    lib.lmz_gpu_encode_batch_dev.argtypes = [v, c_uint, c_uint, v, v, v]
    lib.lmz_gpu_pack_streams_dev.restype = c_int
    lib.lmz_gpu_pack_streams_dev.argtypes = [v, c_uint, v, c_uint, v, v]
    from . import _chunks
    _chunks.bind(lib)


def _load():
    global _lib, _state, _why
    if _state != "unloaded":
        return _lib
    with _lock:
        if _state != "unloaded":
            return _lib
        if os.environ.get("LMZ_NO_GPU"):
            _state, _why = "disabled", "disabled by LMZ_NO_GPU"
            return None
        try:
            from . import build as _build

            path = _build.build()
            if not path:
                _state = "unavailable"
                _why = _build.last_error or "the CUDA decoder did not build"
                return None
            safe, probed = _probe_elsewhere(path)
            if not safe:
                _state, _why = "unavailable", probed
                return None
            lib = ctypes.CDLL(path)
            lib.lmz_gpu_abi_version.restype = ctypes.c_int
            if lib.lmz_gpu_abi_version() != ABI_VERSION:
                _state, _why = "abi-mismatch", "the built CUDA decoder is from another source"
                return None
            _bind(lib)
            if not _selftest(lib):
                _state = "unavailable"
                _why = (f"the CUDA decoder did not reproduce the known plaintext on "
                        f"{probed}; refusing to use it")
                return None
            _lib = lib
            _state = "cuda:" + probed
            _why = ""
        except Exception as exc:
            _lib = None
            _state, _why = "unavailable", f"{type(exc).__name__}: {exc}"
    return _lib


def library():
    """The loaded ctypes library, or raise: for callers that cannot go on without it."""
    lib = _load()
    if lib is None:
        raise RuntimeError(f"the lmz_b200 CUDA library is unavailable: {_why}")
    return lib


def _selftest_plain() -> bytes:
    return bytes(((i * 37) & 0x0F) if i % 3 else 0x40 for i in range(128))


def _selftest(lib) -> bool:
    """Decode a batch whose answer is known before trusting the device
    (lmz/gpu/__init__.py:164-207: 8 copies of a 128-byte skewed plane)."""
    import struct

    import numpy as np

    from . import _streams

    plain = _selftest_plain()
    coded = _streams.encode_batch(np.frombuffer(plain, dtype=np.uint8)[None, :])[0]
    nstr, plane = 8, len(plain)
    streams, offsets = bytearray(), bytearray()
    for _ in range(nstr):
        offsets += struct.pack("<QQ", len(streams), len(coded))
        streams += coded
    out = bytearray(nstr * plane)
    s_addr, _a = _ptr(streams)
    o_addr, _b = _ptr(bytes(offsets))
    d_addr, _c = _ptr(out)
    rc = lib.lmz_gpu_decode_batch(None, s_addr, len(streams), o_addr, nstr, plane, d_addr)
    if rc != OK:
        return rc not in (EBADSTREAM, EMISMATCH)
    return bytes(out) == plain * nstr


def available() -> tuple[bool, str]:
    """Whether the GPU decoder can run, and if not, the reason."""
    _load()
    return (_lib is not None), _why


def state() -> str:
    """What is known without probing (lmz/gpu/__init__.py:220-226)."""
    return _state if _state != "unloaded" else "not probed"


def backend() -> str:
    _load()
    return _state if _lib is not None else "unavailable"


def last_error() -> str:
    lib = _load()
    if lib is None:
        return _why
    return lib.lmz_gpu_last_error().decode(errors="replace")


def _const(name: str, default: int) -> int:
    lib = _load()
    return getattr(lib, name)() if lib is not None else default


def grain() -> int:
    """A plane must be a multiple of this; 1 here (the reference's is 128)."""
    return _const("lmz_gpu_grain", 1)


def header_bytes() -> int:
    return _const("lmz_gpu_header_bytes", 516)


def pad_bytes() -> int:
    return _const("lmz_gpu_pad_bytes", 576)


def _ptr(obj):
    """Address of a host buffer plus a reference that must outlive the call."""
    if obj is None or len(obj) == 0:
        return None, None
    if type(obj) is bytes:
        p = ctypes.c_char_p(obj)
        return ctypes.cast(p, ctypes.c_void_p).value, (p, obj)
    try:
        arr = (ctypes.c_ubyte * len(obj)).from_buffer(obj)
        return ctypes.addressof(arr), arr
    except TypeError:
        b = bytes(obj)
        p = ctypes.c_char_p(b)
        return ctypes.cast(p, ctypes.c_void_p).value, (p, b)


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
    lmz rANS.

    With a CUDA uint8 tensor for `streams` the decode runs device to device
    and a CUDA tensor comes back; `offsets` may then be bytes or a CUDA int64
    tensor of 2*nstr values."""
    lib = _load()
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
    if len(offsets) < nstr * 16:
        raise ValueError(f"offsets holds {len(offsets)} bytes, need {nstr * 16}")

    need = nstr * plane
    dst = out if (out is not None and len(out) >= need) else bytearray(need)
    s_addr, _a = _ptr(streams)
    o_addr, _b = _ptr(offsets)
    d_addr, _c = _ptr(dst)
    h_addr, _d = _ptr(header)
    rc = lib.lmz_gpu_decode_batch(h_addr, s_addr, len(streams), o_addr, nstr, plane, d_addr)
    if rc == OK:
        return memoryview(dst)[:need]
    if rc == EBADSTREAM:
        raise ValueError("malformed rANS stream")
    return None


def encode_batch(planes, nstr: int, plane: int):
    """The inverse of `decode_batch` (the reference has no GPU encoder; its CPU one is
    lmz/kernels.py rans_encode over lmz/native/lmzcore.c:1318-1383): code `nstr` planes
    of `plane` bytes, each with its own histogram.  Returns (streams, offsets) in the
    layout `decode_batch` takes - the streams back to back and 2*nstr little-endian
    uint64 (byte offset, byte length) - and every stream is byte-identical to what the
    reference's encoder writes for that plane.  Host bytes in, bytes out; a CUDA uint8
    tensor in, CUDA tensors out (uint8 streams with pad_bytes() of zeroed slack after
    them, int64 offsets).  None if there is no usable GPU library."""
    lib = _load()
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


def _decode_batch_cuda(lib, streams, offsets, nstr, plane, out, header):
    import torch

    dev = streams.device
    with torch.cuda.device(dev):
        pad = pad_bytes()
        buf = torch.empty(streams.numel() + pad, dtype=torch.uint8, device=dev)
        buf[:streams.numel()].copy_(streams.reshape(-1))
        buf[streams.numel():].zero_()
        if _is_cuda_tensor(offsets):
            offs = offsets.reshape(-1).view(torch.int64)
        else:
            if len(offsets) < nstr * 16:
                raise ValueError(f"offsets holds {len(offsets)} bytes, need {nstr * 16}")
            offs = torch.frombuffer(bytearray(offsets[:nstr * 16]), dtype=torch.int64).to(dev)
        if offs.numel() < 2 * nstr:
            raise ValueError("offsets is too short")
        hdr = None
        if header is not None:
            hdr = header if _is_cuda_tensor(header) else \
                torch.frombuffer(bytearray(header), dtype=torch.uint8).to(dev)
        need = nstr * plane
        dst = out if (out is not None and _is_cuda_tensor(out) and out.numel() >= need) \
            else torch.empty(need, dtype=torch.uint8, device=dev)
        cs = torch.cuda.current_stream(dev).cuda_stream
        rc = lib.lmz_gpu_decode_batch_dev(hdr.data_ptr() if hdr is not None else None,
                                          buf.data_ptr(), offs.data_ptr(), nstr, plane,
                                          dst.data_ptr(), cs, 0)
        if rc == OK:
            # The inputs must stay alive until the kernel has read them.
            torch.cuda.current_stream(dev).synchronize()
            return dst[:need]
        if rc == EBADSTREAM:
            raise ValueError("malformed rANS stream")
        return None


# Byte-value distributions that break frequency tables, as translate() tables
# over uniform random bytes (lmz/gpu/__init__.py:272-278).
_SHAPES = {
    "single symbol": bytes([0x5A]) * 256,
    "two symbols": bytes([0x01]) * 128 + bytes([0xFE]) * 128,
    "near uniform": bytes(range(256)),
    "dominant + tail": bytes([0x20]) * 250 + bytes(range(6)),
    "skewed": bytes([0x40]) * 170 + bytes(range(16)) * 5 + bytes([0x7F]) * 6,
}


def verify(quick: bool = False) -> dict:
    """Decode every awkward shape on this device and check the plaintext comes
    back (lmz/gpu/__init__.py:281-361).  Streams are built by this package's
    own encoder, so the check needs no data files."""
    import random
    import time

    import numpy as np

    from . import __version__, _streams

    report = {"lmz": __version__, "device": None, "ok": False, "checked": 0,
              "failures": [], "gbps": None, "why": ""}
    ok, why = available()
    if not ok:
        report["why"] = why
        return report
    report["device"] = backend().removeprefix("cuda:")

    def batch(table, plane, nstr, seed):
        rnd = random.Random(seed)
        raw = np.frombuffer(rnd.randbytes(plane * nstr), dtype=np.uint8)
        bufs = np.frombuffer(raw.tobytes().translate(table), dtype=np.uint8).reshape(nstr, plane)
        streams, offsets = _streams.pack(_streams.encode_batch(bufs))
        return bufs, streams, offsets

    planes = (4096,) if quick else (1, 17, 128, 4096)
    for name, table in _SHAPES.items():
        for plane in planes:
            for nstr in (1, 17, 129):
                bufs, streams, offsets = batch(table, plane, nstr, hash((name, plane, nstr)) & 0xFFFF)
                try:
                    out = decode_batch(streams, offsets, nstr, plane)
                except ValueError as exc:
                    report["failures"].append(f"{name} plane={plane} n={nstr}: {exc}")
                    continue
                if out is None:
                    report["failures"].append(
                        f"{name} plane={plane} n={nstr}: declined -- {last_error()}")
                    continue
                if bytes(out) != bufs.tobytes():
                    report["failures"].append(f"{name} plane={plane} n={nstr}: output differs")
                report["checked"] += 1

    plane, nstr = (4096, 256) if quick else (32768, 512)
    bufs, streams, offsets = batch(_SHAPES["skewed"], plane, nstr, 4242)
    out = bytearray(nstr * plane)
    decode_batch(streams, offsets, nstr, plane, out=out)
    t = time.perf_counter()
    got = decode_batch(streams, offsets, nstr, plane, out=out)
    dt = time.perf_counter() - t
    if got is not None and dt > 0:
        report["gbps"] = round(nstr * plane / dt / 1e9, 2)
    if got is None or bytes(out) != bufs.tobytes():
        report["failures"].append("throughput batch did not decode correctly")
    report["ok"] = report["checked"] > 0 and not report["failures"]
    return report
