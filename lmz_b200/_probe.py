"""First touch of the CUDA driver, in a process that may die.

Run as a script: `python _probe.py <library path>`.  Loads the library, asks it for
its ABI version and the current device's name, and prints one JSON object.  The
parent (`gpu._Loader`) reads that line; a child that was killed instead of answering
tells the parent that loading the driver is not safe in its own process -- the
reason the reference probes in a child too (lmz/gpu/__init__.py:39-95).
"""
import ctypes
import json
import sys


def main(path: str) -> int:
    answer = {"abi": None, "device": None, "rc": None, "error": None}
    try:
        lib = ctypes.CDLL(path)
        lib.lmz_gpu_abi_version.restype = ctypes.c_int
        answer["abi"] = int(lib.lmz_gpu_abi_version())
        name = ctypes.create_string_buffer(256)
        lib.lmz_gpu_device_name.restype = ctypes.c_int
        lib.lmz_gpu_device_name.argtypes = [ctypes.c_char_p, ctypes.c_int]
        answer["rc"] = int(lib.lmz_gpu_device_name(name, len(name)))
        if answer["rc"] == 0:
            answer["device"] = name.value.decode(errors="replace")
        else:
            lib.lmz_gpu_last_error.restype = ctypes.c_char_p
            answer["error"] = (lib.lmz_gpu_last_error() or b"").decode(errors="replace")
    except Exception as exc:                       # OSError from dlopen, missing symbols ...
        answer["error"] = f"{type(exc).__name__}: {exc}"
    print(json.dumps(answer))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
