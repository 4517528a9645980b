"""The reference's own, unmodified `lmz.gpu` module bound to this library.

INTEGRATION.md's stub is one line: the reference's build step returns the path of
liblmz_b200.so instead of compiling lmz/gpu/lmzgpu.cu.  This test applies exactly that in a
child process and lets the reference's loader run (lmz/gpu/__init__.py:102-161): its
crash-safe probe process dlopens the library, checks `lmz_gpu_abi_version()` and asks for
the device name through its own ctypes declarations.  Without a GPU the answer has to be the
loader's "no CUDA device" verdict -- not an ABI mismatch, not a missing symbol, not a crash;
with one, the reference's known-answer self-test (:164-207) must accept this library's
output.  Skipped where the reference tree is absent (it cannot travel with this repository).
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes, json, sys
ref, lib_path, core = sys.argv[1:4]
sys.path.insert(0, ref)
import lmz.native.build as nb
nb.build = lambda *a, **k: core                      # the reference's C core, compiled out of tree
import lmz.gpu.build as gb
gb.build = lambda *a, **k: lib_path                  # the one-line stub of INTEGRATION.md
import lmz.gpu as g
ok, why = g.available()
out = {"ok": ok, "why": why, "state": g.state(), "backend": g.backend()}
if ok:
    rep = g.verify(quick=True)
    out["verify"] = {k: rep[k] for k in ("ok", "checked", "failures")}
lib = ctypes.CDLL(lib_path)                          # every export the reference declares (:130-148)
out["exports"] = all(hasattr(lib, n) for n in (
    "lmz_gpu_abi_version", "lmz_gpu_last_error", "lmz_gpu_grain", "lmz_gpu_header_bytes", "lmz_gpu_pad_bytes",
    "lmz_gpu_device_name", "lmz_gpu_validate", "lmz_gpu_decode_batch_dev", "lmz_gpu_decode_batch"))
print(json.dumps(out))
"""


def test_unmodified_reference_module_loads_this_library():
    import json
    tree = os.environ.get("LMZ_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    core = os.path.join(ROOT, "oracle", "_ref", "liblmzcore.so")
    if not os.path.exists(os.path.join(tree, "lmz", "gpu", "__init__.py")) or not os.path.exists(core):
        pytest.skip("the reference tree is not on this machine")
    from lmz_b200 import build
    lib = build.build()
    assert lib, build.last_error
    done = subprocess.run([sys.executable, "-c", CHILD, tree, lib, core], capture_output=True, text=True,
                          env={k: v for k, v in os.environ.items() if k != "LMZ_NO_GPU"})
    assert done.returncode == 0, done.stderr[-800:]
    said = json.loads(done.stdout.strip().splitlines()[-1])
    assert said["exports"]
    if said["ok"]:                                   # a GPU is present: the reference's own checks ran on it
        assert said["state"].startswith("cuda:") and said["verify"]["ok"], said
    else:                                            # no GPU: the loader got as far as asking for a device
        assert "no CUDA device" in said["why"], said
        assert said["state"] == "unavailable" and said["backend"] == "unavailable"
