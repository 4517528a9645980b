"""Compress files with the REFERENCE's own `lmz.api.compress`, unmodified.

    python tests/golden/ref_compress.py <reference tree> <source file or directory> <archive> [json options]

Test infrastructure: `tests/test_oracle_vs_reference.py` runs this in a child process
(so the reference's package never enters the test process) and holds the checker's
archive writer to the bytes it produces.  The one shim is the same as in
make_golden.py: the reference's native-core loader is pointed at oracle/_ref/liblmzcore.so,
its own C source compiled out of tree because the reference tree is read-only.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(ref: str, src: str, dst: str, options: str = "{}") -> int:
    sys.path.insert(0, ref)
    import lmz.native.build as nb
    nb.build = lambda *a, **k: os.path.join(ROOT, "oracle", "_ref", "liblmzcore.so")
    from lmz import api, kernels
    assert kernels.backend().startswith("native"), kernels.backend()
    kw = json.loads(options)
    kw.setdefault("workers", os.cpu_count() or 1)
    if os.path.exists(dst):
        os.unlink(dst)
    api.compress(src, dst, **kw)
    return 0


if __name__ == "__main__":
    sys.exit(main(*sys.argv[1:5]))
