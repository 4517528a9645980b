"""Generate the golden fixtures in this directory with the REFERENCE itself.

Run where the reference tree is available and oracle/_ref has been built from it:

    LMZ_REFERENCE=/path/to/lmz python tests/golden/make_golden.py

The reference's Python is imported unmodified; the only shim is that its
native-core loader is pointed at oracle/_ref/liblmzcore.so (the same C source
compiled with the same flags, out of tree because the reference tree is
read-only).  Outputs:

  rans_vectors.npz   plaintexts and the streams `lmz.kernels.rans_encode` wrote
                     for them, over the reference tests' adversarial shapes
  *.lmz              archives written by `lmz.api.compress`
  manifest.json      for each archive: options, size and sha256 of the
                     plaintext `lmz.api.decompress` restored, per-chunk codecs
"""
import hashlib
import json
import os
import shutil
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("LMZ_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
if not os.path.exists(os.path.join(REF, "lmz", "api.py")):
    raise SystemExit("set LMZ_REFERENCE to the reference checkout")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)

import lmz.native.build as _nb  # noqa: E402

_nb.build = lambda *a, **k: os.path.join(ROOT, "oracle", "_ref", "liblmzcore.so")
import lmz  # noqa: E402
from lmz import api, kernels  # noqa: E402

from oracle import synth  # noqa: E402

assert kernels.backend().startswith("native"), kernels.backend()


def lcg(n, seed):
    out, x = bytearray(), seed | 1
    while len(out) < n:
        x = (x * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out += x.to_bytes(8, "little")
    return bytes(out[:n])


def cond_bf16(nelem, seed):
    """BF16 whose mantissa alphabet narrows with the exponent, so the conditioned
    codec wins (the shape of the reference's own fixture, tests/test_lmz.py:84-100)."""
    rng = np.random.default_rng(seed)
    exp = (118 + rng.integers(0, 6, nelem)).astype(np.uint16)
    mant = rng.integers(0, 128, nelem).astype(np.uint16)
    mant = np.where(exp >= 121, mant & 0x03, mant & 0x1F)
    sign = rng.integers(0, 2, nelem).astype(np.uint16)
    return ((sign << 15) | (exp << 7) | mant).astype("<u2").view(np.uint8)


def rans_vectors():
    shapes = {
        "single": lambda n: bytes([7]) * n,
        "two": lambda n: bytes((i & 1) * 200 for i in range(n)),
        "alphabet": lambda n: bytes(i % 256 for i in range(n)),
        "outlier": lambda n: bytes([0] * (n - 1) + [255]),
        "noise": lambda n: lcg(n, n + 5),
        "skewed": lambda n: lcg(n, n + 9).translate(
            bytes([0x40]) * 170 + bytes(range(16)) * 5 + bytes([0x7F]) * 6),
    }
    out = {}
    for n in (1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 255, 256, 4096, 4097):
        for name, make in shapes.items():
            data = make(n)
            enc = kernels.rans_encode(data)
            assert bytes(kernels.rans_decode(enc, n)) == data
            out[f"{name}_{n}_plain"] = np.frombuffer(data, dtype=np.uint8)
            out[f"{name}_{n}_stream"] = np.frombuffer(enc, dtype=np.uint8)
    # majority-symbol states past 2^31 (tests/test_lmz.py:351-382)
    for seed, fmaj, n in ((95, 3998, 4096), (165, 3998, 4096)):
        x, buf = seed | 1, bytearray([0x3E]) * n
        placed, minority = 0, n * (4096 - fmaj) // 4096
        while placed < minority:
            x = (x * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
            pos = x % n
            if buf[pos] == 0x3E:
                buf[pos] = 0x3F
                placed += 1
        enc = kernels.rans_encode(bytes(buf))
        out[f"majority{seed}_{n}_plain"] = np.frombuffer(bytes(buf), dtype=np.uint8)
        out[f"majority{seed}_{n}_stream"] = np.frombuffer(enc, dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "rans_vectors.npz"), **out)
    return len(out) // 2


def archive_case(name, files, manifest, **kw):
    tmp = tempfile.mkdtemp()
    try:
        src = os.path.join(tmp, "src")
        os.makedirs(src)
        for rel, data in files:
            path = os.path.join(src, rel)
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "wb") as f:
                f.write(bytes(data))
        target = src if len(files) > 1 else os.path.join(src, files[0][0])
        dst = os.path.join(HERE, name + ".lmz")
        if os.path.exists(dst):
            os.unlink(dst)
        api.compress(target, dst, workers=1, **kw)
        back = os.path.join(tmp, "back")
        api.decompress(dst, back if len(files) > 1 else os.path.join(tmp, "back.bin"))
        if len(files) > 1:
            with open(dst, "rb") as fh:
                from lmz.format import ArchiveReader
                members = ArchiveReader(fh).members
            plain = b"".join(open(os.path.join(back, m.path), "rb").read() for m in members)
        else:
            plain = open(os.path.join(tmp, "back.bin"), "rb").read()
        with open(dst, "rb") as fh:
            from lmz.format import ArchiveReader
            rd = ArchiveReader(fh)
            codecs = [int(c.codec) for c in rd.chunks]
        manifest[name] = {"options": {k: v for k, v in kw.items()}, "plain_bytes": len(plain),
                          "plain_sha256": hashlib.sha256(plain).hexdigest(),
                          "archive_bytes": os.path.getsize(dst), "codecs": codecs,
                          "lmz_version": lmz.__version__}
    finally:
        shutil.rmtree(tmp)


def st(tensors):
    return synth.safetensors_bytes(tensors).tobytes()


def main():
    n = rans_vectors()
    man = {}
    w = cond_bf16(1 << 20, 1)
    archive_case("bf16_conditioned", [("m.safetensors", st([("w", "BF16", (1 << 20,), w)]))], man)
    g = synth.normal_bf16((96, 1024), 7)
    norm = synth.bf16_bytes(np.ones(1024, np.float32))
    small = st([("a.weight", "BF16", (96, 1024), g), ("a.norm", "BF16", (1024,), norm)])
    archive_case("bf16_mapped", [("m.safetensors", small)], man, mapped=True)
    archive_case("bf16_default_small", [("m.safetensors", small)], man)
    rng = np.random.default_rng(5)
    f32 = (rng.standard_normal(40000) * 0.02).astype("<f4").view(np.uint8)
    i64 = rng.integers(0, 50, 3001).astype("<i8").view(np.uint8)
    archive_case("f32_i64_split", [("m.safetensors", st([("f", "F32", (40000,), f32),
                                                          ("i", "I64", (3001,), i64)]))], man)
    # delta chain: checkpoint 1 nudges one tensor, keeps another identical (a ref)
    a0 = cond_bf16(1 << 20, 3)
    b0 = synth.normal_bf16((64, 1024), 4)
    a1 = a0.copy().view("<u2")
    idx = np.random.default_rng(6).integers(0, a1.size, a1.size // 50)
    a1[idx] ^= 1
    ck0 = st([("a", "BF16", (1 << 20,), a0), ("b", "BF16", (64, 1024), b0)])
    ck1 = st([("a", "BF16", (1 << 20,), a1.view(np.uint8)), ("b", "BF16", (64, 1024), b0)])
    archive_case("delta_chain", [("ck0/model.safetensors", ck0), ("ck1/model.safetensors", ck1)], man)
    archive_case("raw_bytes", [("blob.bin", lcg(5000, 1) + bytes(3000) + b"abc" * 20000)], man)
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(man, f, indent=1, sort_keys=True)
    print(n, "stream vectors;", {k: (v["archive_bytes"], sorted(set(v["codecs"]))) for k, v in man.items()})


if __name__ == "__main__":
    main()
