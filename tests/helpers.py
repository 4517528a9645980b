"""Seeded inputs shared by the tests."""
import struct

import numpy as np

# translate() tables over uniform bytes: the reference's awkward distributions
# (tests/test_lmz.py:2335-2346 in the reference tree).
SHAPES = {
    "single": bytes([0x5A]) * 256,
    "two": bytes([0x01]) * 128 + bytes([0xFE]) * 128,
    "flat": bytes(range(256)),
    "tail": bytes([0x20]) * 250 + bytes(range(6)),
    "skewed": bytes([0x40]) * 170 + bytes(range(16)) * 5 + bytes([0x7F]) * 6,
}


def lcg_bytes(n: int, seed: int = 0) -> bytes:
    """The reference tests' deterministic byte source (tests/test_lmz.py:44-51)."""
    out, x = bytearray(), seed | 1
    while len(out) < n:
        x = (x * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out += x.to_bytes(8, "little")
    return bytes(out[:n])


def shaped(name: str, n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, n, dtype=np.uint8).tobytes().translate(SHAPES[name])
    return np.frombuffer(raw, dtype=np.uint8)


def distribution(name: str, n: int, seed: int) -> np.ndarray:
    """The eight symbol distributions of the decoder stress configuration."""
    rng = np.random.default_rng(seed)
    if name == "uniform":
        return rng.integers(0, 256, n, dtype=np.uint8)
    if name == "single":
        return np.full(n, 0x5A, dtype=np.uint8)
    if name == "two":
        return np.where(rng.random(n) < 0.999, 3, 200).astype(np.uint8)
    if name == "geometric":
        return np.minimum(rng.geometric(0.3, n) - 1, 255).astype(np.uint8)
    if name == "zipf":
        p = 1.0 / np.arange(1, 257) ** 1.1
        return rng.choice(256, size=n, p=p / p.sum()).astype(np.uint8)
    if name in ("exponent", "mantissa"):
        from oracle import synth, native
        w = synth.normal_bf16((n,), seed)
        pa, pb = native.oracle().split_bf16(w)
        return pa if name == "exponent" else pb
    if name == "zero-runs":
        out = rng.integers(0, 256, n, dtype=np.uint8)
        pos = 0
        while pos < n:
            run = int(rng.geometric(0.02))
            out[pos:pos + run] = 0
            pos += run + int(rng.geometric(0.1))
        return out
    raise KeyError(name)


DISTRIBUTIONS = ("uniform", "single", "two", "geometric", "zipf", "exponent", "mantissa",
                 "zero-runs")


def pack_streams(streams):
    offs, pos = bytearray(), 0
    for s in streams:
        offs += struct.pack("<QQ", pos, len(s))
        pos += len(s)
    return b"".join(streams), bytes(offs)
