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
    from oracle import synth
    return synth.stress_plane(name, n, seed)


DISTRIBUTIONS = ("uniform", "single", "two", "geometric", "zipf", "exponent", "mantissa",
                 "zero-runs")


def pack_streams(streams):
    offs, pos = bytearray(), 0
    for s in streams:
        offs += struct.pack("<QQ", pos, len(s))
        pos += len(s)
    return b"".join(streams), bytes(offs)
