"""The CPU oracle against fixtures the reference itself produced (tests/golden/,
written by make_golden.py with the reference's encoder and decoder), and, when
it was built, against the reference's compiled C core."""
import hashlib
import json
import os

import numpy as np
import pytest

from helpers import SHAPES, lcg_bytes, shaped
from oracle import archive as oa, codec, native

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def vectors():
    return np.load(os.path.join(GOLD, "rans_vectors.npz"))


@pytest.fixture(scope="module")
def manifest():
    with open(os.path.join(GOLD, "manifest.json")) as f:
        return json.load(f)


def _cases(vectors):
    return sorted(k[:-6] for k in vectors.files if k.endswith("_plain"))


def test_rans_decode_matches_reference_streams(orc, vectors):
    for case in _cases(vectors):
        plain, stream = vectors[case + "_plain"], vectors[case + "_stream"]
        got, states, cursor = orc.rans_decode_ex(stream, plain.size)
        assert (got == plain).all(), case
        # the reference encoder starts every lane at 2^16 and the decoder ends there
        assert (states == 1 << 16).all() and cursor == stream.size, case


def test_rans_encode_writes_the_reference_bytes(orc, vectors):
    for case in _cases(vectors):
        plain, stream = vectors[case + "_plain"], vectors[case + "_stream"]
        assert orc.rans_encode(plain) == stream.tobytes(), case


def test_numpy_stream_builder_writes_the_reference_bytes(vectors):
    from lmz_b200 import _streams
    for case in _cases(vectors):
        plain, stream = vectors[case + "_plain"], vectors[case + "_stream"]
        if plain.size > 300:
            continue
        assert _streams.encode_batch(plain[None, :])[0] == stream.tobytes(), case


def test_malformed_streams_are_rejected(orc):
    good = orc.rans_encode(np.frombuffer(lcg_bytes(10000, 3), dtype=np.uint8) & 0x3F)
    for name, bad in (("truncated", good[:len(good) // 2]), ("bad magic", b"XX" + good[2:]),
                      ("empty", b""), ("header only", good[:516])):
        with pytest.raises(ValueError):
            orc.rans_decode(np.frombuffer(bad, dtype=np.uint8), 10000)
    skew = bytearray(good)
    skew[4] ^= 1
    with pytest.raises(ValueError):
        orc.rans_decode(np.frombuffer(bytes(skew), dtype=np.uint8), 10000)


def test_archives_decode_to_the_reference_plaintext(orc, manifest):
    for name, info in manifest.items():
        blob = np.fromfile(os.path.join(GOLD, name + ".lmz"), dtype=np.uint8)
        ar = oa.Archive(blob)
        assert ar.records["codec"].tolist() == info["codecs"], name
        out = oa.decode_archive(ar, lib=orc)
        assert out.size == info["plain_bytes"], name
        assert hashlib.sha256(out.tobytes()).hexdigest() == info["plain_sha256"], name


def test_golden_set_covers_every_chunk_kind_on_the_path(manifest):
    seen = set()
    for info in manifest.values():
        seen |= set(info["codecs"])
    assert {0, 1, 2, 3, 4, 5, 8} <= seen, seen


def test_bf16_merge_formula(orc):
    # w = ((b & 0x80) << 8) | (a << 7) | (b & 0x7F), little-endian
    a = np.arange(256, dtype=np.uint8).repeat(256)
    b = np.tile(np.arange(256, dtype=np.uint8), 256)
    w = ((b.astype(np.uint32) & 0x80) << 8) | (a.astype(np.uint32) << 7) | (b & 0x7F)
    assert (orc.merge_bf16(a, b).view("<u2") == w).all()
    pa, pb = orc.split_bf16(w.astype("<u2").view(np.uint8))
    assert (pa == a).all() and (pb == b).all()


def test_bucket_map_rule(orc):
    rng = np.random.default_rng(2)
    for _ in range(50):
        hist = (rng.random(256) ** 8 * rng.integers(1, 1 << 22)).astype(np.uint64)
        lut = orc.bucket_lut(hist, 8)
        total, acc, b = int(hist.sum()), 0, 0
        for s in range(256):
            assert lut[s] == b
            acc += int(hist[s])
            while b + 1 < 8 and acc * 8 >= (b + 1) * total:
                b += 1


def test_crc32_is_zlibs(orc):
    import zlib
    for n in (0, 1, 7, 4096, 100003):
        d = lcg_bytes(n, n)
        assert orc.crc32(np.frombuffer(d, dtype=np.uint8)) == (zlib.crc32(d) & 0xFFFFFFFF)


# ---- the restatement against the reference's compiled core ----------------------------

ref = native.ref()
needs_ref = pytest.mark.skipif(ref is None, reason="oracle/_ref was not built")


@needs_ref
def test_port_and_reference_core_agree_on_streams(orc):
    for name in SHAPES:
        for n in (1, 8, 9, 4095, 4096, 4097, 65537):
            p = shaped(name, n, n + 1)
            s = ref.rans_encode(p)
            assert orc.rans_encode(p) == s == ref.rans_encode_portable(p), (name, n)
            assert (orc.rans_decode(s, n) == p).all() and (ref.rans_decode(s, n) == p).all()


@needs_ref
def test_port_and_reference_core_agree_on_planes(orc):
    from oracle import synth
    w = synth.normal_bf16((1 << 18,), 3)
    for a, b in zip(orc.split_bf16(w), ref.split_bf16(w)):
        assert (a == b).all()
    pa, pb = orc.split_bf16(w)
    h = orc.histogram(pa)
    assert (h == ref.histogram(pa)).all()
    lut = orc.bucket_lut(h)
    assert (lut == ref.bucket_lut(h)).all()
    p1, c1 = orc.bucket_partition(pa, pb, lut)
    p2, c2 = ref.bucket_partition(pa, pb, lut)
    assert (p1 == p2).all() and (c1 == c2).all()
    f32 = np.frombuffer(lcg_bytes(4 * 5000, 1), dtype=np.uint8)
    assert (orc.split_planes(f32, 4) == ref.split_planes(f32, 4)).all()
    from oracle import encode
    parts, cid, flags, _ = encode.encode_chunk(w, 2, codec.KIND_BF16, lib=orc)
    payload = np.frombuffer(b"".join(bytes(p) for p in parts), dtype=np.uint8)
    a = orc.decode_planes(payload, 2, w.size // 2, flags, True)
    b = ref.decode_planes(payload, 2, w.size // 2, flags, True)
    assert (a == b).all() and (a == w).all()
