"""Whole-archive decode on the GPU against the CPU oracle and the source bytes.

Archives are written by the oracle's writer, which emits the reference
encoder's exact chunk bytes (tests/test_oracle_vs_reference.py holds it to
that), and by the reference itself for the committed golden archives."""
import numpy as np
import pytest

from oracle import archive as oa, synth

pytestmark = pytest.mark.gpu


def _roundtrip(blob, source, checksum=True, fuse=True, classify="device"):
    import zlib
    from lmz_b200 import archive, decode, plan
    ar = archive.Archive(blob)
    dec = decode.ArchiveDecoder(ar, checksum=checksum, plan=plan.build_plan(ar, fuse=fuse, classify=classify))
    dec.run()
    dec.check()
    got = dec.output.cpu().numpy()
    want = oa.decode_archive(blob)
    assert got.size == want.size == source.size
    assert (want == source).all()
    assert (got == want).all(), f"first difference at byte {int(np.nonzero(got != want)[0][0])}"
    if checksum:
        ar = dec.archive
        crcs = dec.chunk_crcs()
        for i, rec in enumerate(ar.records):
            d, n = int(rec["dst"]), int(rec["rlen"])
            assert int(crcs[i]) == (zlib.crc32(source[d:d + n]) & 0xFFFFFFFF), f"crc of chunk {i}"
    return dec


@pytest.fixture(scope="module")
def shard():
    return synth.llama_shard([0], 5, scale=0.25, vocab=4000, embed=True, head=True)


@pytest.mark.parametrize("kw", [dict(), dict(mapped=True), dict(chunk_size=1 << 20),
                                dict(chunk_size=2 << 20), dict(chunk_size=(1 << 18) + 2)])
def test_bf16_shard_layouts(shard, kw):
    blob = oa.write_archive([("m.safetensors", shard)], **kw)
    dec = _roundtrip(blob, shard)
    if not kw:
        assert (dec.archive.records["codec"] == 5).any(), "default chunking should condition"


def test_wide_exponent_alphabets_take_the_large_table_instance():
    """BF16 whose exponent byte takes ~200 values (a skewed draw, so rANS still pays):
    the planner must list such chunks after the small-alphabet ones, and the
    256-entry instance of the fused kernel must decode them."""
    from lmz_b200 import archive, plan
    rng = np.random.default_rng(11)
    n = 600_000
    e = np.minimum(rng.geometric(0.03, n) - 1, 199).astype(np.uint16)        # ~200 live exponents
    b = rng.integers(0, 256, n).astype(np.uint16)
    wide = (((b & 0x80) << 8) | (e << 7) | (b & 0x7F)).astype("<u2").view(np.uint8)
    narrow = synth.normal_bf16(300_000, 5)
    src = synth.safetensors_bytes([("wide", "BF16", (n,), wide), ("narrow", "BF16", (300_000,), narrow)])
    blob = oa.write_archive([("m.safetensors", src)], mapped=True)
    p = plan.build_plan(archive.Archive(blob), classify="host")
    assert 0 < p.n_fused_small < p.fused_jobs.size, (p.n_fused_small, p.fused_jobs.size)
    _roundtrip(blob, src, classify="host")
    _roundtrip(blob, src, classify="device")


def test_without_checksums(shard):
    blob = oa.write_archive([("m.safetensors", shard)], mapped=True)
    _roundtrip(blob, shard, checksum=False)


def _float_file(dtype, n, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(n) * 0.02).astype(dtype)
    name = {"float32": "F32", "float64": "F64", "float16": "F16"}[np.dtype(dtype).name]
    return synth.safetensors_bytes([("w", name, (n,), w.view(np.uint8)),
                                    ("tail", "U8", (13,), np.arange(13, dtype=np.uint8))])


@pytest.mark.parametrize("dtype,n", [("float32", 1 << 20), ("float32", 70001), ("float64", 300001),
                                     ("float16", 555555)])
def test_byte_plane_splits(dtype, n):
    src = _float_file(dtype, n, 3)
    for kw in (dict(), dict(mapped=True)):
        _roundtrip(oa.write_archive([("f.safetensors", src)], **kw), src)


@pytest.mark.parametrize("n,pad", [(1 << 20, 0), (70001, 0), (16384 * 9 + 5, 3), (3, 1), (200000, 2)])
def test_fp32_chunks_take_the_fused_kernel(n, pad):
    """FP32 weights of N(0, 0.02): the top byte plane is rANS-coded and the three lower
    planes are stored, so the chunks go to the fused decode + interleave + checksum
    kernel; `pad` shifts the data area to every 4-byte phase of the 16-byte store, and
    the same archive is decoded with the two-pass path and without checksums too."""
    from lmz_b200 import archive, decode, plan
    rng = np.random.default_rng(n)
    w = (rng.standard_normal(n) * 0.02).astype("<f4")
    src = synth.safetensors_bytes([("lead", "F32", (pad,), np.zeros(pad, "<f4").view(np.uint8)),
                                   ("w", "F32", (n,), w.view(np.uint8))])
    for kw in (dict(), dict(mapped=True)):
        blob = oa.write_archive([("f.safetensors", src)], **kw)
        p = plan.build_plan(archive.Archive(blob), fuse="all")
        if n >= 70001:
            assert p.n_fused_f32 > 0 and p.n_fused_f32 == p.fused_jobs.size, (p.n_fused_f32, p.fused_jobs.size)
        assert plan.build_plan(archive.Archive(blob)).n_fused_f32 == 0       # too few to pay
        _roundtrip(blob, src, fuse="all")
        _roundtrip(blob, src, checksum=False, fuse="all")
        two_pass = decode.ArchiveDecoder(blob, fuse=False)
        assert two_pass.plan.fused_jobs.size == 0
        two_pass.run()
        two_pass.check()
        assert (two_pass.output.cpu().numpy() == src).all()


def test_mixed_bf16_and_fp32_members_share_one_fused_launch_list(shard):
    rng = np.random.default_rng(4)
    f32 = synth.safetensors_bytes([("w", "F32", (300000,), (rng.standard_normal(300000) * 0.02).astype("<f4").view(np.uint8))])
    from lmz_b200 import archive, plan
    blob = oa.write_archive([("a.safetensors", shard), ("b.safetensors", f32)], mapped=True)
    p = plan.build_plan(archive.Archive(blob), fuse="all")
    assert 0 < p.n_fused_f32 < p.fused_jobs.size
    _roundtrip(blob, np.concatenate([shard, f32]), fuse="all")


def test_delta_chain_and_refs():
    c0 = synth.llama_shard([0, 1], 9, scale=0.25)
    tensors = oa.parse_safetensors(c0)[1]
    files = [c0]
    for step in (1, 2):
        c = files[-1].copy()
        for i, (name, info) in enumerate(tensors.items()):
            s, e = info["offsets"]
            if i % 5 == 4:
                continue                        # left identical: becomes a ref
            if e - s > 100000:
                c[s:e] = synth.perturbed_bf16(files[-1][s:e], 100 * step + i)
        files.append(c)
    members = [(f"ck/{i}.safetensors", f) for i, f in enumerate(files)]
    for kw in (dict(), dict(chunk_size=1 << 20)):
        blob = oa.write_archive(members, **kw)
        dec = _roundtrip(blob, np.concatenate(files))
        codecs = set(dec.archive.records["codec"].tolist())
        assert {4, 8} <= codecs, codecs


@pytest.mark.parametrize("name", ["t", "tt", "ttt", "tttt"])
def test_conditioned_chunk_with_a_stored_exponent_plane(name):
    """Exponent bytes that do not compress (uniform) under a sign/mantissa byte that depends
    on the exponent's bucket: the encoder conditions the chunk and stores the exponent plane as
    it is, so the histogram, the counting and the finish read it from the payload at whatever
    byte offset it landed on (the tensor's name moves it), and the chunk ends in a ragged piece."""
    from oracle import codec
    rng = np.random.default_rng(3)
    n = (1 << 20) + 12345
    e = rng.integers(0, 256, n).astype(np.uint16)
    noise = rng.random(n) < 0.03
    b = np.where(noise, rng.integers(0, 256, n), (e // 32) * 17 + 3).astype(np.uint16)
    w = (((b & 0x80) << 8) | (e << 7) | (b & 0x7F)).astype("<u2").view(np.uint8)
    src = synth.safetensors_bytes([(name, "BF16", (n,), w)])
    blob = oa.write_archive([("m.safetensors", src)])
    recs = oa.Archive(blob).records
    cond = [r for r in recs if r["codec"] == codec.CODEC_BF16C]
    assert len(cond) == 1
    head = codec.BF16C_HDR.unpack_from(np.frombuffer(blob, dtype=np.uint8), int(cond[0]["off"]))
    assert head[1] == 0 and 3 in head[2:10], "exponent plane stored, some segment coded"
    _roundtrip(blob, src)


def test_delta_whose_exponent_differences_have_a_wide_alphabet():
    """Deltas go to one kernel that decodes both planes of the difference: chunks whose
    exponent differences take a handful of values to its instance with mixed table sizes,
    the others -- here ~150 distinct differences -- to the one with full-size tables for both
    planes.  The sign/mantissa difference is all zeros: a one-symbol stream."""
    from lmz_b200 import archive, plan
    rng = np.random.default_rng(21)
    n = 700_000
    base = rng.integers(0, 65536, n).astype("<u2")
    d = np.minimum(rng.geometric(0.04, n) - 1, 180).astype(np.uint16)
    d[rng.random(n) < 0.5] = 0
    nxt = (base ^ (d << 7)).astype("<u2")
    small = synth.normal_bf16(200_000, 4)
    near = synth.perturbed_bf16(small, 9)
    a = synth.safetensors_bytes([("w", "BF16", (n,), base.view(np.uint8)), ("v", "BF16", (200_000,), small)])
    b = synth.safetensors_bytes([("w", "BF16", (n,), nxt.view(np.uint8)), ("v", "BF16", (200_000,), near)])
    for kw in (dict(mapped=True), dict(chunk_size=(1 << 17) + 6)):
        blob = oa.write_archive([("a.safetensors", a), ("b.safetensors", b)], **kw)
        p = plan.build_plan(archive.Archive(blob))
        assert p.delta_jobs.size >= 2 and p.stream_jobs.size == 0
        _roundtrip(blob, np.concatenate([a, b]))
        _roundtrip(blob, np.concatenate([a, b]), checksum=False)


def test_tiny_and_odd_members():
    rng = np.random.default_rng(0)
    members = [("a.bin", rng.integers(0, 4, 100001, dtype=np.uint8)),      # one rANS-coded byte stream
               ("b.bin", rng.integers(0, 256, 777, dtype=np.uint8)),       # stored
               ("c.bin", np.zeros(1, dtype=np.uint8)),
               ("d.txt", np.frombuffer(b"hello lmz " * 5000, dtype=np.uint8))]   # deflate on the host
    blob = oa.write_archive(members)
    _roundtrip(blob, np.concatenate([m[1] for m in members]))


def test_corruption_is_reported(shard):
    from lmz_b200 import decode
    from lmz_b200.archive import CorruptArchive, FormatError
    blob = bytearray(oa.write_archive([("m.safetensors", shard)], chunk_size=1 << 20))
    ar = oa.Archive(bytes(blob))
    rec = ar.records[3]
    hit = bytearray(blob)
    hit[int(rec["off"]) + int(rec["clen"]) - 100] ^= 0x5A          # inside a stored mantissa plane
    dec = decode.ArchiveDecoder(bytes(hit))
    dec.run()
    with pytest.raises(CorruptArchive, match="checksum"):
        dec.check()
    hit = bytearray(blob)
    hit[int(rec["off"]) + 8 + 600] ^= 0xFF                         # inside the exponent stream
    dec = decode.ArchiveDecoder(bytes(hit))
    dec.run()
    with pytest.raises(CorruptArchive):
        dec.check()
    hit = bytearray(blob)
    hit[int(rec["off"]) + 8] = ord("X")                            # the stream's magic
    dec = decode.ArchiveDecoder(bytes(hit))
    dec.run()
    with pytest.raises(CorruptArchive):
        dec.check()
    with pytest.raises(FormatError):
        decode.ArchiveDecoder(bytes(blob[:-1]))


def test_plain_chunks_with_both_planes_coded():
    """BF16 whose sign/mantissa bytes compress too (a few distinct values): both planes of a
    chunk are rANS streams, and the two-plane kernel decodes, merges and checksums them in the
    first pass without a base; a later member that is a delta against such chunks reads them."""
    from lmz_b200 import archive, plan
    rng = np.random.default_rng(17)
    n = 500_003
    vals = synth.normal_bf16(64, 3).view("<u2")
    w = vals[rng.integers(0, 64, n)].astype("<u2")
    a = synth.safetensors_bytes([("w", "BF16", (n,), w.view(np.uint8))])
    w2 = w.copy()
    hit = rng.random(n) < 0.2
    w2[hit] ^= rng.integers(1, 4, int(hit.sum())).astype("<u2")
    b = synth.safetensors_bytes([("w", "BF16", (n,), w2.view(np.uint8))])
    for kw in (dict(mapped=True), dict(chunk_size=1 << 20)):
        blob = oa.write_archive([("a.safetensors", a), ("b.safetensors", b)], **kw)
        p = plan.build_plan(archive.Archive(blob))
        assert 0 < p.n_delta_plain < p.delta_jobs.size, (p.n_delta_plain, p.delta_jobs.size)
        assert (p.delta_jobs["base_off"][:p.n_delta_plain] == plan.NONE64).all()
        assert (p.delta_jobs["base_off"][p.n_delta_plain:] != plan.NONE64).all()
        _roundtrip(blob, np.concatenate([a, b]))
        _roundtrip(blob, np.concatenate([a, b]), checksum=False)


def test_corrupt_delta_chunks_are_reported():
    """Damage inside either plane's stream of a delta chunk, in a stream's magic and in a
    frequency table: the one-pass delta kernel (or the checksum behind it) reports each."""
    from lmz_b200 import archive, decode, plan
    from lmz_b200.archive import CorruptArchive
    base = synth.safetensors_bytes([("w", "BF16", (300_000,), synth.normal_bf16(300_000, 2))])
    nxt = base.copy()
    s, e = list(oa.parse_safetensors(base)[1].values())[0]["offsets"]
    nxt[s:e] = synth.perturbed_bf16(base[s:e], 5)
    blob = oa.write_archive([("a.safetensors", base), ("b.safetensors", nxt)], mapped=True)
    p = plan.build_plan(archive.Archive(blob))
    assert p.delta_jobs.size
    j = p.delta_jobs[p.delta_jobs.size // 2]
    for where in (int(j["src_a"]) + 548 + 40, int(j["src_b"]) + 548 + 1000, int(j["src_b"]), int(j["src_a"]) + 4 + 2 * 7):
        hit = bytearray(blob)
        hit[where] ^= 0x41
        dec = decode.ArchiveDecoder(bytes(hit))
        dec.run()
        with pytest.raises(CorruptArchive):
            dec.check()
    dec = decode.ArchiveDecoder(blob)
    dec.run()
    dec.check()


def test_corrupt_conditioned_chunks_are_reported(shard):
    """Default chunking: damage to the exponent stream of a conditioned chunk changes its
    histogram, so its bucket sizes no longer match the stored segments - the chunk is
    reported and its segments are not indexed with the wrong counts."""
    import struct
    from lmz_b200 import decode
    from lmz_b200.archive import CorruptArchive
    blob = oa.write_archive([("m.safetensors", shard)])
    ar = oa.Archive(bytes(blob))
    i = int(np.nonzero(ar.records["codec"] == 5)[0][0])
    rec = ar.records[i]
    for where in (46 + 548 + 4000, 46 + 548 + 9):                   # inside the exponent stream
        hit = bytearray(blob)
        hit[int(rec["off"]) + where] ^= 0x81
        dec = decode.ArchiveDecoder(bytes(hit))
        dec.run()
        with pytest.raises(CorruptArchive):
            dec.check()
    # a segment length that disagrees with the bucket population (header field, lmz/codec.py:50)
    hit = bytearray(blob)
    pos = int(rec["off"]) + 1 + 1 + 8 + 4                            # k, exp_m, sm_m[8], exp_len -> seg_len[0]
    n0 = struct.unpack_from("<I", hit, pos)[0]
    struct.pack_into("<I", hit, pos, n0 - 16)
    struct.pack_into("<I", hit, pos + 4, struct.unpack_from("<I", hit, pos + 4)[0] + 16)
    dec = decode.ArchiveDecoder(bytes(hit))
    dec.run()
    with pytest.raises(CorruptArchive):
        dec.check()


def test_tensor_views(shard):
    import torch
    from lmz_b200 import decode
    blob = oa.write_archive([("m.safetensors", shard)], mapped=True)
    dec = decode.ArchiveDecoder(blob)
    dec.run()
    dec.check()
    ts = dec.tensors()
    info = oa.parse_safetensors(shard)[1]
    assert len(ts) == len(info)
    for (path, name), t in ts.items():
        s, e = info[name]["offsets"]
        assert t.dtype == torch.bfloat16 and list(t.shape) == info[name]["shape"]
        assert t.contiguous().view(torch.uint8).reshape(-1).cpu().numpy().tobytes() == shard[s:e].tobytes()


def test_tensor_addressed_decode():
    """decode_tensors uploads and decodes only the chunks a tensor needs - through every
    layout, and through deltas and refs, whose sources it must bring along."""
    import torch
    from lmz_b200 import archive, decode, multi
    c0 = synth.llama_shard([0, 1], 9, scale=0.25)
    info = oa.parse_safetensors(c0)[1]
    c1 = c0.copy()
    names = list(info)
    for i, name in enumerate(names):
        s, e = info[name]["offsets"]
        if i % 3 and e - s > 100000:
            c1[s:e] = synth.perturbed_bf16(c0[s:e], 300 + i)
    members = [("ck/0.safetensors", c0), ("ck/1.safetensors", c1)]
    hdr = c0.size - max(t["offsets"][1] for t in info.values())       # safetensors header bytes
    for kw in (dict(), dict(mapped=True), dict(chunk_size=1 << 20)):
        blob = oa.write_archive(members, **kw)
        ar = archive.Archive(blob)
        pick = [("ck/1.safetensors", names[1]), ("ck/1.safetensors", names[-2]), ("ck/0.safetensors", names[3])]
        got = decode.decode_tensors(ar, pick)
        assert set(got) == set(pick)
        for (member, name), t in got.items():
            src = c0 if member.endswith("0.safetensors") else c1
            s, e = info[name]["offsets"]
            assert t.dtype == torch.bfloat16 and list(t.shape) == info[name]["shape"]
            assert t.contiguous().view(torch.uint8).reshape(-1).cpu().numpy().tobytes() == \
                src[hdr + s:hdr + e].tobytes(), (kw, member, name)
        # a small tensor needs a small part of the archive
        key = ("ck/1.safetensors", "model.norm.weight") if "model.norm.weight" in info else pick[0]
        sel = multi.cover(ar, [ar.tensor_index()[key][2:4]])
        assert sel.size < ar.records.size / 4, (sel.size, ar.records.size)
    with pytest.raises(KeyError):
        decode.decode_tensors(ar, [names[0]])             # in both members: ambiguous


def test_reference_written_archives_decode_to_the_reference_plaintext():
    """The committed archives were written by the reference's own `lmz compress`;
    the recorded digest is of what its `decompress` restored."""
    import hashlib
    import json
    import os
    from lmz_b200 import decode
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with open(os.path.join(gold, "manifest.json")) as f:
        man = json.load(f)
    for name, info in man.items():
        blob = np.fromfile(os.path.join(gold, name + ".lmz"), dtype=np.uint8)
        out = decode.decode_archive(blob).cpu().numpy()
        assert out.size == info["plain_bytes"], name
        assert hashlib.sha256(out.tobytes()).hexdigest() == info["plain_sha256"], name


def test_reference_written_streams_decode(gpu):
    import os
    from helpers import pack_streams
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    v = np.load(os.path.join(gold, "rans_vectors.npz"))
    for case in sorted(k[:-6] for k in v.files if k.endswith("_plain")):
        plain, stream = v[case + "_plain"], v[case + "_stream"]
        blob, offs = pack_streams([stream.tobytes()] * 3)
        out = gpu.decode_batch(blob, offs, 3, plain.size)
        assert bytes(out) == plain.tobytes() * 3, case


def test_pipelined_upload_decodes_the_same_bytes(shard):
    import torch
    from lmz_b200 import decode
    for kw in (dict(mapped=True), dict()):
        blob = oa.write_archive([("m.safetensors", shard)], **kw)
        pd = decode.PipelinedDecoder(blob, nslices=5)
        assert len(pd.slices) == (5 if kw else min(5, len(pd.slices)))
        pinned = torch.frombuffer(bytearray(blob), dtype=torch.uint8).pin_memory()
        out = pd.run_from_host(pinned)
        pd.check()
        assert (out.cpu().numpy() == shard).all()
        auto = decode.PipelinedDecoder(blob)                 # slice count chosen by chunk size
        assert len(auto.slices) == (8 if kw else 1)
        assert (auto.run_from_host(pinned).cpu().numpy() == shard).all()
        auto.check()


def test_pythia_shaped_delta_chain():
    """Checkpoint delta chain on the Pythia-160m architecture (12 layers, hidden 768,
    FFN 3072, vocab 50304) at half width: checkpoint 0 from N(0, 0.02), each later one
    the previous plus N(0, 1e-4) on a random 30 % of elements; both later checkpoints
    are coded as deltas against checkpoint 0 (the earliest member holding the tensor)."""
    files = synth.delta_chain_files(hidden=384, ffn=1536, vocab=25152, layers=12)
    # one tensor of checkpoint 1 left as it was in checkpoint 0: stored as a reference
    # (the reference deduplicates identical tensors of 64 KiB or more, lmz/api.py:47,260)
    s, e = oa.parse_safetensors(files[1])[1]["l0.attn.o.weight"]["offsets"]
    files[1] = files[1].copy()
    files[1][s:e] = files[0][s:e]
    blob = oa.write_archive([(f"step{i}/model.safetensors", f) for i, f in enumerate(files)])
    dec = _roundtrip(blob, np.concatenate(files))
    recs = dec.archive.records
    assert (recs["codec"] == 8).sum() >= 2 and (recs["codec"] == 4).sum() >= 1
    assert len(blob) < 0.6 * sum(f.size for f in files)


def test_per_rank_tensor_parallel_slices():
    """Tensor-parallel slices as separate members: each rank's archive holds only its
    slice (here FP32, esize-4 byte-plane chunks) and decodes on its own."""
    rng = np.random.default_rng(11)
    full = (rng.standard_normal((1024, 4096)) * 0.02).astype("<f4")
    for rank in range(2):
        col = np.ascontiguousarray(full[rank * 512:(rank + 1) * 512])          # column-parallel
        row = np.ascontiguousarray(full[:, rank * 2048:(rank + 1) * 2048])     # row-parallel
        src = synth.safetensors_bytes([("q.weight", "F32", col.shape, col.view(np.uint8).reshape(-1)),
                                       ("o.weight", "F32", row.shape, row.view(np.uint8).reshape(-1))])
        dec = _roundtrip(oa.write_archive([(f"rank{rank}.safetensors", src)]), src)
        t = dec.tensors()[(f"rank{rank}.safetensors", "o.weight")]
        assert t.cpu().numpy().tobytes() == row.tobytes()


def test_load_archive_streams_a_file_through_staging(shard, tmp_path):
    """decode.load_archive: file -> page-locked staging -> HBM with the decode of earlier
    slices under the copies; small staging blocks here so that every slice takes several."""
    from lmz_b200 import decode
    for kw in (dict(mapped=True), dict()):
        blob = oa.write_archive([("m.safetensors", shard)], **kw)
        path = tmp_path / f"a{len(kw)}.lmz"
        path.write_bytes(blob)
        stats = {}
        out = decode.load_archive(str(path), stats=stats)
        assert (out.cpu().numpy() == shard).all()
        assert stats["h2d_bytes"] <= len(blob) and stats["run_s"] > 0
        ar = decode.fmt.Archive(str(path))
        pd = decode.PipelinedDecoder(ar)
        small = decode.Staging(block=1 << 12, depth=3, threads=2)      # thousands of blocks through three buffers
        assert (pd.run_from_file(staging=small).cpu().numpy() == shard).all()
        pd.check()


def test_host_and_device_classification_agree(shard):
    """The fused jobs sorted by alphabet on the host (numpy / the library's host helper) and
    on the device (k_classify) decode to the same bytes, wide alphabets included."""
    rng = np.random.default_rng(12)
    n = 400_000
    e = np.minimum(rng.geometric(0.03, n) - 1, 199).astype(np.uint16)
    b = rng.integers(0, 256, n).astype(np.uint16)
    wide = (((b & 0x80) << 8) | (e << 7) | (b & 0x7F)).astype("<u2").view(np.uint8)
    f32 = (rng.standard_normal(300_000) * 0.02).astype("<f4").view(np.uint8)
    src = synth.safetensors_bytes([("wide", "BF16", (n,), wide), ("narrow", "BF16", (200_000,), synth.normal_bf16(200_000, 6))])
    src2 = synth.safetensors_bytes([("f", "F32", (300_000,), f32)])
    both = np.concatenate([src, src2])
    blob = oa.write_archive([("a.safetensors", src), ("b.safetensors", src2)], mapped=True)
    from lmz_b200 import archive, decode, plan
    ar = archive.Archive(blob)
    for classify in ("host", "device"):
        p = plan.build_plan(ar, fuse="all", classify=classify)
        assert p.device_classify == (classify == "device") and p.n_fused_f32 > 0
        dec = decode.ArchiveDecoder(ar, plan=p)
        dec.run()
        dec.check()
        assert (dec.output.cpu().numpy() == both).all()
