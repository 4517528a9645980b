"""Host-side logic on the CPU: the library's exported symbols, the archive
reader, the planner's classification and its rejection of hostile input."""
import ctypes
import os
import re
import struct
import subprocess
import sys

import numpy as np
import pytest

from oracle import archive as oa, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    from lmz_b200 import build
    path = build.build()
    assert path, build.last_error
    return path


def test_library_exports_every_declared_symbol(lib_path):
    """Loads without a GPU and exports everything include/lmz_b200.h declares."""
    with open(os.path.join(ROOT, "include", "lmz_b200.h")) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    names = set(re.findall(r"\b(lmz_(?:gpu|host)_\w+)\s*\(", text))
    assert len(names) >= 13, names
    lib = ctypes.CDLL(lib_path)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared but not exported"
    lib.lmz_gpu_abi_version.restype = ctypes.c_int
    assert lib.lmz_gpu_abi_version() == 1
    assert lib.lmz_gpu_header_bytes() == 516 and lib.lmz_gpu_grain() == 1
    assert lib.lmz_gpu_pad_bytes() >= 272
    sizes = (ctypes.c_uint * 5)()
    lib.lmz_gpu_struct_sizes(ctypes.byref(sizes))
    from lmz_b200 import plan
    assert tuple(sizes) == (plan.STREAM_JOB.itemsize, plan.CHUNK_JOB.itemsize,
                            plan.COND_JOB.itemsize, plan.COND_STATE_BYTES, plan.FUSED_JOB.itemsize)
    assert lib.lmz_gpu_piece_bytes() == plan.PIECE


def test_alphabet_sizes_helper_matches_the_planner_fallback(lib_path, orc):
    """lmz_host_alphabet_sizes (host code of the library) and the planner's numpy
    count agree on streams with 1 ... 256 live symbols."""
    from lmz_b200 import plan
    rng = np.random.default_rng(3)
    streams, want = [], []
    for live in (1, 2, 24, 104, 105, 200, 256):
        syms = rng.choice(256, live, replace=False).astype(np.uint8)
        data = np.concatenate([syms, syms[rng.integers(0, live, 4000)]])
        streams.append(orc.rans_encode(data))
        want.append(live)
    blob = np.frombuffer(b"".join(streams), dtype=np.uint8)
    offs = np.cumsum([0] + [len(s) for s in streams[:-1]]).astype(np.uint64)
    assert plan._alphabet_sizes(blob, offs).tolist() == want          # numpy path (no library loaded here)
    lib = ctypes.CDLL(lib_path)
    lib.lmz_host_alphabet_sizes.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    out = np.zeros(len(streams), dtype=np.uint16)
    assert lib.lmz_host_alphabet_sizes(blob.ctypes.data, offs.ctypes.data, offs.size, out.ctypes.data) == 0
    assert out.tolist() == want


def test_validate_is_host_side(lib_path, orc):
    lib = ctypes.CDLL(lib_path)
    lib.lmz_gpu_validate.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint]
    lib.lmz_gpu_last_error.restype = ctypes.c_char_p
    s = orc.rans_encode(np.arange(4096, dtype=np.uint32).astype(np.uint8) & 7)
    off = struct.pack("<QQ", 0, len(s))
    assert lib.lmz_gpu_validate(s, off, 1) == 0
    assert lib.lmz_gpu_validate(b"XX" + s[2:], off, 1) == -3
    assert b"magic" in lib.lmz_gpu_last_error()
    bad = bytearray(s)
    bad[6] ^= 1
    assert lib.lmz_gpu_validate(bytes(bad), off, 1) == -3
    assert lib.lmz_gpu_validate(s, struct.pack("<QQ", 0, 100), 1) == -3


def _hold_build_lock(args):
    import time
    from lmz_b200 import build
    with build._build_lock():
        t0 = time.monotonic()
        time.sleep(args)
        return t0, time.monotonic()


def test_concurrent_builds_take_turns(lib_path):
    """One rank per GPU may find the library stale at the same moment: the build lock
    admits one process at a time (the others then find the library fresh)."""
    import multiprocessing as mp
    from lmz_b200 import build
    with mp.get_context("spawn").Pool(2) as pool:
        (a0, a1), (b0, b1) = pool.map(_hold_build_lock, [0.4, 0.4])
    assert a1 <= b0 or b1 <= a0, "both processes held the build lock at once"
    assert build.build() == build.LIB and not build._stale()


def test_import_is_free_of_cuda_side_effects():
    """Importing the package neither builds nor loads anything, and LMZ_NO_GPU
    disables the decoder (the reference's tests/test_lmz.py:2573-2607)."""
    code = ("import lmz_b200, sys; from lmz_b200 import gpu;"
            "assert gpu.state() == 'not probed', gpu.state();"
            "assert gpu.header_bytes.__name__;"
            "print('ok')")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert out.stdout.strip() == "ok", out.stderr
    env = dict(os.environ, LMZ_NO_GPU="1")
    out = subprocess.run([sys.executable, "-c",
                          "from lmz_b200 import gpu; ok, why = gpu.available(); print(ok, why);"
                          "print(gpu.decode_batch(b'', b'', 1, 8))"],
                         cwd=ROOT, capture_output=True, text=True, env=env)
    assert out.stdout.startswith("False") and "LMZ_NO_GPU" in out.stdout, out.stdout + out.stderr
    assert "None" in out.stdout


@pytest.fixture(scope="module")
def shard():
    return synth.llama_shard([0], 5, scale=0.125, vocab=1000, embed=True)


def test_reader_and_planner_classify_every_layout(shard):
    from lmz_b200 import archive, plan
    for kw, kinds in ((dict(), {0, 3}), (dict(mapped=True), {0, 1}), (dict(chunk_size=1 << 20), {0, 1})):
        blob = oa.write_archive([("m.safetensors", shard)], **kw)
        ar = archive.Archive(blob)
        assert ar.total == shard.size and ar.page_mapped == bool(kw.get("mapped"))
        p = plan.build_plan(ar)
        assert set(p.chunks["kind"].tolist()) == kinds
        assert p.n_pieces == int(((ar.records["rlen"].astype(np.int64) + 65535) // 65536).sum())
        assert sorted(p.chunks["record"].tolist()) == list(range(ar.records.size))
        assert p.piece_split[-1] == p.n_pieces
        # scratch regions of the stream jobs never overlap
        d = np.sort(p.stream_jobs, order="dst_off")
        assert (d["dst_off"][1:] >= d["dst_off"][:-1] + d["n"][:-1]).all()
        assert p.seg_jobs.size <= 8 * p.cond_jobs.size
        idx = ar.tensor_index()
        assert ("m.safetensors", "model.embed_tokens.weight") in idx


def test_planner_lists_fp32_chunks_after_bf16_in_the_fused_jobs(shard):
    """4-byte-element chunks whose top plane alone is coded are fused jobs of their own
    kind: listed after the BF16 ones, `mant_off` at stored plane 0 with planes 1 and 2
    following at n and 2n, the stream at plane 3, n = rlen / 4."""
    from lmz_b200 import archive, plan
    rng = np.random.default_rng(8)
    f32 = synth.safetensors_bytes([("w", "F32", (50000,), (rng.standard_normal(50000) * 0.02).astype("<f4").view(np.uint8))])
    blob = oa.write_archive([("a.safetensors", shard), ("b.safetensors", f32)], mapped=True)
    ar = archive.Archive(blob)
    p = plan.build_plan(ar, fuse="all")
    assert plan.build_plan(ar).n_fused_f32 == 0        # fewer than FUSE_F32_MIN: two passes
    nf = p.n_fused_f32
    assert 0 < nf < p.fused_jobs.size and p.n_fused_f32_small <= nf
    assert p.n_fused_small <= p.fused_jobs.size - nf
    for j in p.fused_jobs[-nf:]:
        c = p.chunks[np.nonzero(p.chunks["piece0"] == j["piece0"])[0][-1]]
        assert int(c["esize"]) == 4 and int(j["n"]) * 4 == int(c["rlen"])
        po = c["plane_off"]
        assert int(j["mant_off"]) == int(po[0]) and int(po[1]) == int(po[0]) + int(j["n"])
        assert int(po[2]) == int(po[0]) + 2 * int(j["n"]) and int(j["src_off"]) == int(po[3])
    assert plan.build_plan(ar, fuse=False).fused_jobs.size == 0


def test_planner_gives_two_plane_deltas_jobs_of_their_own(shard):
    """A delta chunk whose difference is a BF16 chunk with both planes coded gets a job for
    the kernel that decodes both planes and undoes the delta in one pass: no scratch streams,
    its pieces in the group the finish kernels skip, base and planes as the chunk says."""
    from lmz_b200 import archive, plan
    nxt = shard.copy()
    s, e = list(oa.parse_safetensors(shard)[1].values())[0]["offsets"]
    nxt[s:e] = synth.perturbed_bf16(shard[s:e], 77)
    blob = oa.write_archive([("a.safetensors", shard), ("b.safetensors", nxt)], mapped=True)
    ar = archive.Archive(blob)
    p = plan.build_plan(ar)
    ndelta = int((ar.records["codec"] == 8).sum())
    assert ndelta and 0 < p.delta_jobs.size <= ndelta
    chunk_at = {int(c["piece0"]): c for c in p.chunks}
    for j in p.delta_jobs:
        c = chunk_at[int(j["piece0"])]
        rec = ar.records[int(c["record"])]
        assert int(rec["codec"]) == 8 and int(c["base_off"]) == int(j["base_off"]) and int(j["n"]) * 2 == int(rec["rlen"])
        assert int(c["scratch_mask"]) == 0
        assert p.piece_split[2] <= int(j["piece0"]) < p.piece_split[3]
        lo, hi = int(rec["off"]), int(rec["off"]) + int(rec["clen"])
        assert lo < int(j["src_a"]) < int(j["src_b"]) < hi and int(j["src_a"]) + int(j["len_a"]) == int(j["src_b"])
        assert int(j["src_b"]) + int(j["len_b"]) == hi
    assert plan.build_plan(ar, fuse=False).delta_jobs.size == 0


def test_reader_rejects_damage(shard):
    from lmz_b200 import archive
    blob = oa.write_archive([("m.safetensors", shard)], mapped=True)
    with pytest.raises(archive.FormatError):
        archive.Archive(blob[:50])
    with pytest.raises(archive.FormatError):
        archive.Archive(b"NOPE" + blob[4:])
    with pytest.raises(archive.FormatError):
        archive.Archive(blob[:-3] + b"xyz")
    bad = bytearray(blob)
    bad[4] = 99                                   # unknown format version
    with pytest.raises(archive.FormatError):
        archive.Archive(bytes(bad))


def _rewrite_table(blob, mutate):
    """The archive with its record table edited by `mutate(records)`."""
    import json
    import zlib
    ar = oa.Archive(blob)
    recs = ar.records.copy()
    mutate(recs)
    toff = struct.unpack_from("<Q", blob, len(blob) - 40)[0]
    table_c = zlib.compress(recs.tobytes(), 3)
    man_c = zlib.compress(json.dumps(ar.manifest, separators=(",", ":")).encode(), 3)
    return (bytes(blob[:toff]) + table_c + man_c +
            oa.FOOTER.pack(toff, len(table_c), toff + len(table_c), len(man_c), oa.TAIL))


def test_planner_rejects_hostile_records(shard):
    from lmz_b200 import archive, plan
    blob = oa.write_archive([("m.safetensors", shard)], chunk_size=1 << 20)

    def gap(r):
        r["dst"][2] += 16

    with pytest.raises(archive.FormatError, match="cover"):
        plan.build_plan(archive.Archive(_rewrite_table(blob, gap)))

    def outside(r):
        r["off"][1] = 1 << 40

    with pytest.raises(archive.FormatError):
        archive.Archive(_rewrite_table(blob, outside))

    def wraps(r):                                  # off + clen would wrap past 2^64 into range
        r["off"][1] = (1 << 64) - 8

    def in_header(r):
        r["off"][1] = 4

    for hostile in (wraps, in_header):
        with pytest.raises(archive.FormatError, match="outside the payload"):
            archive.Archive(_rewrite_table(blob, hostile))

    def unknown_codec(r):
        r["codec"][1] = 7

    with pytest.raises(archive.FormatError, match="codec 7"):
        plan.build_plan(archive.Archive(_rewrite_table(blob, unknown_codec)))

    def wrong_plane_len(r):
        r["rlen"][1] -= 2

    with pytest.raises(archive.FormatError):
        plan.build_plan(archive.Archive(_rewrite_table(blob, wrong_plane_len)))


def test_planner_enforces_single_hop_sources():
    from lmz_b200 import archive, plan
    c0 = synth.llama_shard([0], 9, scale=0.125)
    c1 = c0.copy()
    info = oa.parse_safetensors(c0)[1]
    s, e = info["model.layers.0.mlp.up_proj.weight"]["offsets"]
    c1[s:e] = synth.perturbed_bf16(c0[s:e], 5)
    blob = oa.write_archive([("a/0.safetensors", c0), ("a/1.safetensors", c1)])
    ar = archive.Archive(blob)
    p = plan.build_plan(ar)
    assert p.piece_split[3] < p.piece_split[5], "expected refs/deltas in pass 2"
    assert p.base_bytes > 0
    delta = int(np.nonzero(ar.records["codec"] == 8)[0][0])
    other = int(np.nonzero(ar.records["codec"] == 4)[0][0])

    def chain(r):                                  # point the delta at a ref chunk's output
        pass

    recs = ar.records
    bad = bytearray(blob)
    struct.pack_into("<Q", bad, int(recs["off"][delta]), int(recs["dst"][other]))
    with pytest.raises(archive.CorruptArchive, match="points at another"):
        plan.build_plan(archive.Archive(bytes(bad)))
    bad = bytearray(blob)
    struct.pack_into("<Q", bad, int(recs["off"][delta]), ar.total)
    with pytest.raises(archive.CorruptArchive, match="outside"):
        plan.build_plan(archive.Archive(bytes(bad)))
