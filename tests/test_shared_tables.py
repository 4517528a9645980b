"""The shared-table archive option: BF16 chunks whose exponent planes are coded against one
frequency table per run of chunks (the format lever the reference proposes in
docs/gpu-residency-handover.md:37-66 and for which scratchpad/gpu/shared_enc.c is the
encoder; the chunk layout, `CODEC_BF16T`, is this repository's).  CPU: the checker's
writer and decoder, and the planner.  GPU: the fused shared-table instance against the
checker and the source bytes."""
import struct
import zlib

import numpy as np
import pytest

from oracle import archive as oa, codec, synth


@pytest.fixture(scope="module")
def shard():
    return synth.llama_shard([0], 5, scale=0.25, vocab=2000, embed=True)


def test_checker_writes_and_reads_shared_table_archives(shard, orc):
    own = oa.write_archive([("m.safetensors", shard)], mapped=True)
    shared = oa.write_archive([("m.safetensors", shard)], mapped=True, shared_tables=160)
    a = oa.Archive(shared)
    assert a.flags & codec.FLAG_SHARED_TABLES and a.manifest["shared_tables"]["count"] >= 2
    assert (a.records["codec"] == codec.CODEC_BF16T).sum() >= 0.9 * a.records.size
    assert len(shared) < len(own), "one table per run must be smaller than one per 64 KiB chunk"
    assert (oa.decode_archive(shared, lib=orc) == shard).all()
    # a shared-table stream is an ordinary stream once its table is put back in front
    c = a.records[np.nonzero(a.records["codec"] == codec.CODEC_BF16T)[0][3]]
    pl = a.payload(c)
    len0, len1, toff = codec.BF16T_HDR.unpack_from(pl, 0)
    stream = bytes(a.blob[toff:toff + 516]) + bytes(pl[16:16 + len0])
    exp = orc.rans_decode(stream, int(c["rlen"]) // 2)
    d = int(c["dst"])
    assert (exp == orc.split_bf16(shard[d:d + int(c["rlen"])])[0]).all()
    # uncorrelated runs keep their own tables (the choice is by measured cross-entropy)
    rng = np.random.default_rng(3)
    mixed = []
    for i in range(24):                            # exponent alphabets that move from chunk to chunk
        e = (rng.integers(0, 6, 32768) + 10 * i).astype(np.uint16)
        b = rng.integers(0, 256, 32768).astype(np.uint16)
        mixed.append((((b & 0x80) << 8) | (e << 7) | (b & 0x7F)).astype("<u2").view(np.uint8))
    src = synth.safetensors_bytes([("w", "BF16", (24 * 32768,), np.concatenate(mixed))])
    arc = oa.Archive(oa.write_archive([("m.safetensors", src)], mapped=True, shared_tables=8))
    assert (arc.records["codec"] == codec.CODEC_BF16T).sum() == 0


def test_planner_lists_shared_table_chunks_table_by_table(shard):
    from lmz_b200 import archive, plan
    blob = oa.write_archive([("a.safetensors", shard), ("b.safetensors", synth.llama_shard([1], 6, scale=0.125))],
                            mapped=True, shared_tables=100)
    ar = archive.Archive(blob)
    p = plan.build_plan(ar)
    nt = int((ar.records["codec"] == archive.CODEC_BF16T).sum())
    assert nt > 0 and p.n_fused_t % plan.T_GROUP == 0 and p.n_fused_t >= nt
    tj = p.fused_jobs[p.n_fused:]
    assert int((tj["n"] > 0).sum()) == nt
    for c in range(0, tj.size, plan.T_GROUP):                     # one table per thread block
        assert np.unique(tj["flags"][c:c + plan.T_GROUP]).size == 1
    assert p.tables.shape == (int(tj["flags"].max()) + 1, plan.TABLE_STRIDE)
    assert (p.tables[:, :2] == np.frombuffer(b"R1", dtype=np.uint8)).all()
    # a slice of the archive plans only its own chunks, and still finds tables that lie before it
    g = np.arange(ar.records.size)[150:260]
    r = ar.records
    lo, hi = int(r["off"][g].min()), int((r["off"][g].astype(np.int64) + r["clen"][g]).max())
    ps = plan.build_plan(ar, select=g, payload_range=(lo, hi))
    assert int((ps.fused_jobs["n"][ps.n_fused:] > 0).sum()) == int((r["codec"][g] == archive.CODEC_BF16T).sum())
    # hostile: a table offset outside the payload region
    first = int(np.nonzero(r["codec"] == archive.CODEC_BF16T)[0][0])
    bad = bytearray(blob)
    struct.pack_into("<Q", bad, int(r["off"][first]) + 8, len(blob))
    with pytest.raises(archive.CorruptArchive, match="outside the payload"):
        plan.build_plan(archive.Archive(bytes(bad)))
    bad = bytearray(blob)
    struct.pack_into("<I", bad, int(r["off"][first]) + 4, 7)       # plane 1 length != element count
    with pytest.raises(archive.CorruptArchive, match="inconsistent"):
        plan.build_plan(archive.Archive(bytes(bad)))


@pytest.mark.gpu
@pytest.mark.parametrize("run", [2, 64, 80, 1000])
def test_gpu_decodes_shared_table_archives(gpu, shard, orc, run):
    from lmz_b200 import archive, decode
    src = [("a.safetensors", shard), ("b.safetensors", synth.llama_shard([1], 6, scale=0.125))]
    whole = np.concatenate([d for _, d in src])
    blob = oa.write_archive(src, mapped=True, shared_tables=run)
    want = oa.decode_archive(blob, lib=orc)
    assert (want == whole).all()
    for checksum in (True, False):
        dec = decode.ArchiveDecoder(blob, checksum=checksum)
        assert dec.plan.n_fused_t > 0
        dec.run()
        dec.check()
        got = dec.output.cpu().numpy()
        assert (got == want).all(), f"first difference at byte {int(np.nonzero(got != want)[0][0])}"
        if checksum:
            crcs = dec.chunk_crcs()
            for i, rec in enumerate(dec.archive.records):
                d, n = int(rec["dst"]), int(rec["rlen"])
                assert int(crcs[i]) == (zlib.crc32(whole[d:d + n]) & 0xFFFFFFFF), f"crc of chunk {i}"
    # sliced upload and the file pipeline take the same path
    pd = decode.PipelinedDecoder(blob, nslices=3)
    assert (pd.run_from_file().cpu().numpy() == whole).all()
    pd.check()


@pytest.mark.gpu
def test_gpu_reports_damage_in_shared_table_archives(gpu, shard):
    from lmz_b200 import archive, decode
    blob = oa.write_archive([("m.safetensors", shard)], mapped=True, shared_tables=80)
    ar = oa.Archive(blob)
    t = np.nonzero(ar.records["codec"] == codec.CODEC_BF16T)[0]
    toff = codec.BF16T_HDR.unpack_from(ar.payload(ar.records[t[5]]), 0)[2]
    for what, pos in (("table magic", toff), ("table frequency", toff + 4 + 2 * 118),
                      ("coded word", int(ar.records["off"][t[7]]) + 16 + 40)):
        bad = bytearray(blob)
        bad[pos] ^= 0x21
        dec = decode.ArchiveDecoder(bytes(bad))
        dec.run()
        with pytest.raises(archive.CorruptArchive):
            dec.check()
