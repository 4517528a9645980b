"""The save path: BF16 safetensors bytes in HBM -> an lmz archive, chunk payloads framed on the
device.  The file must be, byte for byte in its payload and chunk records, what the checker's
writer produces for the same input -- and that writer is held to the reference's own
`lmz.api.compress` output by tests/test_oracle_vs_reference.py -- and it must decode back,
on the device and on the CPU, to the source."""
import numpy as np
import pytest

from oracle import archive as oa, synth

pytestmark = pytest.mark.gpu


def _same_as_checker(path, files, **kw):
    theirs = np.fromfile(path, dtype=np.uint8)
    ours = np.frombuffer(oa.write_archive(files, **kw), dtype=np.uint8)
    a, b = oa.Archive(ours), oa.Archive(theirs)
    assert a.records.size == b.records.size
    bad = np.nonzero(a.records != b.records)[0]
    assert bad.size == 0, (int(bad[0]), a.records[bad[0]], b.records[bad[0]])
    ta = int(np.frombuffer(ours[-40:-32].tobytes(), dtype="<u8")[0])
    tb = int(np.frombuffer(theirs[-40:-32].tobytes(), dtype="<u8")[0])
    assert ta == tb and (ours[:ta] == theirs[:tb]).all()
    return theirs


def _cases():
    rng = np.random.default_rng(2)
    shard = synth.llama_shard([0], 5, scale=0.25, vocab=2000, embed=True)            # weights + all-ones norms
    noise = rng.integers(0, 65536, 300_001, dtype=np.uint16).astype("<u2").view(np.uint8)   # nothing to gain: stored chunks
    e = (120 + rng.integers(0, 3, 200_000)).astype(np.uint16)                          # both planes low-entropy
    m = rng.integers(0, 4, 200_000).astype(np.uint16)
    narrow = ((e << 7) | m).astype("<u2").view(np.uint8)
    odd = synth.safetensors_bytes([("n", "BF16", (300_001,), noise), ("w", "BF16", (200_000,), narrow),
                                   ("t", "BF16", (7,), synth.normal_bf16((7,), 3))])
    return {"shard": shard, "odd": odd}


@pytest.mark.parametrize("name", ["shard", "odd"])
@pytest.mark.parametrize("kw", [dict(mapped=True), dict(chunk_size=1 << 20), dict(chunk_size=(1 << 18) + 2)],
                         ids=["mapped", "1MiB", "256KiB+2"])
def test_device_written_archive_equals_the_checkers(gpu, tmp_path, name, kw):
    import torch
    from lmz_b200 import decode, save
    src = _cases()[name]
    files = [("m.safetensors", src)]
    path = str(tmp_path / "out.lmz")
    stats = {}
    n = save.save_archive(path, [("m.safetensors", torch.from_numpy(src.copy()).cuda())],
                          chunk_size=kw.get("chunk_size", 64 << 10), mapped=bool(kw.get("mapped")), stats=stats)
    blob = _same_as_checker(path, files, **kw)
    assert n == blob.size and stats["payload_bytes"] > 0
    assert (oa.decode_archive(blob) == src).all()
    assert (decode.decode_archive(path).cpu().numpy() == src).all()


def test_two_members_and_what_the_writer_declines(gpu, tmp_path):
    import torch
    from lmz_b200 import decode, save
    a = synth.llama_shard([0], 5, scale=0.125, vocab=1000, embed=True)
    b = synth.llama_shard([1], 6, scale=0.125)
    path = str(tmp_path / "two.lmz")
    save.save_archive(path, [("a.safetensors", torch.from_numpy(a).cuda()), ("b.safetensors", torch.from_numpy(b).cuda())])
    _same_as_checker(path, [("a.safetensors", a), ("b.safetensors", b)], mapped=True, delta=False)
    assert (decode.decode_archive(path).cpu().numpy() == np.concatenate([a, b])).all()
    f32 = synth.safetensors_bytes([("f", "F32", (100,), np.zeros(400, np.uint8))])
    with pytest.raises(ValueError, match="BF16"):
        save.save_archive(path, [("f.safetensors", torch.from_numpy(f32).cuda())])
    with pytest.raises(ValueError, match="chunk_size"):
        save.save_archive(path, [("a.safetensors", torch.from_numpy(a).cuda())], chunk_size=8 << 20)
