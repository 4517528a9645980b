"""Write an lmz archive from bytes that are already in HBM.

The reference compresses on the CPU only (lmz/api.py:651-815 `compress`,
lmz/codec.py:914-1009 `encode_chunk`); this is the same work for the layout the GPU path is
quoted on -- BF16 safetensors members cut into small chunks (`lmz compress --mapped`, or any
chunk size below 2 MiB; from there up the reference conditions the sign/mantissa plane on
the exponent, lmz/codec.py:955-969, which this writer does not do) -- with the per-chunk
work on the device:

    split every chunk into its exponent and sign/mantissa planes   lmz/native/lmzcore.c:430-437
    rANS-code every plane with its own histogram                   lmzcore.c:882-979, 1318-1383
    keep a coded plane only where it pays                          lmz/codec.py:385-393, 396-398
    frame the chunk: plane lengths, then the planes                lmz/codec.py:989-1003
    crc32 of the chunk's plaintext                                 lmz/codec.py:931

and the container (records, manifest, footer; lmz/format.py:279-322) and the few bytes of
safetensors header on the host.  The chunk bytes are the reference encoder's: its early
exits for a hopeless plane (a sampled entropy estimate and a cost estimate from the
histogram, lmz/codec.py:356-372) only predict the comparison that is made here on the real
coded length, and for planes of at most 196 608 bytes -- where its sample is the whole
plane -- they never disagree with it.
"""
from __future__ import annotations

import ctypes
import json
import struct
import zlib

import numpy as np

from . import archive as fmt, gpu

MIN_GAIN_FLOOR = 1024            # lmz/codec.py:396-398: a coded stream must save max(1024, n >> 8) bytes
COND_MIN_BYTES = 2 << 20         # chunks of a mebi-element or more are exponent-conditioned by the reference
BATCH_BYTES = 512 << 20          # BF16 bytes framed per round of kernel launches


def _safetensors_layout(head: bytes):
    """(data start, {name: {dtype, shape, offsets}}) of a safetensors file from its first bytes
    (lmz/planner.py:196-237)."""
    if len(head) < 8:
        raise ValueError("not a safetensors file")
    n = struct.unpack_from("<Q", head, 0)[0]
    if n > len(head) - 8:
        raise ValueError("the safetensors header is longer than the bytes given")
    meta = json.loads(bytes(head[8:8 + n]).decode("utf-8"))
    tensors = {k: {"dtype": v["dtype"], "shape": list(v["shape"]),
                   "offsets": [8 + n + v["data_offsets"][0], 8 + n + v["data_offsets"][1]]}
               for k, v in meta.items() if k != "__metadata__"}
    return 8 + n, tensors


def _header_chunk(raw: bytes, level: int = 1):
    """(payload, codec, flags) of a run of container bytes, as the reference codes them when it
    has no zstd (lmz/codec.py:1005-1009 over _encode_stream :373-393): deflate where that saves
    max(1024, n >> 8) bytes, else stored."""
    n = len(raw)
    best = zlib.compress(raw, min(max(level, 1), 9))
    if len(best) > n - (n >> 5) or len(best) + max(MIN_GAIN_FLOOR, n >> 8) >= n:
        return raw, fmt.CODEC_STORED, 0
    return best, fmt.CODEC_ZSTD, fmt.METHOD_DEFLATE


def save_archive(path, members, chunk_size: int = 64 << 10, mapped: bool = True, stats=None):
    """Write `members` = [(member path, CUDA uint8 tensor holding a BF16 safetensors file)] as
    an lmz archive.  Every tensor must be BF16.  Returns the number of bytes written.
    `stats`, a dict, receives `device_s` (the kernels: split + encode + frame + checksum, timed
    with CUDA events) and `payload_bytes`.  The framed payload comes back through a page-locked
    buffer that the module keeps between calls and goes to the file batch by batch."""
    if chunk_size < (64 << 10) or chunk_size >= COND_MIN_BYTES or chunk_size % 2:
        raise ValueError("chunk_size must be even, at least 64 KiB and below 2 MiB")
    with open(path, "wb") as f:
        return _write_archive(f, members, chunk_size, mapped, stats)


def _write_archive(f, members, chunk_size, mapped, stats):
    import torch
    lib = gpu.library()
    recs_parts, metas, base = [], [], 0                      # record arrays, in file order
    device_s = 0.0
    f.write(bytes(fmt.HEADER.size))                          # the header goes in last: it holds the total size

    def add_records(dst, rlen, crc, codec, esize, flags, clen):
        part = np.zeros(len(dst), dtype=fmt.RECORD)
        part["dst"], part["rlen"], part["crc"], part["codec"] = dst, rlen, crc, codec
        part["esize"], part["flags"], part["clen"] = esize, flags, clen
        recs_parts.append(part)

    for mpath, data in members:
        if not (type(data).__module__.startswith("torch") and data.is_cuda and data.dtype == torch.uint8):
            raise ValueError("a member must be a CUDA uint8 tensor")
        flat = data.reshape(-1)
        size = int(flat.numel())
        head = bytes(flat[:min(size, 8)].cpu().numpy())
        hlen = struct.unpack("<Q", head)[0] if len(head) == 8 else 0
        head = bytes(flat[:min(size, 8 + hlen)].cpu().numpy())
        start, tensors = _safetensors_layout(head)
        if any(t["dtype"] != "BF16" for t in tensors.values()):
            raise ValueError("this writer takes BF16 members only")
        if (size - start) % 2:
            raise ValueError("a BF16 data area has an odd number of bytes")
        # the header: byte chunks of at most chunk_size (lmz/planner.py:582-652)
        for s in range(0, start, chunk_size):
            raw = head[s:min(s + chunk_size, start)]
            payload, codec, flags = _header_chunk(raw)
            add_records([base + s], [len(raw)], [zlib.crc32(raw) & 0xFFFFFFFF], [codec], [1], [flags], [len(payload)])
            f.write(payload)
        # the data area: BF16 chunks, framed on the device
        body = flat[start:]
        nbytes = int(body.numel())
        # (in batches: the coder's slots take a little over twice the bytes they code)
        batch = max(1, BATCH_BYTES // chunk_size) * chunk_size
        for b0 in range(0, nbytes, batch):
            part = body[b0:min(b0 + batch, nbytes)]
            payload, clen, codec, flags, crc, kernel_s = _frame_bf16(lib, part, chunk_size)
            device_s += kernel_s
            at = np.arange(clen.size, dtype=np.int64) * chunk_size
            add_records(base + start + b0 + at, np.minimum(chunk_size, int(part.numel()) - at), crc, codec,
                        np.full(clen.size, 2), flags, clen)
            f.write(memoryview(payload))                      # the chunks' payloads back to back, in record order
        metas.append({"path": mpath, "size": size, "dst": base, "kind": "safetensors", "mode": 0o644, "crc": 0,
                      "tensors": {k: dict(v) for k, v in tensors.items()}})
        base += size
    recs = np.concatenate(recs_parts) if recs_parts else np.zeros(0, dtype=fmt.RECORD)
    clens = recs["clen"].astype(np.int64)
    recs["off"] = fmt.HEADER.size + np.cumsum(clens) - clens
    off = fmt.HEADER.size + int(clens.sum())
    manifest = {"version": 1, "tool": "lmz-b200 device writer", "level": 1, "chunk_size": chunk_size,
                "mapped": bool(mapped), "aligned": False, "entropy": "deflate", "checksum": "crc32",
                "total_size": base, "members": metas, "chunks": int(recs.size), "table_raw_len": int(recs.nbytes)}
    table_c = zlib.compress(recs.tobytes(), 3)
    man_c = zlib.compress(json.dumps(manifest, separators=(",", ":")).encode(), 3)
    f.write(table_c)
    f.write(man_c)
    f.write(fmt.FOOTER.pack(off, len(table_c), off + len(table_c), len(man_c), fmt.TAIL))
    f.seek(0)
    f.write(fmt.HEADER.pack(fmt.MAGIC, 6, fmt.FLAG_PAGE_MAPPED if mapped else 0, base, 0, 0))
    if stats is not None:
        stats.update(device_s=device_s, payload_bytes=off - fmt.HEADER.size)
    return off + len(table_c) + len(man_c) + fmt.FOOTER.size


_host = {}


def _host_buffer(nbytes: int):
    """A page-locked host buffer of at least `nbytes`, kept between calls (allocating one is slow)."""
    import torch
    buf = _host.get("buf")
    if buf is None or buf.numel() < nbytes:
        _host["buf"] = buf = torch.empty(max(nbytes, 64 << 20), dtype=torch.uint8).pin_memory()
    return buf


def _frame_bf16(lib, body, chunk_size: int):
    """Chunk payloads of one BF16 data area, on the device.  Returns host arrays: the payload
    bytes of all chunks back to back (a view of the module's page-locked buffer: use it before
    the next call), per chunk its length, codec id, flags and crc32, and the kernels' seconds."""
    import torch
    dev = body.device
    nbytes = int(body.numel())
    nfull, tail = divmod(nbytes, chunk_size)
    nchunks = nfull + (1 if tail else 0)
    with torch.cuda.device(dev):
        cs = torch.cuda.current_stream(dev).cuda_stream
        e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        e0.record()
        planes = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        lens = torch.zeros(2 * nchunks, dtype=torch.int32, device=dev)
        rc = lib.lmz_gpu_split_bf16_dev(body.data_ptr(), nbytes, chunk_size, planes.data_ptr(), cs)
        if rc != gpu.OK:
            raise RuntimeError(f"plane split failed ({rc}): {gpu.last_error()}")
        # every plane is coded; which coded planes are kept is decided on their lengths
        slot = lib.lmz_gpu_encode_slot_bytes(chunk_size // 2)
        slot_tail = lib.lmz_gpu_encode_slot_bytes(tail // 2) if tail else 0
        slots = torch.empty(2 * nfull * slot + 2 * slot_tail + 512, dtype=torch.uint8, device=dev)
        sbase = (slots.data_ptr() + 511) & ~511
        if nfull:
            rc = lib.lmz_gpu_encode_batch_dev(planes.data_ptr(), 2 * nfull, chunk_size // 2, sbase,
                                              lens.data_ptr(), cs)
        if rc == gpu.OK and tail:
            rc = lib.lmz_gpu_encode_batch_dev(planes.data_ptr() + nfull * chunk_size, 2, tail // 2,
                                              sbase + 2 * nfull * slot, lens.data_ptr() + 8 * nfull, cs)
        if rc != gpu.OK:
            raise RuntimeError(f"plane encode failed ({rc}): {gpu.last_error()}")
        meta = torch.zeros((nchunks, 4), dtype=torch.int32, device=dev)          # clen, codec, flags, crc
        rc = lib.lmz_gpu_frame_bf16_dev(body.data_ptr(), nbytes, chunk_size, lens.data_ptr(), meta.data_ptr(),
                                        None, None, None, None, cs)              # pass 1: sizes and choices
        if rc != gpu.OK:
            raise RuntimeError(f"chunk framing failed ({rc}): {gpu.last_error()}")
        clen = meta[:, 0].to(torch.int64)
        offs = (torch.cumsum(clen, 0) - clen).contiguous()
        e1.record()
        total = int(clen.sum())                                                  # (the host needs the size: a sync)
        out = torch.empty(total + 16, dtype=torch.uint8, device=dev)
        e2.record()
        rc = lib.lmz_gpu_frame_bf16_dev(body.data_ptr(), nbytes, chunk_size, lens.data_ptr(), meta.data_ptr(),
                                        planes.data_ptr(), ctypes.c_void_p(sbase), offs.data_ptr(),
                                        out.data_ptr(), cs)                      # pass 2: the bytes
        if rc != gpu.OK:
            raise RuntimeError(f"chunk framing failed ({rc}): {gpu.last_error()}")
        from . import decode
        tabs = decode._crc_tables(lib, dev)
        rc = lib.lmz_gpu_crc32_chunks_dev(body.data_ptr(), nbytes, chunk_size, tabs.data_ptr(),
                                          meta.data_ptr(), cs)
        if rc != gpu.OK:
            raise RuntimeError(f"chunk checksum failed ({rc}): {gpu.last_error()}")
        e3.record()
        host = _host_buffer(total)[:total]
        host.copy_(out[:total], non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        m = meta.cpu().numpy()
        kernel_s = (e0.elapsed_time(e1) + e2.elapsed_time(e3)) / 1e3
        return (host.numpy(), m[:, 0].astype(np.int64), m[:, 1], m[:, 2],
                m[:, 3].astype(np.int64) & 0xFFFFFFFF, kernel_s)
