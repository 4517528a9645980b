#!/usr/bin/env python
"""Benchmark: decoded plaintext GB/s of an lmz archive of a Llama-3.1-8B-shaped
BF16 model (random-init, seeded) on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

A step is one decode of the whole archive (every chunk) into HBM.  `value` is
measured with the compressed bytes already resident in HBM (CUDA events around
exactly K steps, max over ranks); `e2e` includes, every step, the host->device
copy of the archive from pinned memory and the device->host read of the
per-chunk verdicts.  Each rank decodes its own full replica (weak scaling; no
collective on the data path).  `--impl reference` times the reference's own
CPU decoder (its C core compiled into oracle/_ref, driven by all host threads)
on a bounded sample of the same archive.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    # the headline configuration: 32 layers, hidden 4096, FFN 14336, 8 KV heads of 128, vocab 128256
    "llama-3.1-8b": dict(layers=32, hidden=4096, ffn=14336, kv=1024, vocab=128256, shards=4),
    "llama-8layer": dict(layers=8, hidden=4096, ffn=14336, kv=1024, vocab=1024, shards=1),
    "llama-2layer": dict(layers=2, hidden=4096, ffn=14336, kv=1024, vocab=1024, shards=1),
    "llama-tiny": dict(layers=2, hidden=1024, ffn=3584, kv=256, vocab=8000, shards=2),
    # the single 4096 x 14336 BF16 tensor (117 MB) of the first configuration
    "config1-tensor": dict(kind="spec", spec=[[("w", "BF16", (4096, 14336))]]),
    # other configurations (not the headline): each rank's own 1/8 tensor-parallel slice of a
    # 70B BF16 model (17.6 GB) or of an FP32 XLM-R-large container, and a 3-checkpoint BF16
    # delta chain on the Pythia-160m shapes
    "llama-3-70b-tp8": dict(layers=80, hidden=8192, ffn=28672, kv=1024, vocab=128256, shards=4, tp=8),
    "xlmr-large-f32-tp8": dict(kind="xlmr", layers=24, hidden=1024, ffn=4096, vocab=250002, tp=8),
    "xlmr-large-f32": dict(kind="xlmr", layers=24, hidden=1024, ffn=4096, vocab=250002),
    "pythia-160m-chain": dict(kind="chain", layers=12, hidden=768, ffn=3072, vocab=50304),
}
METRIC = "decoded plaintext GB/s per B200 & per box (1/2/4/8 GPU), byte-exact vs CPU"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--model", default="llama-3.1-8b", choices=sorted(MODELS) + ["stress"],
                    help="a model archive, or 'stress': the decoder stress batch matrix (batch decode entry point)")
    ap.add_argument("--stress-pool", type=int, default=256, help="distinct streams per (distribution, length)")
    ap.add_argument("--stress-lengths", default="1,17,4096,65536,1048576,4194304")
    ap.add_argument("--stress-batches", default="1,7,64,4096")
    ap.add_argument("--layout", default="mapped", choices=("mapped", "default"),
                    help="mapped = 64 KiB blocks (lmz compress --mapped); default = 8 MiB chunks")
    ap.add_argument("--chunk-size", type=int, default=0, help="override the layout's chunk size")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--shared-tables", type=int, default=0,
                    help="write the archive with the shared-table option: one exponent table per run of N BF16 chunks "
                         "(a multiple of 80 fills the decoder's thread blocks)")
    ap.add_argument("--no-crc", action="store_true", help="skip the per-chunk crc32")
    ap.add_argument("--no-fuse", action="store_true",
                    help="decode planes to scratch and merge in k_finish instead of the fused kernel")
    ap.add_argument("--no-cache", action="store_true")
    ap.add_argument("--cpu-sample-mb", type=int, default=2048)
    return ap.parse_args()


def workload_name(a) -> str:
    cs = a.chunk_size or ((64 << 10) if a.layout == "mapped" else (8 << 20))
    dt = "f32" if MODELS[a.model].get("kind") == "xlmr" else "bf16"
    st = f", one shared exponent table per {a.shared_tables} chunks" if getattr(a, "shared_tables", 0) else ""
    return f"{a.model} {dt} N(0,0.02) seed {a.seed}, lmz archive, {cs >> 10} KiB chunks{st}"


def per_rank_archives(a) -> bool:
    """Tensor-parallel configurations: every rank decodes an archive of its own."""
    return MODELS[a.model].get("tp", 1) > 1


def archive_key(model: str, layout: str, chunk_size: int, seed: int, shared_tables: int = 0) -> str:
    return f"lmzb200-{model}-{layout}-{chunk_size}-{seed}" + (f"-t{shared_tables}" if shared_tables else "")


def build_archive(model: str, layout: str, chunk_size: int = 0, seed: int = 1, nproc=None,
                  want_files: bool = False, shared_tables: int = 0):
    """The synthetic archive of a workload, written by the checker's reference-exact
    writer.  Returns (archive bytes, files) where files is [(relative path, bytes)] of
    the model's source files when `want_files` (else None)."""
    from oracle import archive as oa, bigwrite, synth
    m = dict(MODELS[model])
    kind = m.pop("kind", "llama")
    mapped = layout == "mapped"
    cs = chunk_size or None
    if kind == "chain":
        files = [(f"step{i}/model.safetensors", f) for i, f in enumerate(synth.delta_chain_files(**m))]
        blob = np.frombuffer(oa.write_archive(files, chunk_size=cs, mapped=mapped, shared_tables=shared_tables),
                             dtype=np.uint8)
        return blob, (files if want_files else None)
    spec = m["spec"] if kind == "spec" else synth.xlmr_spec(**m) if kind == "xlmr" else synth.llama_spec(**m)
    blob, layouts = bigwrite.write_model_archive(spec, seed=seed, chunk_size=cs, mapped=mapped, nproc=nproc,
                                                 shared_tables=shared_tables)
    files = None
    if want_files:
        files = [(f"model-{i + 1:05d}-of-{len(layouts):05d}.safetensors", lay.bytes(0, lay.size))
                 for i, lay in enumerate(layouts)]
    return blob, files


def model_files_and_archive(model: str, layout: str, seed: int = 1):
    """(source files, archive, pin key) -- what tests/golden/make_bench_pins.py compares
    with the reference's own writer."""
    blob, files = build_archive(model, layout, 0, seed, want_files=True)
    return files, blob, archive_key(model, layout, 0, seed)


def archive_digests(blob) -> dict:
    """sha256 of the payload region and of the raw chunk records."""
    import hashlib
    from oracle import archive as oa
    recs = oa.Archive(blob).records
    toff = int(np.frombuffer(np.asarray(blob[-40:-32]).tobytes(), dtype="<u8")[0])
    return {"payload_sha256": hashlib.sha256(memoryview(np.ascontiguousarray(blob[32:toff]))).hexdigest(),
            "records_sha256": hashlib.sha256(recs.tobytes()).hexdigest()}


def pin_status(key: str, blob) -> str:
    """Compare an archive with the digests tests/golden/bench_pins.json holds for it
    (written from the reference's own `lmz.api.compress` output on the same files)."""
    try:
        with open(os.path.join(ROOT, "tests", "golden", "bench_pins.json")) as f:
            pin = json.load(f).get(key)
    except OSError:
        pin = None
    if pin is None:
        return ("no pin: the shared-table option is this repository's format extension" if "-t" in key.rsplit("-", 1)[-1]
                else "no pin for this workload")
    d = archive_digests(blob)
    if d["payload_sha256"] != pin["payload_sha256"] or d["records_sha256"] != pin["records_sha256"]:
        raise SystemExit(f"the generated archive {key} differs from the reference-written pin")
    return "payload and chunk records sha256-equal to the reference writer's output"


def get_archive(a, rank: int, barrier) -> np.ndarray:
    """The benchmark archive as a numpy byte array, generated once per box and
    cached in /dev/shm (ranks other than 0 wait for rank 0), and checked there against
    its reference-written pin; the verdict is kept beside the cached file."""
    own = per_rank_archives(a)
    seed = a.seed * 64 + rank if own else a.seed
    key = archive_key(a.model, a.layout, a.chunk_size, seed, getattr(a, "shared_tables", 0))
    cache = os.path.join("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp", key + ".lmz")
    if (own or rank == 0) and (a.no_cache or not os.path.exists(cache)):
        t = time.time()
        nproc = max(1, (os.cpu_count() or 1) // int(os.environ.get("LOCAL_WORLD_SIZE", "1"))) if own else None
        blob, _ = build_archive(a.model, a.layout, a.chunk_size, seed, nproc=nproc,
                                shared_tables=getattr(a, "shared_tables", 0))
        with open(cache + ".pin", "w") as f:
            f.write(pin_status(key, blob))
        tmp = cache + f".{os.getpid()}"
        blob.tofile(tmp)
        os.replace(tmp, cache)
        print(f"[bench] wrote {cache}: {blob.size / 1e9:.2f} GB in {time.time() - t:.1f}s",
              file=sys.stderr)
    barrier()
    # one copy of the archive per box: every rank maps the same pages
    return np.memmap(cache, dtype=np.uint8, mode="r+")


def archive_pin(a, rank: int = 0) -> str:
    own = per_rank_archives(a)
    key = archive_key(a.model, a.layout, a.chunk_size, a.seed * 64 + rank if own else a.seed,
                      getattr(a, "shared_tables", 0))
    try:
        with open(os.path.join("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp", key + ".lmz.pin")) as f:
            return f.read()
    except OSError:
        return "unknown"


class ClockSampler:
    """SM clock and throttle reasons of one GPU while a region runs: read through NVML
    (read-only queries) every 10 ms by a thread of this process, so that even a timed region
    of a few tens of milliseconds gets samples; nvidia-smi in a loop where NVML cannot be
    loaded."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index
        self.nvml = self.handle = self.t = None
        self.stop = threading.Event()

    def _open_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        handle = None
        try:                                   # the CUDA device's own NVML handle, whatever the visible-device order
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            handle = None
        if handle is None:
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        self.nvml, self.handle = pynvml, handle
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

    def _sample(self):
        n, h = self.nvml, self.handle
        mhz = float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))
        bits = int(n.nvmlDeviceGetCurrentClocksEventReasons(h))
        flags = [bool(bits & m) for m in (n.nvmlClocksEventReasonHwSlowdown, n.nvmlClocksEventReasonHwThermalSlowdown,
                                          n.nvmlClocksEventReasonSwThermalSlowdown, n.nvmlClocksEventReasonSwPowerCap)]
        self.rows.append([mhz, self.max_mhz, 0.0] + ["Active" if f else "Not Active" for f in flags])

    def _poll(self):
        while not self.stop.is_set():
            try:
                self._sample()
            except Exception:
                return
            self.stop.wait(0.01)

    def __enter__(self):
        try:
            self._open_nvml()
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.nvml is not None:
            self.stop.set()
            self.t.join(timeout=2)
            return
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(self.NAMES, r[3:7]):
                if str(v).lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


_CPU = {}


def _cpu_work(span):
    """Decode records[lo:hi] of the sample in a worker process (reference C core)."""
    from oracle import archive as oa
    ar, picks, lib = _CPU["ar"], _CPU["picks"], _CPU["lib"]
    done = 0
    for i in picks[span[0]:span[1]]:
        c = ar.records[i]
        oa._decode_plain(ar, c, True, lib)
        done += int(c["rlen"])
    return done


def cpu_decode_sample(blob, sample_mb: int, threads: int, lib_kind: str):
    """Time the CPU decoder over the first `sample_mb` of plaintext chunks on `threads`
    cores.  Worker processes rather than threads: the reference's Python driver is
    GIL-bound on small chunks (it caps itself at 2 threads there, lmz/api.py:1001-1017),
    and the baseline should show what its C core does with every core.
    Returns (GB/s, description, kind)."""
    import multiprocessing as mp
    from oracle import archive as oa, codec, native
    lib = native.ref() if lib_kind == "reference" else native.oracle()
    if lib is None:
        lib, lib_kind = native.oracle(), "port"
    ar = oa.Archive(blob)
    picks, total = [], 0
    for i, c in enumerate(ar.records):
        if c["codec"] in (codec.CODEC_REF, codec.CODEC_DELTA):
            continue
        picks.append(i)
        total += int(c["rlen"])
        if total >= sample_mb << 20:
            break
    _CPU.update(ar=ar, picks=picks, lib=lib)
    nspan = threads * 8
    edges = np.linspace(0, len(picks), nspan + 1).astype(int)
    spans = [(int(a), int(b)) for a, b in zip(edges[:-1], edges[1:]) if b > a]
    with mp.get_context("fork").Pool(threads) as pool:
        pool.map(_cpu_work, [(0, min(len(picks), threads))])       # warm the workers
        t = time.perf_counter()
        done = sum(pool.map(_cpu_work, spans, chunksize=1))
        dt = time.perf_counter() - t
    what = (f"first {len(picks)} chunks ({done / 1e6:.0f} MB plaintext) of the same archive, "
            f"decode + crc32, {threads} worker processes, C core = {lib_kind}")
    return done / dt / 1e9, what, lib_kind


_RESULT = sys.stdout


def own_stdout():
    """Keep stdout for the one JSON line: libraries that write to file descriptor 1
    (NCCL prints its version banner there) are sent to stderr instead."""
    global _RESULT
    sys.stdout.flush()
    _RESULT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict):
    _RESULT.write(json.dumps(line) + "\n")
    _RESULT.flush()


def main():
    a = parse_args()
    own_stdout()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.model == "stress":
        return run_stress(a, rank)
    if a.impl == "reference":
        return run_reference(a, rank)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    def barrier():
        if world > 1:
            dist.barrier()

    from lmz_b200 import decode, gpu
    ok, why = gpu.available()
    if not ok:
        raise SystemExit(f"the CUDA library is unavailable: {why}")
    blob = get_archive(a, rank, barrier)
    dec = decode.ArchiveDecoder(blob, checksum=not a.no_crc, fuse=not a.no_fuse)
    p = dec.plan
    plain, coded = p.total, p.coded_bytes

    # ---- warm-up + correctness gate ---------------------------------------------------
    for _ in range(max(a.warmup, 3)):
        dec.run()
    dec.check()
    verify_sample(dec, blob)
    barrier()
    torch.cuda.synchronize()

    # ---- timed region: K whole-archive decodes, inputs resident -------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        e0.record()
        for _ in range(a.steps):
            dec.run()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    barrier()
    dec.check()
    t_all = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    ms = float(t_all.item())
    value = world * plain * a.steps / (ms / 1e3) / 1e9

    # ---- per-phase device times (each phase launched alone, CUDA events) ---------------
    phase_ms = {}
    for name, mask in (("stream_decode", 1), ("cond", 2), ("finish", 4), ("verdict", 8), ("fused", 16)):
        ts = []
        for _ in range(3):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(); dec.run(phases=mask); s1.record()
            torch.cuda.synchronize()
            ts.append(s0.elapsed_time(s1))
        phase_ms[name] = float(np.mean(ts[1:]))
    dec.run()

    # ---- end to end: pinned host archive -> device, decode, verdicts back ---------------
    # The public host-to-HBM call: the upload is cut into slices so slice i decodes
    # while slice i+1 is still crossing PCIe.
    pd = decode.PipelinedDecoder(dec.archive, checksum=not a.no_crc)
    pinned = pin_host(np.asarray(blob[:int(dec.archive.table_off)]))
    nres = sum(s.plan.chunks.size + 1 for s in pd.slices)
    host_res = torch.empty(nres, dtype=torch.int32).pin_memory()

    def e2e_step():
        pd.run_from_host(pinned)
        pos = 0
        for s in pd.slices:
            nck = s.plan.chunks.size
            host_res[pos:pos + nck].copy_(s.d_chunk_crc[:nck], non_blocking=True)
            host_res[pos + nck:pos + nck + 1].copy_(s.d_any_bad, non_blocking=True)
            pos += nck + 1
        torch.cuda.synchronize()
        pos = 0
        for s in pd.slices:
            pos += s.plan.chunks.size + 1
            if int(host_res[pos - 1]) != 0:
                raise SystemExit("end-to-end step reported a corrupt chunk")

    e2e_step()                                     # warm-up, and a full verification
    pd.check()
    if not torch.equal(pd.d_out[:plain], dec.output):
        raise SystemExit("pipelined decode differs from the resident decode")
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    t_all = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    e2e_s = float(t_all.item())
    e2e_value = world * plain * a.steps / e2e_s / 1e9
    h2d_bytes, nslices = int(pd.h2d_bytes), len(pd.slices)

    # ---- N = 1: a whole load from the file, nothing prepared (open, plan, stage, upload, decode, check) ----
    cold = None
    if world == 1:
        del pd
        runs = []
        for _ in range(2):
            st = {}
            t0 = time.perf_counter()
            got = decode.load_archive(blob.filename, checksum=not a.no_crc, stats=st)
            runs.append((time.perf_counter() - t0, st))
            if not torch.equal(got, dec.output):
                raise SystemExit("load_archive differs from the resident decode")
            del got
        best = min(runs, key=lambda r: r[0])
        cold = {"value": round(plain / best[0] / 1e9, 2), "unit": "GB/s", "seconds": round(best[0], 4),
                "first_call_seconds": round(runs[0][0], 4),
                "open_s": round(best[1]["open_s"], 4), "plan_s": round(best[1]["plan_s"], 4),
                "h2d_bytes": int(best[1]["h2d_bytes"]), "slices": best[1]["slices"],
                "api": "lmz_b200.decode.load_archive(path): page-cached file -> mapped -> planned slice by slice "
                       "under the copies -> pageable-to-pinned staging -> HBM -> decode -> every verdict checked"}

    # ---- N > 1: the one archive partitioned over the ranks (no collective on the data path) ----
    part = gather = None
    if world > 1 and not per_rank_archives(a):
        from lmz_b200 import multi
        del pd
        sd = multi.ShardedDecoder(dec.archive, rank, world, checksum=not a.no_crc)
        for _ in range(3):
            sd.run()
        sd.check()
        if not torch.equal(sd.owned(), dec.output[sd.range[0]:sd.range[1]]):
            raise SystemExit("a rank's share of the partitioned decode differs from the full decode")
        barrier()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(a.steps):
            sd.run()
        p1.record()
        torch.cuda.synchronize()
        t_all = torch.tensor([p0.elapsed_time(p1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
        pms = float(t_all.item()) / a.steps
        # end to end: every rank uploads only the stretch of the payload its own chunks lie in,
        # from its own page-locked registration of that stretch, decodes, reads its verdicts back
        lo, hi = sd.payload_range if sd.payload_range else (0, 0)
        unpin_host(pinned)                       # the whole-archive registration of the replica leg
        own_pin = pin_host(np.asarray(blob[lo:hi]))
        nck = sd.decoder.plan.chunks.size
        res = torch.empty(nck + 1, dtype=torch.int32).pin_memory()

        def part_step():
            sd.decoder.upload(own_pin, non_blocking=True)
            sd.run()
            res[:nck].copy_(sd.decoder.d_chunk_crc[:nck], non_blocking=True)
            res[nck:].copy_(sd.decoder.d_any_bad, non_blocking=True)
            torch.cuda.synchronize()
            if int(res[nck]) != 0:
                raise SystemExit("partitioned end-to-end step reported a corrupt chunk")

        part_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            part_step()
        t_all = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
        pe2e = float(t_all.item()) / a.steps
        h2d_all = torch.tensor([hi - lo], dtype=torch.float64, device="cuda")
        dist.all_reduce(h2d_all, op=dist.ReduceOp.SUM)
        part = {"value": round(plain / (pms / 1e3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(pms, 3),
                "efficiency_vs_replicas": round(plain / (pms / 1e3) / 1e9 / value, 4),
                "e2e": {"value": round(plain / pe2e / 1e9, 2), "unit": "GB/s", "seconds": round(pe2e, 4),
                        "h2d_bytes_per_step": int(h2d_all.item()), "d2h_bytes_per_step": int((nck + 1) * 4 * world),
                        "h2d_gbs_all_ranks": round(float(h2d_all.item()) / pe2e / 1e9, 1)},
                "what": f"one archive, chunks partitioned over {world} GPUs by output range, each rank uploading "
                        f"and decoding only its share into its own HBM (no collective)"}
        unpin_host(own_pin)
        del sd, own_pin
        # optional full replica on every rank: equal output slices, one in-place NCCL all-gather
        sr = multi.ShardedDecoder(dec.archive, rank, world, checksum=not a.no_crc, replica=True)
        sr.run()
        sr.check()
        sr.all_gather()
        torch.cuda.synchronize()
        if not torch.equal(sr.decoder.d_out[:plain], dec.output):
            raise SystemExit("the gathered replica differs from the full decode")
        reps = max(3, min(a.steps, 10))
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(reps):
            sr.all_gather()
        g1.record()
        torch.cuda.synchronize()
        t_all = torch.tensor([g0.elapsed_time(g1)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
        gms = float(t_all.item()) / reps
        recv = sr.width * (world - 1)
        gather = {"ms": round(gms, 3), "bytes_received_per_gpu": int(recv),
                  "gbs_per_gpu": round(recv / (gms / 1e3) / 1e9, 1),
                  "what": "NCCL all_gather_into_tensor, in place in the output buffer (no staging copy), after the decode; "
                          "reported apart from decode GB/s"}
        del sr

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    # dominant kernel: the one with the largest device time
    # algorithmic bytes of each kernel: what it must read plus what it must write
    fj, tj = p.fused_jobs[:p.n_fused], p.fused_jobs[p.n_fused:]      # own tables; shared tables (BF16)
    # element size of each fused job: BF16 chunks first, 4-byte-element chunks last
    fes = np.full(fj.size, 2, dtype=np.int64)
    fes[fj.size - p.n_fused_f32:] = 4
    f_stored = int(((fes - 1) * fj["n"]).sum() + tj["n"].sum())      # stored planes read by the fused kernel
    f_plain = int((fes * fj["n"]).sum() + 2 * tj["n"].sum())
    f_coded = int(fj["src_len"].sum() + tj["src_len"].sum())
    fused_bytes = f_coded + f_stored + f_plain                        # stream + planes in, plaintext out
    stream_bytes = int(p.stream_jobs["src_len"].sum() + p.stream_jobs["n"].sum())
    fin_plain = plain - f_plain
    finish_bytes = int(coded - f_coded - f_stored - p.stream_jobs["src_len"].sum()
                       + p.stream_jobs["n"].sum() + fin_plain + p.base_bytes)
    kbytes = {"stream_decode": stream_bytes, "finish": finish_bytes, "fused": fused_bytes}
    kname = {"stream_decode": "k_rans / k_stream<bytes>",
             "finish": "k_stream<delta> + k_finish" if p.delta_jobs.size else "k_finish",
             "fused": "k_stream<f32>" if p.n_fused_f32 * 2 > fj.size + tj.size else
                      "k_stream<bf16, shared tables>" if tj.size > fj.size else "k_stream<bf16>"}
    dom = max(kbytes, key=lambda k: phase_ms[k])
    dom_bytes = kbytes[dom]
    achieved = dom_bytes / (phase_ms[dom] / 1e3) / 1e9
    whole = (coded + plain + p.base_bytes) / (ms / a.steps / 1e3) / 1e9
    traffic = None
    if dom == "fused" and not p.n_fused_f32 and not p.n_fused_t:
        # DRAM bytes of one launch, scaled from the committed ncu capture of a smaller
        # archive of the same chunks (traffic is proportional to the chunks processed)
        try:
            with open(os.path.join(ROOT, "profiles", "k_stream_bf16_dram_traffic.json")) as f:
                tj = json.load(f)
            traffic = int((tj["dram_bytes_read"] + tj["dram_bytes_write"])
                          * (2 * int(fj["n"].sum())) / tj["plaintext_bytes"])
        except Exception:
            traffic = None
    if world == 1:
        cpu_base = cpu_baseline_subprocess(a)
        batch = batch_decode_compare(dec, p)
        saved = None
        if a.layout == "mapped" and not a.shared_tables:
            try:
                saved = save_side(dec, a)
            except (OSError, RuntimeError, ValueError) as exc:     # a side measurement: the line is printed without it
                saved = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        other = default_layout_side(a, barrier) if a.layout == "mapped" and a.model == "llama-3.1-8b" else None
    else:
        cpu_base = batch = other = saved = None        # timed at N=1 only
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": round(ms / a.steps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": workload_name(a), "plaintext_bytes": plain, "coded_bytes": coded,
                   "chunks": int(p.chunks.size),
                   "rans_streams": int(p.fused_jobs.size + 2 * p.delta_jobs.size + p.stream_jobs.size + p.seg_jobs.size),
                   "crc32": not a.no_crc, "archive": archive_pin(a, rank),
                   "parity": "device crc32 of every chunk equals its record; 24 spread chunks byte-compared with the CPU oracle",
                   "per_gpu": "its own tensor-parallel slice" if per_rank_archives(a) else "full replica",
                   "l2": f"no flush: each step streams {coded / 1e9:.1f} GB in and {plain / 1e9:.1f} GB out, far beyond the 126 MB L2"},
        "clocks": clk.summary(),
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s",
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(host_res.numel() * 4),
                "api": f"lmz_b200.decode.PipelinedDecoder.run_from_host, {nslices} slices, archive planned and pinned beforehand",
                "cold": cold},
        "gpu_launches": int(dec.launches_per_run * a.steps),
        "roofline": {"bound": "hbm", "kernel": kname[dom],
                     "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": peak_kind,
                     "algorithmic_bytes_per_launch": dom_bytes,
                     "whole_decode": {"achieved": round(whole, 1), "frac": round(whole / peak, 4),
                                      "bytes": coded + plain + p.base_bytes}},
        "phase_ms": {k: round(v, 3) for k, v in phase_ms.items()},
        "cpu_baseline": cpu_base,
        "save": saved,
        "batch_decode": batch,
        "default_layout": other,
        "partitioned": part,
        "allgather": gather,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()


_STRESS = {}


def _stress_make(args):
    """(plaintext, per-stream-table stream, histogram) of one pool stream, in a worker process."""
    from oracle import native, synth
    dist, n, i = args
    plain = synth.stress_plane(dist, n, 7919 * i + n)
    return plain, native.best().rans_encode(plain), np.bincount(plain, minlength=256)


def _stress_shared(args):
    from oracle import native
    plain, freqs = args
    return native.best().rans_encode_shared(plain, freqs)


def run_stress(a, rank: int):
    """The decoder stress matrix: 8 symbol distributions x stream lengths x batch sizes, each
    batch decoded through `lmz_gpu_decode_batch_dev` once with per-stream frequency tables
    and once with one shared table, device resident, CUDA events, best of 5 after 3 warm-up
    launches, every cell's output compared with the plaintext on the device.  Streams come
    from a pool of `--stress-pool` distinct ones per (distribution, length), written by the
    reference-exact CPU encoder and cycled when a batch is larger than the pool.  Where the
    reference's own CUDA decoder (oracle/_ref/liblmzgpu.so) accepts the shape (plane a multiple
    of 128) it is timed on the same device buffers."""
    if rank != 0:
        return
    import ctypes
    import multiprocessing as mp

    import torch

    from lmz_b200 import gpu
    from oracle import native, synth
    ok, why = gpu.available()
    if not ok:
        raise SystemExit(f"the CUDA library is unavailable: {why}")
    lib = gpu.library()
    sig = [ctypes.c_void_p] * 3 + [ctypes.c_uint, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
    ref_path = os.path.join(ROOT, "oracle", "_ref", "liblmzgpu.so")
    ref = ctypes.CDLL(ref_path) if os.path.exists(ref_path) else None
    if ref is not None:
        ref.lmz_gpu_decode_batch_dev.restype = ctypes.c_int
        ref.lmz_gpu_decode_batch_dev.argtypes = sig
    lengths = [int(x) for x in a.stress_lengths.split(",")]
    batches = [int(x) for x in a.stress_batches.split(",")]
    cs = torch.cuda.current_stream().cuda_stream
    pad = gpu.pad_bytes()
    cells, tot_bytes, tot_ms, peak = [], 0, 0.0, measured_peak()[0]
    best_cell = None
    clk_ctx = ClockSampler(0)
    t_start = time.time()
    with clk_ctx as clk, mp.get_context("fork").Pool(os.cpu_count() or 1) as pool:
        for dist in synth.STRESS_DISTRIBUTIONS:
            for n in lengths:
                P = max(1, min(a.stress_pool, max(batches)))
                made = pool.map(_stress_make, [(dist, n, i) for i in range(P)], chunksize=max(1, P // 64))
                plains = [m[0] for m in made]
                freqs = native.best().rans_freqs(np.sum([m[2] for m in made], axis=0))
                shared = pool.map(_stress_shared, [(pl, freqs) for pl in plains], chunksize=max(1, P // 64))
                d_plain = torch.from_numpy(np.stack(plains)).cuda()
                hdr = torch.frombuffer(bytearray(b"R1\0\0" + freqs.astype("<u2").tobytes()), dtype=torch.uint8).cuda()
                for kind, streams in (("per-stream", [m[1] for m in made]), ("shared", shared)):
                    lens = np.array([len(x) for x in streams], dtype=np.int64)
                    starts = np.cumsum(lens) - lens
                    d_blob = torch.zeros(int(lens.sum()) + pad, dtype=torch.uint8, device="cuda")
                    d_blob[:int(lens.sum())] = torch.frombuffer(bytearray(b"".join(streams)), dtype=torch.uint8).cuda()
                    for B in batches:
                        idx = np.arange(B) % P
                        offs = np.empty(2 * B, dtype=np.int64)
                        offs[0::2], offs[1::2] = starts[idx], lens[idx]
                        d_off = torch.from_numpy(offs).cuda()
                        out = torch.empty(B * n, dtype=torch.uint8, device="cuda")
                        h = hdr.data_ptr() if kind == "shared" else None

                        def timed(fn):
                            best = None
                            for it in range(8):
                                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                                e0.record()
                                rc = fn(h, d_blob.data_ptr(), d_off.data_ptr(), B, n, out.data_ptr(), cs, 0)
                                e1.record()
                                torch.cuda.synchronize()
                                if rc != 0:
                                    return None
                                if it >= 3:
                                    best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
                            return best

                        def same():
                            got = out.view(B, n)
                            return all(torch.equal(got[r0:r0 + P], d_plain[:min(P, B - r0)]) for r0 in range(0, B, P))

                        out.zero_()
                        ms = timed(lib.lmz_gpu_decode_batch_dev)
                        if ms is None:
                            raise SystemExit(f"stress cell {dist}/{n}/{B}/{kind} failed: {gpu.last_error()}")
                        if not same():
                            raise SystemExit(f"stress cell {dist}/{n}/{B}/{kind} decoded to the wrong bytes")
                        cell = {"dist": dist, "len": n, "batch": B, "tables": kind, "ms": round(ms, 4),
                                "gbps": round(B * n / ms / 1e6, 2), "ref_gbps": None}
                        if ref is not None and n % 128 == 0:
                            out.zero_()
                            rms = timed(ref.lmz_gpu_decode_batch_dev)
                            if rms is not None:
                                if not same():
                                    raise SystemExit(f"the reference's decoder differs on {dist}/{n}/{B}/{kind}")
                                cell["ref_gbps"] = round(B * n / rms / 1e6, 2)
                        moved = int(lens[idx].sum()) + B * n
                        cell["hbm_frac"] = round(moved / ms / 1e6 / peak, 4)
                        cells.append(cell)
                        tot_bytes += B * n
                        tot_ms += ms
                        if best_cell is None or cell["gbps"] > best_cell["gbps"]:
                            best_cell = dict(cell, moved=moved)
                        del out, d_off
                    del d_blob
                del d_plain
                print(f"[stress] {dist} {n}: {time.time() - t_start:.0f}s", file=sys.stderr)
    # CPU baseline: the reference-exact CPU decoder on one cell's pool, every core
    cpu = cpu_stress_baseline(a)
    value = tot_bytes / tot_ms / 1e6
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": 1, "steps": 5, "warmup": 3,
        "ms_per_step": round(tot_ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic",
        "config": {"workload": "decoder stress batch: 8 distributions x lengths x batch sizes x {per-stream, shared} tables, "
                               "lmz_gpu_decode_batch_dev", "lengths": lengths, "batches": batches,
                   "pool": f"{a.stress_pool} distinct streams per (distribution, length), cycled in larger batches",
                   "value_is": "total symbols of all cells / total best-of-5 time of all cells",
                   "l2": "the largest cells stream up to 17 GB per launch; small cells fit the 126 MB L2 and are launch-bound"},
        "clocks": clk.summary(),
        "e2e": None, "gpu_launches": len(cells) * 8,
        "roofline": {"bound": "hbm", "kernel": "k_stream<bytes> / k_rans", "achieved": round(best_cell["moved"] / best_cell["ms"] / 1e6, 1),
                     "peak": peak, "unit": "GB/s", "frac": best_cell["hbm_frac"], "traffic": None,
                     "cell": {k: best_cell[k] for k in ("dist", "len", "batch", "tables")}},
        "cpu_baseline": cpu,
        "cells": cells,
    }
    emit(line)


def cpu_stress_baseline(a):
    """`lmz_rans_decode` of the reference's C core (the checker's port where it is absent) over
    64 exponent-like streams of 1 Mi symbols, one worker process per core."""
    import multiprocessing as mp
    from oracle import native
    made = [_stress_make(("exponent", 1 << 20, i)) for i in range(8)]
    _STRESS["streams"] = [m[1] for m in made]
    threads = os.cpu_count() or 1
    with mp.get_context("fork").Pool(threads) as pool:
        pool.map(_stress_decode, range(threads))
        t = time.perf_counter()
        done = sum(pool.map(_stress_decode, range(threads * 8)))
        dt = time.perf_counter() - t
    return {"value": round(done / dt / 1e9, 3), "unit": "GB/s", "cores": threads,
            "kind": "reference" if native.ref() is not None else "port",
            "sample": f"{threads * 8} decodes of 1 Mi-symbol exponent-like streams, {threads} worker processes"}


def _stress_decode(i):
    from oracle import native
    s = _STRESS["streams"][i % len(_STRESS["streams"])]
    return int(native.best().rans_decode(s, 1 << 20).size)


def save_side(dec, a):
    """The way back: the first BF16 member of the decoded model, as it sits in HBM, written as an
    lmz archive by `lmz_b200.save.save_archive` (plane split, rANS coding, framing and crc32 on the
    device; the container and the record list on the host), then decoded again and compared.
    `device_gbs` counts the device work alone, `value` the whole call including the host's
    Python loop over the chunk records and the write to a RAM-backed file."""
    import tempfile

    import torch

    from lmz_b200 import decode, save
    ar = dec.archive
    pick = next((m for m in ar.members if m.get("kind") == "safetensors" and
                 all(t["dtype"] == "BF16" for t in m.get("tensors", {}).values())), None)
    if pick is None:
        return None
    lo, size = int(pick["dst"]), int(pick["size"])
    member = dec.output[lo:lo + size]
    tmpdir = "/dev/shm" if os.path.isdir("/dev/shm") else None
    with tempfile.NamedTemporaryFile(suffix=".lmz", dir=tmpdir) as f:
        best = None
        for _ in range(2):
            st = {}
            t0 = time.perf_counter()
            nbytes = save.save_archive(f.name, [(pick["path"], member)], chunk_size=64 << 10, mapped=True, stats=st)
            dt = time.perf_counter() - t0
            if best is None or dt < best[0]:
                best = (dt, st, nbytes)
        back = decode.ArchiveDecoder(f.name)
        back.run()
        back.check()
        if not torch.equal(back.output, member):
            raise SystemExit("the archive written on the device does not decode to the member it was written from")
        del back
    return {"value": round(size / best[0] / 1e9, 2), "unit": "GB/s", "seconds": round(best[0], 3),
            "device_gbs": round(size / best[1]["device_s"] / 1e9, 1), "plaintext_bytes": size,
            "archive_bytes": int(best[2]),
            "api": "lmz_b200.save.save_archive: one BF16 safetensors member resident in HBM -> .lmz file, 64 KiB chunks"}


def batch_decode_compare(dec, p):
    """`lmz_gpu_decode_batch_dev` on the archive's own exponent streams (device resident,
    per-stream tables, 32768 symbols each): this library, and the reference's CUDA decoder
    on the same inputs when oracle/_ref/liblmzgpu.so exists (its lmz/gpu/lmzgpu.cu compiled
    for sm_100 by oracle/Makefile).  Symbols per second, best of 5, CUDA events.  `encode` is
    `lmz_gpu_encode_batch_dev` on the decoded planes, checked against the archive's streams."""
    import ctypes
    import torch
    from lmz_b200 import gpu
    fj = p.fused_jobs[:p.n_fused]
    sel = np.nonzero(fj["n"] == 32768)[0][:65536]
    if sel.size < 1024:
        return None
    offs = np.empty(2 * sel.size, dtype=np.uint64)
    offs[0::2], offs[1::2] = fj["src_off"][sel], fj["src_len"][sel]
    d_off = torch.from_numpy(offs.view(np.int64)).cuda()
    nstr, plane = int(sel.size), 32768
    cs = torch.cuda.current_stream().cuda_stream

    def run(lib):
        fn = lib.lmz_gpu_decode_batch_dev
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint, ctypes.c_uint, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_uint]
        out = torch.zeros(nstr * plane, dtype=torch.uint8, device="cuda")
        best = None
        for i in range(8):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(None, dec.d_payload.data_ptr(), d_off.data_ptr(), nstr, plane, out.data_ptr(), cs, 0)
            e1.record()
            torch.cuda.synchronize()
            if rc != 0:
                return None, None
            if i >= 3:
                best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
        return nstr * plane / (best / 1e3) / 1e9, out

    ours, out = run(gpu.library())
    res = {"streams": nstr, "plane": plane, "unit": "GB/s of symbols", "value": round(ours, 1),
           "reference_gpu": None, "encode": None}
    # and back: the GPU encoder must reproduce the archive's streams (written by the
    # reference-exact CPU encoder) from the decoded planes, length for length, byte for byte
    lib = gpu.library()
    slot = lib.lmz_gpu_encode_slot_bytes(plane)
    slots = torch.empty(nstr * slot, dtype=torch.uint8, device="cuda")
    lens = torch.zeros(nstr, dtype=torch.int32, device="cuda")
    best = None
    for i in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.lmz_gpu_encode_batch_dev(out.data_ptr(), nstr, plane, slots.data_ptr(), lens.data_ptr(), cs)
        e1.record()
        torch.cuda.synchronize()
        if rc != 0:
            raise SystemExit("batch encode failed: " + gpu.last_error())
        if i >= 2:
            best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
    if not np.array_equal(lens.cpu().numpy().astype(np.int64), fj["src_len"][sel].astype(np.int64)):
        raise SystemExit("re-encoded stream lengths differ from the archive's")
    for i in np.linspace(0, nstr - 1, 64).astype(np.int64):
        n, o = int(fj["src_len"][sel[i]]), int(fj["src_off"][sel[i]])
        if not torch.equal(slots[(i + 1) * slot - n:(i + 1) * slot], dec.d_payload[o:o + n]):
            raise SystemExit(f"re-encoded stream {i} differs from the archive's bytes")
    res["encode"] = round(nstr * plane / (best / 1e3) / 1e9, 1)
    del slots
    ref_path = os.path.join(ROOT, "oracle", "_ref", "liblmzgpu.so")
    if os.path.exists(ref_path):
        ref, ref_out = run(ctypes.CDLL(ref_path))
        if ref is not None:
            if not torch.equal(out, ref_out):
                raise SystemExit("batch decode differs from the reference's CUDA decoder")
            res["reference_gpu"] = round(ref, 1)
    return res


def default_layout_side(a, barrier):
    """The reference's default 8 MiB chunking (exponent-conditioned BF16), which a GPU
    decodes at the latency of one 4 Mi-symbol stream per chunk: the same model, measured
    beside the headline."""
    import argparse as _ap
    import torch
    from lmz_b200 import decode
    b = _ap.Namespace(**vars(a))
    b.layout, b.chunk_size = "default", 0
    blob = get_archive(b, 0, barrier)
    dec = decode.ArchiveDecoder(blob, checksum=not a.no_crc)
    for _ in range(2):
        dec.run()
    dec.check()
    verify_sample(dec, blob, nsample=6)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        dec.run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    phase = {}
    for name, mask in (("stream_decode", 1), ("cond", 2), ("finish", 4)):
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(); dec.run(phases=mask); s1.record()
        torch.cuda.synchronize()
        phase[name] = round(s0.elapsed_time(s1), 3)
    p = dec.plan
    peak, _ = measured_peak()
    moved = p.coded_bytes + p.total
    return {"workload": workload_name(b), "plaintext_bytes": int(p.total), "chunks": int(p.chunks.size),
            "rans_streams": int(p.fused_jobs.size + 2 * p.delta_jobs.size + p.stream_jobs.size + p.seg_jobs.size),
            "value": round(p.total / (ms / 1e3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(ms, 3),
            "roofline_frac": round(moved / (ms / 1e3) / 1e9 / peak, 4), "archive": archive_pin(b),
            "phase_ms": phase}


def cpu_baseline_subprocess(a):
    """The CPU baseline, timed in a fresh interpreter: its worker processes are forked,
    which a process holding a CUDA context and page-locked mappings should not do."""
    import subprocess
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "1",
           "--warmup", "0", "--model", a.model, "--layout", a.layout, "--seed", str(a.seed),
           "--cpu-sample-mb", str(a.cpu_sample_mb)]
    if a.chunk_size:
        cmd += ["--chunk-size", str(a.chunk_size)]
    if a.shared_tables:
        cmd += ["--shared-tables", str(a.shared_tables)]
    if a.no_cache:
        cmd += ["--no-cache"]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=1200)
    if r.returncode != 0:
        raise SystemExit("cpu baseline failed: " + r.stderr[-400:])
    return json.loads(r.stdout.strip().splitlines()[-1])["cpu_baseline"]


_REGISTERED = set()


def pin_host(arr):
    """A pinned host tensor over `arr`: the mapped archive is page-locked in place
    (no second copy per rank); if that is refused, a pinned copy is made.  A range must
    not be registered twice (the runtime keeps the refusal as its last error): release
    the earlier registration with `unpin_host` first."""
    import torch
    t = torch.from_numpy(arr)
    rc = int(torch.cuda.cudart().cudaHostRegister(t.data_ptr(), t.numel(), 0))
    if rc == 0:
        _REGISTERED.add(t.data_ptr())
        return t
    c = torch.empty(t.numel(), dtype=torch.uint8).pin_memory()
    c.copy_(t)
    return c


def unpin_host(t):
    """Undo `pin_host`'s registration of `t` (nothing to do for a pinned copy)."""
    import torch
    if t.data_ptr() in _REGISTERED:
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaHostUnregister(t.data_ptr())
        _REGISTERED.discard(t.data_ptr())


def verify_sample(dec, blob, nsample: int = 24):
    """Byte-compare a spread of chunks against the CPU oracle, and every chunk's
    device-computed crc32 against the archive's records."""
    from oracle import archive as oa, codec
    ar = oa.Archive(blob)
    recs = ar.records
    if dec.checksum:
        crcs = dec.chunk_crcs()
        have = recs["crc"] != 0
        if not (crcs[have] == recs["crc"][have]).all():
            raise SystemExit("device crc32 differs from the archive's records")
    idx = np.unique(np.linspace(0, recs.size - 1, nsample).astype(np.int64))
    out = dec.output
    for i in idx:
        c = recs[i]
        if c["codec"] in (codec.CODEC_REF, codec.CODEC_DELTA):
            continue
        want = oa._decode_plain(ar, c, True, None)
        got = out[int(c["dst"]):int(c["dst"]) + int(c["rlen"])].cpu().numpy()
        if not (got == want).all():
            raise SystemExit(f"chunk {i} differs from the CPU oracle")


def run_reference(a, rank: int):
    """The reference's CPU decode of a bounded sample, all host threads, rank 0 only."""
    if rank != 0:
        return
    blob = get_archive(a, 0, lambda: None)
    threads = os.cpu_count() or 1
    from oracle import archive as oa
    ar = oa.Archive(blob)
    from lmz_b200 import archive as fmt, plan as planner      # host-side planning only: no GPU is touched
    p = planner.build_plan(fmt.Archive(blob), fuse=not a.no_fuse)
    vals = []
    for i in range(a.warmup + a.steps):
        v, what, kind = cpu_decode_sample(blob, a.cpu_sample_mb, threads, "reference")
        if i >= a.warmup:
            vals.append(v)
    v = float(np.mean(vals))
    sample_bytes = min(ar.total, a.cpu_sample_mb << 20)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(v, 3), "unit": "GB/s",
        "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(sample_bytes / v / 1e6, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": workload_name(a), "plaintext_bytes": int(p.total), "coded_bytes": int(p.coded_bytes),
                   "chunks": int(p.chunks.size),
                   "rans_streams": int(p.fused_jobs.size + 2 * p.delta_jobs.size + p.stream_jobs.size + p.seg_jobs.size),
                   "crc32": not a.no_crc, "archive": archive_pin(a, 0),
                   "parity": "device crc32 of every chunk equals its record; 24 spread chunks byte-compared with the CPU oracle",
                   "per_gpu": "its own tensor-parallel slice" if per_rank_archives(a) else "full replica",
                   "l2": f"no flush: each step streams {p.coded_bytes / 1e9:.1f} GB in and {p.total / 1e9:.1f} GB out, far beyond the 126 MB L2"},
        "cpu_baseline": {"value": round(v, 3), "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": what},
        "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    emit(line)


if __name__ == "__main__":
    main()
