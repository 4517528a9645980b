"""Pin the benchmark's synthetic archives to the REFERENCE's own writer.

    python tests/golden/make_bench_pins.py <reference tree> [model:layout ...]

For each benchmark workload this writes the model's files to a scratch directory,
compresses them with the reference's unmodified `lmz.api.compress` (through
ref_compress.py) and with the checker's parallel writer (`oracle/bigwrite.py`, the one
`bench.py` uses), requires the payload bytes and the chunk records of the two archives to
be identical, and records their sha256 in bench_pins.json.  `bench.py` compares the archive
it generates on the GPU box with these pins, so every benchmark number is measured on bytes
the reference's encoder would have written.  Needs the reference tree and oracle/_ref.
"""
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
from oracle import archive as oa  # noqa: E402

PINS = os.path.join(HERE, "bench_pins.json")
DEFAULT = ["llama-tiny:mapped", "llama-tiny:default", "llama-2layer:mapped", "llama-2layer:default",
           "config1-tensor:default", "config1-tensor:mapped"]


def digests(blob: np.ndarray) -> dict:
    ar = oa.Archive(blob)
    toff = int(np.frombuffer(blob[-40:-32].tobytes(), dtype="<u8")[0])
    return {"payload_sha256": hashlib.sha256(memoryview(blob[32:toff])).hexdigest(),
            "records_sha256": hashlib.sha256(ar.records.tobytes()).hexdigest(),
            "payload_bytes": toff - 32, "records": int(ar.records.size), "plain_bytes": int(ar.total)}


def main(ref: str, wanted) -> int:
    pins = json.load(open(PINS)) if os.path.exists(PINS) else {}
    for item in wanted:
        model, layout = item.split(":")
        files, ours, key = bench.model_files_and_archive(model, layout, seed=1)
        tmp = tempfile.mkdtemp(prefix="lmzpin-")
        try:
            src = os.path.join(tmp, "src")
            for rel, data in files:
                path = os.path.join(src, rel)
                os.makedirs(os.path.dirname(path), exist_ok=True)
                np.asarray(data).tofile(path)
            target = src if len(files) > 1 else os.path.join(src, files[0][0])
            dst = os.path.join(tmp, "ref.lmz")
            t = time.time()
            opts = {"mapped": True} if layout == "mapped" else {}
            subprocess.run([sys.executable, os.path.join(HERE, "ref_compress.py"), ref, target, dst,
                            json.dumps(opts)], check=True)
            theirs = np.fromfile(dst, dtype=np.uint8)
            a, b = digests(ours), digests(theirs)
            if a != b:
                raise SystemExit(f"{item}: the checker's writer and the reference disagree\n{a}\n{b}")
            pins[key] = dict(a, reference_seconds=round(time.time() - t, 1))
            print(item, key, a["records"], "records identical", flush=True)
        finally:
            shutil.rmtree(tmp)
        with open(PINS, "w") as f:
            json.dump(pins, f, indent=1, sort_keys=True)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2:] or DEFAULT))
