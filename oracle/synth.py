"""Seeded synthetic inputs with the shapes of the benchmark configurations.

Test infrastructure only.  No dataset or checkpoint is read: weights are drawn
from N(0, sigma) by seed, rounded to BF16 (or kept FP32), and laid out as
safetensors files, which is the container the reference's planner parses
(lmz/planner.py:196-237).
"""
from __future__ import annotations

import json

import numpy as np


def bf16_bytes(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bytes, round-to-nearest-even (what torch's .to(bfloat16) does)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16).view(np.uint8)


def normal_bf16(shape, seed: int, sigma: float = 0.02) -> np.ndarray:
    rng = np.random.default_rng(seed)
    n = int(np.prod(shape))
    return bf16_bytes(rng.standard_normal(n, dtype=np.float32) * np.float32(sigma))


def safetensors_bytes(tensors) -> np.ndarray:
    """Serialise [(name, dtype string, shape, uint8 data)] as one safetensors file."""
    meta, pos = {}, 0
    for name, dt, shape, data in tensors:
        meta[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [pos, pos + data.size]}
        pos += data.size
    head = json.dumps(meta, separators=(",", ":")).encode()
    head += b" " * (-(8 + len(head)) % 8)
    out = np.empty(8 + len(head) + pos, dtype=np.uint8)
    out[:8] = np.frombuffer(len(head).to_bytes(8, "little"), dtype=np.uint8)
    out[8:8 + len(head)] = np.frombuffer(head, dtype=np.uint8)
    p = 8 + len(head)
    for _n, _d, _s, data in tensors:
        out[p:p + data.size] = data
        p += data.size
    return out


def llama_layer_shapes(hidden=4096, ffn=14336, kv=1024):
    return [("self_attn.q_proj.weight", (hidden, hidden)), ("self_attn.k_proj.weight", (kv, hidden)),
            ("self_attn.v_proj.weight", (kv, hidden)), ("self_attn.o_proj.weight", (hidden, hidden)),
            ("mlp.gate_proj.weight", (ffn, hidden)), ("mlp.up_proj.weight", (ffn, hidden)),
            ("mlp.down_proj.weight", (hidden, ffn)),
            ("input_layernorm.weight", (hidden,)), ("post_attention_layernorm.weight", (hidden,))]


def llama_shard(layers, seed: int, hidden=4096, ffn=14336, kv=1024, vocab=0,
                embed=False, head=False, scale: float = 1.0) -> np.ndarray:
    """One safetensors shard of a Llama-architecture model: the given layer
    indices, optionally the embedding and the output head.  `scale` < 1 shrinks
    every matrix dimension for CPU-sized test cases."""
    h, f, k, v = (max(8, int(d * scale)) for d in (hidden, ffn, kv, max(vocab, 8)))
    tensors, s = [], seed * 1000003
    if embed:
        tensors.append(("model.embed_tokens.weight", "BF16", (v, h), normal_bf16((v, h), s)))
        s += 1
    for li in layers:
        for name, shape in llama_layer_shapes(h, f, k):
            s += 1
            if len(shape) == 1:
                data = bf16_bytes(np.ones(shape, dtype=np.float32))
            else:
                data = normal_bf16(shape, s)
            tensors.append((f"model.layers.{li}.{name}", "BF16", shape, data))
    if head:
        tensors.append(("model.norm.weight", "BF16", (h,), bf16_bytes(np.ones(h, np.float32))))
        tensors.append(("lm_head.weight", "BF16", (v, h), normal_bf16((v, h), s + 7)))
    return safetensors_bytes(tensors)


def perturbed_bf16(prev: np.ndarray, seed: int, frac: float = 0.3, sigma: float = 1e-4):
    """prev (bf16 bytes) plus N(0, sigma) noise on a random `frac` of elements."""
    rng = np.random.default_rng(seed)
    w = (prev.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    mask = rng.random(w.size) < frac
    w = w + mask * rng.standard_normal(w.size, dtype=np.float32) * np.float32(sigma)
    return bf16_bytes(w)


# ---------------------------------------------------------------- whole models
# A model is described as shards of (name, dtype string, shape) tensors.  Bytes
# are generated per 8 MiB block of a shard's data area from a seed, so any
# process can produce any block without the rest of the model in memory; 1-D
# "norm" tensors are then overwritten with 1.0.

BLOCK = 8 << 20


def _tp_shape(name: str, shape, tp: int):
    """One rank's slice of a weight under `tp`-way tensor parallelism: projections
    into the hidden size (o_proj, down_proj, the encoder's output dense layers) are
    cut along their input columns, every other matrix along its output rows (the
    vocabulary padded up to a multiple of tp), 1-D tensors are replicated."""
    if tp == 1 or len(shape) == 1:
        return tuple(shape)
    rows, cols = shape
    if any(k in name for k in ("o_proj", "down_proj", "output.dense")):
        return (rows, cols // tp)
    return (-(-rows // tp), cols)


def llama_spec(layers=32, hidden=4096, ffn=14336, kv=1024, vocab=128256, shards=4, tp=1):
    """Llama-architecture tensor list (BF16, untied embeddings) cut into `shards`
    safetensors files by layer range; with tp > 1, one rank's tensor-parallel slice."""
    per = -(-layers // shards)
    out = []
    for s in range(shards):
        t = []
        if s == 0:
            t.append(("model.embed_tokens.weight", "BF16", (vocab, hidden)))
        for li in range(s * per, min(layers, (s + 1) * per)):
            for name, shape in llama_layer_shapes(hidden, ffn, kv):
                t.append((f"model.layers.{li}.{name}", "BF16", shape))
        if s == shards - 1:
            t.append(("model.norm.weight", "BF16", (hidden,)))
            t.append(("lm_head.weight", "BF16", (vocab, hidden)))
        out.append([(n, d, _tp_shape(n, sh, tp)) for n, d, sh in t])
    return out


def xlmr_spec(layers=24, hidden=1024, ffn=4096, vocab=250002, tp=1):
    """XLM-R-large-shaped FP32 encoder as one safetensors file (biases and layer
    norms included); with tp > 1, one rank's tensor-parallel slice."""
    t = [("embeddings.word_embeddings.weight", "F32", (vocab, hidden)),
         ("embeddings.position_embeddings.weight", "F32", (514, hidden)),
         ("embeddings.LayerNorm.weight", "F32", (hidden,))]
    for li in range(layers):
        pre = f"encoder.layer.{li}."
        for nm, shape in (("attention.self.query", (hidden, hidden)), ("attention.self.key", (hidden, hidden)),
                          ("attention.self.value", (hidden, hidden)), ("attention.output.dense", (hidden, hidden)),
                          ("intermediate.dense", (ffn, hidden)), ("output.dense", (hidden, ffn))):
            t.append((pre + nm + ".weight", "F32", shape))
            t.append((pre + nm + ".bias", "F32", (shape[0],)))
        t.append((pre + "attention.output.LayerNorm.weight", "F32", (hidden,)))
        t.append((pre + "output.LayerNorm.weight", "F32", (hidden,)))
    return [[(n, d, _tp_shape(n, sh, tp)) for n, d, sh in t]]


def delta_chain_files(hidden=768, ffn=3072, vocab=50304, layers=12, checkpoints=3, seed=7000):
    """Safetensors files of a Pythia-shaped BF16 checkpoint chain: checkpoint 0 from
    N(0, 0.02); each later one is the previous plus N(0, 1e-4) noise on a random 30 %
    of elements, rounded to BF16."""
    h, f, v = hidden, ffn, vocab
    names = [("embed.weight", (v, h))]
    for li in range(layers):
        names += [(f"l{li}.attn.qkv.weight", (3 * h, h)), (f"l{li}.attn.o.weight", (h, h)),
                  (f"l{li}.mlp.up.weight", (f, h)), (f"l{li}.mlp.down.weight", (h, f)),
                  (f"l{li}.ln.weight", (h,))]
    names.append(("embed_out.weight", (v, h)))
    files, prev = [], None
    for ck in range(checkpoints):
        tensors = []
        for i, (name, shape) in enumerate(names):
            if len(shape) == 1:
                data = bf16_bytes(np.ones(shape, np.float32))
            elif ck == 0:
                data = normal_bf16(shape, seed + i)
            else:
                data = perturbed_bf16(prev[i], 100 * ck + i, frac=0.3, sigma=1e-4)
            tensors.append((name, "BF16", shape, data))
        prev = [t[3] for t in tensors]
        files.append(safetensors_bytes(tensors))
    return files


_ESZ = {"BF16": 2, "F32": 4}


class ShardLayout:
    """Byte layout of one synthetic safetensors shard."""

    def __init__(self, tensors, seed: int, sigma: float = 0.02):
        self.seed, self.sigma = seed, sigma
        meta, pos, self.norms = {}, 0, []
        for name, dt, shape in tensors:
            n = int(np.prod(shape)) * _ESZ[dt]
            meta[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [pos, pos + n]}
            if len(shape) == 1:
                self.norms.append((pos, pos + n, dt))
            pos += n
        self.dtype = tensors[0][1]
        head = json.dumps(meta, separators=(",", ":")).encode()
        head += b" " * (-(8 + len(head)) % 8)
        self.header = len(head).to_bytes(8, "little") + head
        self.data_start = len(self.header)
        self.data_size = pos
        self.size = self.data_start + pos
        self.tensors = {k: {"dtype": v["dtype"], "shape": v["shape"],
                            "offsets": [self.data_start + v["data_offsets"][0],
                                        self.data_start + v["data_offsets"][1]]}
                        for k, v in meta.items()}

    def _block(self, b: int, n: int) -> np.ndarray:
        cache = self.__dict__.setdefault("_cache", {})
        blk = cache.get(b)
        if blk is None:
            rng = np.random.default_rng((self.seed, b))
            if self.dtype == "BF16":
                blk = bf16_bytes(rng.standard_normal(n // 2, dtype=np.float32) * np.float32(self.sigma))
            else:
                blk = (rng.standard_normal(n // 4, dtype=np.float32)
                       * np.float32(self.sigma)).view(np.uint8)
            if len(cache) >= 2:
                cache.pop(next(iter(cache)))
            cache[b] = blk
        return blk

    def data(self, lo: int, hi: int) -> np.ndarray:
        """Bytes [lo, hi) of the data area."""
        out = np.empty(hi - lo, dtype=np.uint8)
        for b in range(lo // BLOCK, (hi - 1) // BLOCK + 1):
            b0 = b * BLOCK
            n = min(BLOCK, self.data_size - b0)
            blk = self._block(b, n)
            a, z = max(lo, b0), min(hi, b0 + n)
            out[a - lo:z - lo] = blk[a - b0:z - b0]
        one = {"BF16": np.frombuffer(b"\x80\x3f", dtype=np.uint8),
               "F32": np.frombuffer(b"\x00\x00\x80\x3f", dtype=np.uint8)}
        for s, e, dt in self.norms:
            a, z = max(lo, s), min(hi, e)
            if a < z:
                w = one[dt]
                full = np.tile(w, (e - s) // w.size)
                out[a - lo:z - lo] = full[a - s:z - s]
        return out

    def bytes(self, lo: int = 0, hi: int | None = None) -> np.ndarray:
        """Bytes [lo, hi) of the whole file (header included)."""
        hi = self.size if hi is None else hi
        out = np.empty(hi - lo, dtype=np.uint8)
        hdr = np.frombuffer(self.header, dtype=np.uint8)
        if lo < self.data_start:
            z = min(hi, self.data_start)
            out[:z - lo] = hdr[lo:z]
        if hi > self.data_start:
            a = max(lo, self.data_start)
            out[a - lo:] = self.data(a - self.data_start, hi - self.data_start)
        return out


STRESS_DISTRIBUTIONS = ("uniform", "single", "two", "geometric", "zipf", "exponent", "mantissa", "zero-runs")


def stress_plane(name: str, n: int, seed: int) -> np.ndarray:
    """One byte plane of the decoder stress configuration: uniform over 256 values, a single
    symbol, two symbols at p = 0.999, geometric p = 0.3, Zipf s = 1.1, the exponent bytes and
    the sign/mantissa bytes of N(0, 0.02) BF16 weights, and runs of zeros between random bytes."""
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
        w = normal_bf16((n,), seed).view("<u2")
        if name == "exponent":
            return ((w >> 7) & 0xFF).astype(np.uint8)                 # lmz/native/lmzcore.c:430-437
        return (((w >> 8) & 0x80) | (w & 0x7F)).astype(np.uint8)
    if name == "zero-runs":
        out = rng.integers(0, 256, n, dtype=np.uint8)
        pos = 0
        while pos < n:
            run = int(rng.geometric(0.02))
            out[pos:pos + run] = 0
            pos += run + int(rng.geometric(0.1))
        return out
    raise KeyError(name)
