"""Builds lmz rANS streams with numpy, many streams at a time.

`gpu.verify()` and the load-time self-test need streams whose plaintext is
known; the reference makes them with its CPU encoder
(lmz/gpu/__init__.py:164-207, 303-315).  This is an independent encoder that
writes the same format (lmz/native/lmzcore.c:882-979, 1318-1383), vectorised
across the streams of a batch.  It encodes only -- nothing here decodes.
"""
from __future__ import annotations

import numpy as np

PROB_SCALE = 4096
HEADER = 516


def normalize(counts) -> np.ndarray:
    """Histogram -> 256 frequencies summing to 4096 (lmz/native/lmzcore.c:882-937)."""
    c = np.asarray(counts, dtype=np.uint64)
    total = int(c.sum())
    if total == 0:
        raise ValueError("empty histogram")
    f = (c * np.uint64(PROB_SCALE) // np.uint64(total)).astype(np.int64)
    f[(c > 0) & (f == 0)] = 1
    s = int(f.sum())
    if s < PROB_SCALE:
        f[int(np.argmax(c))] += PROB_SCALE - s
    else:
        excess = s - PROB_SCALE
        while excess > 0:
            bi = int(np.argmax(f))
            if f[bi] <= 1:
                raise ValueError("cannot normalise")
            take = min(int(f[bi]) - 1, excess)
            f[bi] -= take
            excess -= take
    return f.astype(np.uint16)


def header_bytes(freqs) -> bytes:
    return b"R1\0\0" + np.asarray(freqs, dtype="<u2").tobytes()


def encode_batch(plains: np.ndarray, freqs: np.ndarray | None = None, shared: bool = False):
    """Encode every row of `plains` ([B, n] uint8).  Returns a list of B streams.

    `freqs` is one table ([256]) for the whole batch or None for a table per
    row.  With `shared` the 516-byte header is left off each stream (the
    layout of scratchpad/gpu/shared_enc.c:1-13)."""
    plains = np.ascontiguousarray(plains, dtype=np.uint8)
    B, n = plains.shape
    if freqs is None:
        F = np.stack([normalize(np.bincount(row, minlength=256)) for row in plains])
    else:
        F = np.broadcast_to(np.asarray(freqs, dtype=np.uint16), (B, 256))
    F = F.astype(np.uint64)
    S = np.cumsum(F, axis=1) - F
    rows = np.arange(B)
    state = np.full((B, 8), 1 << 16, dtype=np.uint64)
    words = np.zeros((B, max(n, 1)), dtype=np.uint16)
    cnt = np.zeros(B, dtype=np.int64)
    for i in range(n - 1, -1, -1):
        lane = i & 7
        sym = plains[:, i]
        f = F[rows, sym]
        if (f == 0).any():
            raise ValueError("a symbol has no frequency in the table")
        x = state[:, lane]
        need = x >= (f << np.uint64(20))
        idx = np.nonzero(need)[0]
        if idx.size:
            words[idx, cnt[idx]] = (x[idx] & np.uint64(0xFFFF)).astype(np.uint16)
            cnt[idx] += 1
            x = np.where(need, x >> np.uint64(16), x)
        state[:, lane] = x + S[rows, sym] + (x // f) * (np.uint64(PROB_SCALE) - f)
    out = []
    for b in range(B):
        body = state[b].astype("<u4").tobytes() + words[b, :cnt[b]][::-1].astype("<u2").tobytes()
        out.append(body if shared else header_bytes(F[b].astype(np.uint16)) + body)
    return out


def pack(streams):
    """Concatenate streams back to back; returns (bytes, offsets) where offsets
    is the 2*nstr little-endian u64 (offset, length) table `decode_batch` takes."""
    offs = np.zeros((len(streams), 2), dtype="<u8")
    pos = 0
    for i, s in enumerate(streams):
        offs[i] = (pos, len(s))
        pos += len(s)
    return b"".join(streams), offs.tobytes()
