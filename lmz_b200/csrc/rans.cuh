// The 8-lane interleaved rANS decoder core.
//
// One stream is decoded by one group of 8 lanes (lane k owns state k, reference
// lmz/native/lmzcore.c:1409-1530); a warp carries four streams.  A lane's need
// for a refill depends only on its own state, so one warp vote plus a popcount
// of the lanes below gives every lane its byte offset from the shared cursor.
//
// Compressed bytes are streamed through a per-group shared-memory ring filled
// by CTA-local bulk async copies (256 B per copy, completion on an mbarrier).
// The ring starts at the 16-byte boundary below the stream, so the stream's own
// header (frequency table and initial states) arrives through the same ring.
#pragma once
#include "common.cuh"

namespace lmz {

// Decode tables in shared memory.
//   narrow (per-stream tables): slot -> symbol (4096 x u8) and
//                               symbol -> (freq-1) << 12 | start (256 x u32)
//   wide   (one table per CTA): slot -> (freq-1) << 20 | start << 8 | symbol
// Frequency is stored minus one because a single-symbol stream has f = 4096.
struct NarrowTab {
    uint8_t *sym;
    uint32_t *sf;
};

// Per-group streaming state.  Cursor and counters are bytes/slots measured
// from `abase`, the 16-byte boundary at or below the stream's first byte.
struct Ring {
    uint8_t *buf;          // RING bytes, 128-byte aligned
    uint64_t *bars;        // NSLOT mbarriers
    const uint8_t *abase;
    uint32_t valid_slots;  // slots that overlap the stream
    uint32_t issued;       // slots requested so far (meaningful on lane k == 0)
    uint32_t ready;        // slots this lane has seen complete
    bool dead;             // a wait ran out; stop waiting, the job is reported failed

    __device__ __forceinline__ void issue(uint32_t cursor, bool leader)
    {
        if (!leader) return;
        uint32_t lim = cursor / SLOT + NSLOT;
        if (lim > valid_slots) lim = valid_slots;
        while (issued < lim) {
            uint32_t j = issued % NSLOT;
            mbar_expect_tx(&bars[j], SLOT);
            bulk_g2s(buf + j * SLOT, abase + (size_t)issued * SLOT, SLOT, &bars[j]);
            issued++;
        }
    }

    // Make bytes [.., upto) resident (clamped to the stream's own slots).
    __device__ __forceinline__ void require(uint32_t upto)
    {
        uint32_t need = (upto + SLOT - 1) / SLOT;
        if (need > valid_slots) need = valid_slots;
        while (ready < need) {
            if (!dead && !mbar_wait(&bars[ready % NSLOT], (ready / NSLOT) & 1u)) dead = true;
            ready++;
        }
    }

    __device__ __forceinline__ uint32_t byte_at(uint32_t o) const { return buf[o & (RING - 1)]; }
    __device__ __forceinline__ uint32_t u16_at(uint32_t o) const
    {
        return byte_at(o) | (byte_at(o + 1) << 8);
    }
    __device__ __forceinline__ uint32_t u32_at(uint32_t o) const
    {
        return u16_at(o) | (u16_at(o + 2) << 16);
    }
};

// Warp-cooperative table build for ONE stream from its 256 frequencies.
// `freq_of(s)` returns symbol s's frequency.  Every lane of the warp calls
// this; returns false (on all lanes) if the frequencies do not sum to 4096.
// Lane j owns symbols 8j..8j+7.  Rare symbols are written by their owner,
// common ones (f >= 64) by the whole warp so the fill stays balanced.
template <bool WIDE, class FreqOf>
__device__ __forceinline__ bool build_table(FreqOf freq_of, uint8_t *sym_tab, uint32_t *sf_tab,
                                            uint32_t *wide_tab, uint32_t lane)
{
    uint32_t f[8], tot = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        f[i] = freq_of(lane * 8 + i);
        tot += f[i];
    }
    uint32_t incl = tot;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= (uint32_t)d) incl += v;
    }
    uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    // A frequency above the scale would index past the tables; the sum test
    // below rejects the stream, but the fill must not run first.
    bool sane = __all_sync(0xffffffffu, tot <= PROB_SCALE) && total == PROB_SCALE;
    if (!sane) return false;
    uint32_t start = incl - tot;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint32_t s = lane * 8 + i, fi = f[i], st = start;
        start += fi;
        uint32_t packed_w = ((fi ? fi - 1 : 0) << 20) | (st << 8) | s;
        if (!WIDE) sf_tab[s] = ((fi ? fi - 1 : 0) << 12) | st;
        bool big = fi >= 64;
        if (!big) {
            for (uint32_t t = 0; t < fi; t++) {
                if (WIDE) wide_tab[st + t] = packed_w;
                else sym_tab[st + t] = (uint8_t)s;
            }
        }
        uint32_t m = __ballot_sync(0xffffffffu, big);
        while (m) {
            int src = __ffs(m) - 1;
            m &= m - 1;
            uint32_t bf = __shfl_sync(0xffffffffu, fi, src);
            uint32_t bs = __shfl_sync(0xffffffffu, st, src);
            uint32_t bsym = (uint32_t)src * 8 + i;
            uint32_t bw = ((bf - 1) << 20) | (bs << 8) | bsym;
            for (uint32_t t = lane; t < bf; t += 32) {
                if (WIDE) wide_tab[bs + t] = bw;
                else sym_tab[bs + t] = (uint8_t)bsym;
            }
        }
    }
    __syncwarp();
    return true;
}

// One decode step for this lane.  `active` is false for lanes past the end of
// a ragged stream: they keep their state, refill nothing and emit nothing.
template <bool WIDE>
__device__ __forceinline__ uint32_t rans_step(uint32_t &x, uint32_t &cursor, const Ring &ring,
                                              const NarrowTab &nt, const uint32_t *wide_tab,
                                              uint32_t lt_mask, uint32_t grp_mask, bool active)
{
    uint32_t slot = x & (PROB_SCALE - 1);
    uint32_t sym, x2;
    if (WIDE) {
        uint32_t e = wide_tab[slot];
        sym = e & 0xffu;
        x2 = ((e >> 20) + 1) * (x >> PROB_BITS) + slot - ((e >> 8) & 0xfffu);
    } else {
        sym = nt.sym[slot];
        uint32_t p = nt.sf[sym];
        x2 = ((p >> 12) + 1) * (x >> PROB_BITS) + slot - (p & 0xfffu);
    }
    bool need = active && x2 < RANS_LOW;
    uint32_t vote = __ballot_sync(0xffffffffu, need);
    uint32_t o = cursor + 2 * __popc(vote & lt_mask);
    uint32_t w = ring.u16_at(o);
    if (active) x = need ? ((x2 << 16) | w) : x2;
    cursor += 2 * __popc(vote & grp_mask);
    return sym;
}

}  // namespace lmz
