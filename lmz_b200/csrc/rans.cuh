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

// Decode tables in shared memory, three layouts:
//   T_NARROW  per stream, 5 KiB: slot -> symbol (4096 x u8), then
//             symbol -> (freq-1) << 12 | start (256 x u32).  Two dependent loads.
//   T_WIDE    one per CTA, 16 KiB: slot -> (freq-1) << 20 | start << 8 | symbol.
//             One dependent load; affordable when the whole CTA shares a table, or
//             (T_WIDE1, one per stream, holding 4096 - freq) when a launch has so few
//             streams that only the length of the per-symbol chain matters: 13 fit an SM.
//   T_COMPACT per stream, 2 KiB: level 1 has one word per 16 slots holding four
//             times the index of the live symbol covering the bucket's first slot
//             (bits 0-9, i.e. its byte offset in level 2) and a bit per in-bucket
//             position t where another live symbol starts (bit 16+t); a popcount
//             of the bits at or below the slot's position gives the live-symbol
//             index exactly, and level 2 holds one entry per live symbol,
//             (4096 - freq) << 20 | start << 8 | symbol.  Two dependent loads and a
//             popcount, at 40 % of the narrow layout's footprint or less.  Level-1
//             words may be strided (L1S) so that several streams interleave.
// Narrow and wide store the frequency minus one because a single-symbol stream has
// f = 4096; compact stores 4096 - f for the same reason.
enum : int { T_NARROW = 0, T_WIDE = 1, T_COMPACT = 2, T_WIDE1 = 3, T_WIDE13 = 4 };   // T_WIDE1 / T_WIDE13: a wide table per stream, 12 / 13 streams per SM (a launch choice, the same table)

struct Tables {
    uint8_t *sym;        // T_NARROW
    uint32_t *sf;        // T_NARROW
    uint32_t *wide;      // T_WIDE
    uint32_t *l1;        // T_COMPACT: 256 words
    uint32_t *cf;        // T_COMPACT: up to 256 words
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
// Compact layout only: `rot` is added to every live-symbol index, in level 1 and
// in the position of the level-2 entry (streams that share a warp rotate their
// level 2 apart so that their popular entries fall in different banks);
// `nlive_out`, when not NULL, receives the number of live symbols, and a stream
// with more than `max_live` of them is refused before anything is written.
template <int MODE, int L1S = 1, class FreqOf>
__device__ __forceinline__ bool build_table(FreqOf freq_of, const Tables &tb, uint32_t lane,
                                            uint32_t rot = 0, uint32_t *nlive_out = nullptr,
                                            uint32_t max_live = 256)
{
    uint32_t f[8], tot = 0, nlive = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        f[i] = freq_of(lane * 8 + i);
        tot += f[i];
        nlive += f[i] != 0;
    }
    // one scan carries both prefix sums: frequencies (<= 4096 each lane once
    // sane) in the low half, live-symbol counts in the high half
    uint32_t both = (tot & 0xffffu) | (nlive << 16), incl = both;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= (uint32_t)d) incl += v;
    }
    // A frequency above the scale would index past the tables, and a lane total
    // above 16 bits would corrupt the packed scan: reject before any fill.
    bool lane_ok = tot <= PROB_SCALE;
    uint32_t total = __shfl_sync(0xffffffffu, incl, 31) & 0xffffu;
    uint32_t lanes_sum = __reduce_add_sync(0xffffffffu, lane_ok ? tot : PROB_SCALE + 1);
    if (!__all_sync(0xffffffffu, lane_ok) || lanes_sum != PROB_SCALE || total != PROB_SCALE)
        return false;
    const uint32_t all_live = __shfl_sync(0xffffffffu, incl, 31) >> 16;
    if (nlive_out) *nlive_out = all_live;
    if (all_live > max_live) return false;
    uint32_t start = (incl - both) & 0xffffu, live = ((incl - both) >> 16) + rot;
    if (MODE == T_COMPACT) {
#pragma unroll
        for (int i = 0; i < 8; i++) tb.l1[(lane * 8 + i) * L1S] = 0;
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint32_t s = lane * 8 + i, fi = f[i], st = start, li = live;
        start += fi;
        live += fi != 0;
        // wide: freq - 1; compact and per-stream wide: 4096 - freq, which turns the state update into
        // x - (x >> 12) * (4096 - f) - start with no separate slot term
        uint32_t packed = ((MODE == T_COMPACT || MODE == T_WIDE1 ? PROB_SCALE - fi : (fi ? fi - 1 : 0)) << 20) | (st << 8) | s;
        if (MODE == T_NARROW) tb.sf[s] = ((fi ? fi - 1 : 0) << 12) | st;
        if (MODE == T_COMPACT && fi) {
            tb.cf[li] = packed;
            if (st & 15u) atomicOr(&tb.l1[(st >> 4) * L1S], 1u << (16 + (st & 15u)));
        }
        // work items of this symbol: slots (narrow/wide) or covered bucket heads (compact)
        uint32_t lo = MODE == T_COMPACT ? (st + 15) >> 4 : st;
        uint32_t cnt = MODE == T_COMPACT ? (fi ? ((st + fi - 1) >> 4) + 1 - lo : 0) : fi;
        if (MODE == T_COMPACT && fi && ((st + fi - 1) >> 4) + 1 < lo) cnt = 0;
        bool big = cnt >= 64;
        if (!big) {
            for (uint32_t t = 0; t < cnt; t++) {
                if (MODE == T_WIDE || MODE == T_WIDE1) tb.wide[lo + t] = packed;
                else if (MODE == T_NARROW) tb.sym[lo + t] = (uint8_t)s;
                else atomicOr(&tb.l1[(lo + t) * L1S], li << 2);
            }
        }
        uint32_t m = __ballot_sync(0xffffffffu, big);
        while (m) {
            int src = __ffs(m) - 1;
            m &= m - 1;
            uint32_t bc = __shfl_sync(0xffffffffu, cnt, src);
            uint32_t bl = __shfl_sync(0xffffffffu, lo, src);
            uint32_t bp = __shfl_sync(0xffffffffu, packed, src);
            uint32_t bi = __shfl_sync(0xffffffffu, li, src);
            for (uint32_t t = lane; t < bc; t += 32) {
                if (MODE == T_WIDE || MODE == T_WIDE1) tb.wide[bl + t] = bp;
                else if (MODE == T_NARROW) tb.sym[bl + t] = (uint8_t)bp;
                else atomicOr(&tb.l1[(bl + t) * L1S], bi << 2);
            }
        }
    }
    __syncwarp();
    return true;
}

// One decode step for this lane.  `active` is false for lanes past the end of
// a ragged stream: they keep their state, refill nothing and emit nothing.
template <int MODE>
__device__ __forceinline__ uint32_t rans_step(uint32_t &x, uint32_t &cursor, const Ring &ring,
                                              const Tables &tb, uint32_t lt_mask,
                                              uint32_t grp_mask, bool active)
{
    uint32_t slot = x & (PROB_SCALE - 1);
    uint32_t sym, x2;
    if (MODE == T_NARROW) {
        sym = tb.sym[slot];
        uint32_t p = tb.sf[sym];
        x2 = ((p >> 12) + 1) * (x >> PROB_BITS) + slot - (p & 0xfffu);
    } else {
        static_assert(MODE != T_COMPACT && MODE != T_WIDE1, "compact and per-stream wide tables are decoded by k_stream");
        uint32_t e = tb.wide[slot];
        sym = e & 0xffu;
        x2 = ((e >> 20) + 1) * (x >> PROB_BITS) + slot - ((e >> 8) & 0xfffu);
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
