// Batch rANS decode kernel: one 8-lane group per stream, four streams per warp,
// decoded bytes written stream by stream to global memory.
#pragma once
#include "rans.cuh"

namespace lmz {

struct RansArgs {
    const uint8_t *src;         // compressed bytes (16-byte aligned base, PAD_BYTES of slack after)
    const StreamJob *jobs;      // njobs descriptors, or NULL to use `offs`/`plane`
    const uint64_t *offs;       // reference layout: (offset, length) pairs
    uint32_t plane;             // symbols per stream when `offs` is used
    uint32_t njobs;
    uint8_t *dst;
    const uint8_t *shared_hdr;  // 516-byte table shared by every stream (WIDE kernels)
    uint32_t *status;           // one word per job, may be NULL
    uint32_t *any_bad;          // set non-zero when a job fails hard, may be NULL
};

// Shared-memory footprint.  The per-group stride is chosen so the four staging
// areas of a warp sit 8 banks apart.
constexpr uint32_t STAGE_BYTES = 160;
constexpr uint32_t WIDE_TAB_BYTES = PROB_SCALE * 4;

// Bytes of per-stream tables, and the whole per-group footprint, by table layout.
__host__ __device__ constexpr uint32_t table_bytes(int mode)
{
    return mode == T_NARROW ? PROB_SCALE + 1024 : 0;
}
__host__ __device__ constexpr uint32_t group_bytes(int mode)
{
    // ring | tables | staging | mbarriers | pad (stride = 8 banks mod 32)
    return RING + table_bytes(mode) + STAGE_BYTES + 32 + (mode == T_WIDE ? 32 : 96);
}
static_assert(group_bytes(T_NARROW) == 6432 && group_bytes(T_WIDE) == 1248, "per-group shared memory layout");

template <int MODE>
__host__ __device__ constexpr uint32_t rans_smem_bytes(int warps)
{
    return (MODE == T_WIDE ? WIDE_TAB_BYTES : 0) + warps * 4 * group_bytes(MODE);
}

// Point a group's table pointers at its slice of shared memory.
template <int MODE>
__device__ __forceinline__ Tables group_tables(uint8_t *gp, uint32_t *wide_tab)
{
    Tables tb{};
    if (MODE == T_NARROW) {
        tb.sym = gp + RING;
        tb.sf = reinterpret_cast<uint32_t *>(gp + RING + PROB_SCALE);
    } else {
        static_assert(MODE == T_NARROW || MODE == T_WIDE, "the other table layouts are decoded by k_stream");
        tb.wide = wide_tab;
    }
    return tb;
}

template <int MODE, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) k_rans(RansArgs a)
{
    constexpr bool WIDE = MODE == T_WIDE;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t k = lane & 7u, g = lane >> 3;
    const uint32_t grp_mask = 0xffu << (g * 8), lt_mask = ((1u << k) - 1u) << (g * 8);
    constexpr uint32_t GB = group_bytes(MODE);
    uint32_t *wide_tab = WIDE ? reinterpret_cast<uint32_t *>(smem) : nullptr;
    uint8_t *warp_base = smem + (WIDE ? WIDE_TAB_BYTES : 0) + (size_t)warp * 4 * GB;
    uint8_t *gp = warp_base + (size_t)g * GB;

    Ring ring;
    ring.buf = gp;
    const Tables tb = group_tables<MODE>(gp, wide_tab);
    uint8_t *stage = gp + RING + table_bytes(MODE);
    ring.bars = reinterpret_cast<uint64_t *>(stage + STAGE_BYTES);

    // ---- this group's stream ------------------------------------------------
    const uint32_t job = (blockIdx.x * WARPS + warp) * 4 + g;
    const bool have = job < a.njobs;
    uint64_t soff = 0, doff = 0;
    uint32_t slen = 0, n = 0;
    if (have) {
        if (a.jobs) {
            StreamJob j = a.jobs[job];
            soff = j.src_off; doff = j.dst_off; slen = j.src_len; n = j.n;
        } else {
            soff = a.offs[2 * job]; slen = (uint32_t)a.offs[2 * job + 1];
            n = a.plane; doff = (uint64_t)job * a.plane;
        }
    }
    constexpr uint32_t LEAD = WIDE ? STATE_BYTES : HDR_BYTES + STATE_BYTES;
    uint32_t st = ST_OK;
    if (n != 0 && slen < LEAD) { st = ST_BAD_HEADER; n = 0; }
    if (n == 0) slen = 0;
    const uint8_t *sbase = a.src + soff;
    const uint32_t skew = (uint32_t)(reinterpret_cast<uintptr_t>(sbase) & 15u);
    ring.abase = sbase - skew;
    ring.valid_slots = n ? (skew + slen + SLOT - 1) / SLOT : 0;
    ring.issued = 0; ring.ready = 0; ring.dead = false;

    if (k == 0)
        for (uint32_t j = 0; j < NSLOT; j++) mbar_init(&ring.bars[j], 1);
    mbar_fence_init();
    __syncthreads();

    ring.issue(0, k == 0);
    __syncwarp();
    ring.require(skew + LEAD);

    // ---- tables --------------------------------------------------------------
    if (WIDE) {
        if (warp == 0) {
            const uint8_t *h = a.shared_hdr;
            bool ok = build_table<T_WIDE>(
                [&](uint32_t s) { return (uint32_t)h[4 + 2 * s] | ((uint32_t)h[5 + 2 * s] << 8); },
                tb, lane);
            if (!ok || h[0] != 'R' || h[1] != '1') wide_tab[0] = 0xffffffffu;  // poison marker
        }
        __syncthreads();
        // A table that did not validate poisons every stream of the block.
        if (wide_tab[0] == 0xffffffffu && n) { st = ST_BAD_HEADER; n = 0; }
    } else {
#pragma unroll 1
        for (uint32_t gg = 0; gg < 4; gg++) {
            uint32_t on = __shfl_sync(0xffffffffu, n, gg * 8);
            if (!on) continue;
            uint32_t sk = __shfl_sync(0xffffffffu, skew, gg * 8);
            uint8_t *rb = warp_base + (size_t)gg * GB;
            auto rd = [&](uint32_t o) { return (uint32_t)rb[o & (RING - 1)]; };
            bool ok = build_table<MODE>(
                [&](uint32_t s) { return rd(sk + 4 + 2 * s) | (rd(sk + 5 + 2 * s) << 8); },
                group_tables<MODE>(rb, nullptr), lane);
            ok = ok && rd(sk) == 'R' && rd(sk + 1) == '1';
            if (!ok && g == gg) { st = ST_BAD_HEADER; n = 0; }
        }
    }
    __syncwarp();

    uint32_t x = ring.u32_at(skew + (WIDE ? 0 : HDR_BYTES) + 4 * k);
    uint32_t cursor = skew + LEAD;
    uint8_t *out = a.dst + doff;
    const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;

    // ---- tiles ---------------------------------------------------------------
    const uint32_t my_tiles = (n + TILE - 1) / TILE;
    const uint32_t warp_tiles = __reduce_max_sync(0xffffffffu, my_tiles);
#pragma unroll 1
    for (uint32_t t = 0; t < warp_tiles; t++) {
        const uint32_t done = t * TILE;
        const uint32_t rem = n > done ? n - done : 0;
        __syncwarp();
        if (rem) {
            ring.issue(cursor, k == 0);
            ring.require(cursor + 2 * TILE);
        }
        __syncwarp();
        if (__all_sync(0xffffffffu, rem >= TILE)) {
#pragma unroll
            for (uint32_t s = 0; s < TILE / NLANES; s++) {
                uint32_t sym = rans_step<MODE>(x, cursor, ring, tb, lt_mask, grp_mask, true);
                stage[s * NLANES + k] = (uint8_t)sym;
            }
        } else {
#pragma unroll 1
            for (uint32_t s = 0; s < TILE / NLANES; s++) {
                bool active = s * NLANES + k < rem;
                uint32_t sym = rans_step<MODE>(x, cursor, ring, tb, lt_mask, grp_mask, active);
                if (active) stage[s * NLANES + k] = (uint8_t)sym;
            }
        }
        __syncwarp();
        if (rem >= TILE && aligned) {
            uint4 v = *reinterpret_cast<const uint4 *>(stage + k * 16);
            *reinterpret_cast<uint4 *>(out + done + k * 16) = v;
        } else if (rem) {
            uint32_t cnt = rem < TILE ? rem : TILE;
            for (uint32_t i = k * 16; i < k * 16 + 16 && i < cnt; i++) out[done + i] = stage[i];
        }
    }

    // ---- verdict -------------------------------------------------------------
    bool rest = x == RANS_LOW;
    uint32_t all_rest = __ballot_sync(0xffffffffu, rest) & grp_mask;
    if (have && k == 0) {
        if (st == ST_OK && n) {
            uint32_t used = cursor - skew;
            if (ring.dead) st = ST_TIMEOUT;
            else if (used > slen) st = ST_OVERRUN;
            else if (used != slen || all_rest != grp_mask) st = ST_SLACK;
        }
        if (a.status) a.status[job] = st;
        if (a.any_bad && st != ST_OK && st != ST_SLACK) atomicOr(a.any_bad, 1u);
    }
}

}  // namespace lmz
