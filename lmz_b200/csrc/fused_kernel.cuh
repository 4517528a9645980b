// k_stream: the throughput kernel.  One 8-lane group per rANS stream, compact
// per-stream tables, and the stream's consumer fused into the decode loop:
//
//   SINK_BYTES  the decoded plane is written as is (decode_batch, scratch planes)
//   SINK_BF16   a CODEC_BF16 chunk whose exponent plane is rANS and whose
//               sign/mantissa plane is stored: each 128-symbol tile is merged with
//               128 stored bytes (lmz/native/lmzcore.c:439-447), written once as
//               256 bytes of BF16, and folded into the chunk's CRC-32 -- no
//               scratch plane, no second pass
//   SINK_F32    a CODEC_SPLIT chunk of 4-byte elements whose top byte plane is rANS
//               and whose three lower planes are stored back to back: each tile is
//               interleaved with 3 x 128 stored bytes (lmz/native/lmzcore.c:289-347),
//               written once as 512 bytes and folded into the chunk's CRC-32
//   SINK_DELTA  a delta chunk (lmz/codec.py:1012-1057) whose difference is a CODEC_BF16
//               chunk with both planes rANS: two neighbouring groups of a warp decode the two
//               planes in step, the merged difference is XOR-ed with the base bytes already
//               in the output space, written once and checksummed (CFN = 192: a 128-entry
//               level 2 for the first plane, a 256-entry one for the second)
//
// Differences from k_rans that buy instructions and occupancy:
//   * shared memory is laid out by kind (all level-1 tables, all level-2 tables,
//     all rings ...) so each table base is aligned to its size and an address is
//     (index bits) | base in one logic op; a warp's four level-1 tables interleave
//     word by word, which drops the index shift and keeps the four streams' lookups
//     in different banks
//   * the input ring (4 x 128 B) is followed by a mirror of its first 272 bytes,
//     filled by the same bulk copies, so a tile reads linearly with no wrap masks
//   * refill offsets come from a 4-step history of the group's votes: one
//     byte-permute and one popcount per step instead of two popcounts
//   * CFN = 128: level 2 has 128 slots, the four streams of a warp rotated 8
//     entries apart so their popular symbols sit in different banks; streams with
//     more than 104 live symbols must be given to the CFN = 256 instance
//   * CFN = 0: no levels, a 16 KiB slot -> entry table per stream and 12 streams per
//     CTA, 256-symbol tiles: for launches so small that only the length of a symbol's
//     dependent chain counts (one lookup instead of two and a popcount)
//   * CFN = 0 with a fourth warp: 13 streams per CTA -- the tables on 16 KiB boundaries, the rings
//     (shorter) in what is left below the first and above the last -- and every symbol stored
//     straight to its output byte (no staging row)
//   * CFN = -1: the same wide table once per CTA, for batches whose streams share one
//     516-byte table (lmz_gpu_decode_batch's d_hdr) or for the chunks of a shared-table
//     archive (StreamArgs.tables); a stream is then states + words
#pragma once
#include "chunk_kernels.cuh"
#include "rans.cuh"

namespace lmz {

enum : int { SINK_BYTES = 0, SINK_BF16 = 1, SINK_F32 = 2, SINK_DELTA = 3 };
constexpr uint32_t F_SLOT = 128, F_NSLOT = 4, F_RING = F_SLOT * F_NSLOT;
constexpr uint32_t F_MIRROR = 272;                 // a tile reads at most 256 + 2 bytes ahead
constexpr uint32_t F_RING_BYTES = F_RING + F_MIRROR;        // 784
constexpr uint32_t F_STAGE = 144;                  // 128 + 16: groups land 4 banks apart
// The per-stream wide instance (CFN = 0) runs one warp per scheduler, where every
// instruction of tile bookkeeping is paid in full, and has shared memory to spare beside
// its 12 tables: its tiles are twice as long (256 symbols) and its ring twice as deep.
__host__ __device__ constexpr bool stream_long_tiles(int cfn, int warps) { return cfn == 0 && (warps == 3 || warps == 4); }
// The same with a thirteenth stream (a fourth warp that carries one): thirteen tables on 16 KiB
// boundaries leave 19 KiB in two pieces, under the first and above the last, enough for rings of six
// slots instead of eight and for no staging rows -- every symbol goes straight to its byte of the output.  For launches of 12 x SMs + 1 ... 13 x SMs
// streams (the 1915 long streams of an 8B model at the reference's default chunking, on 148 SMs).
__host__ __device__ constexpr bool stream_direct(int cfn, int warps) { return cfn == 0 && warps == 4; }
constexpr uint32_t F_DIRECT_GROUPS = 13;
__host__ __device__ constexpr uint32_t stream_tile(int cfn, int warps) { return stream_long_tiles(cfn, warps) ? 256u : 128u; }
__host__ __device__ constexpr uint32_t stream_nslot(int cfn, int warps) { return stream_direct(cfn, warps) ? 6u : stream_long_tiles(cfn, warps) ? 8u : F_NSLOT; }
__host__ __device__ constexpr uint32_t stream_mirror(int cfn, int warps) { return stream_long_tiles(cfn, warps) ? 528u : F_MIRROR; }
__host__ __device__ constexpr uint32_t stream_ring_bytes(int cfn, int warps)
{
    return F_SLOT * stream_nslot(cfn, warps) + stream_mirror(cfn, warps);
}
__host__ __device__ constexpr uint32_t stream_stage(int cfn, int warps) { return stream_direct(cfn, warps) ? 0u : stream_long_tiles(cfn, warps) ? 272u : F_STAGE; }
constexpr uint32_t F_LOGS = 3;                     // eight copies of the CRC slice tables (32 KiB), one per lane of a group: see CrcQuarters
constexpr uint32_t F_CRC_BYTES = (4096u << F_LOGS) + 4096u;   // + the row-advance tables, once
constexpr uint32_t F_ROW = 256, F_UNIT = 32;       // bytes of BF16 one group / one lane emits per tile
constexpr int F_SMALL_CFN = 128;                   // level-2 slots of the dense instance
constexpr int F_HYBRID_CFN = 192;                  // delta sink: 128-entry tables for first planes, 256-entry for second planes
constexpr uint32_t F_SMALL_LIVE = F_SMALL_CFN - 24; // largest alphabet it takes (the warp's streams sit 0, 8, 16, 24 entries in)

struct FusedJob {
    uint64_t src_off;    // rANS stream, bytes from the source base
    uint64_t mant_off;   // SINK_BF16: the stored sign/mantissa plane, bytes from the source base;
                         // SINK_F32: stored plane 0, planes 1 and 2 follow at n and 2n
    uint64_t dst_off;    // first output byte
    uint32_t src_len;
    uint32_t n;          // symbols (= elements)
    uint32_t piece0;     // first piece id of the chunk (for piece_crc)
    uint32_t flags;
};
static_assert(sizeof(FusedJob) == 40, "FusedJob layout is shared with the host");

// SINK_DELTA: a delta chunk (lmz/codec.py:1012-1057) whose difference is a CODEC_BF16 chunk
// with both planes rANS-coded.  Two neighbouring stream groups of a warp decode the two
// planes in step; the merged difference is XOR-ed with the base bytes, which are already in
// the output space, and written once.
struct DeltaJob {
    uint64_t src_a, src_b;   // the exponent plane's and the sign/mantissa plane's streams
    uint64_t dst_off;        // first output byte
    uint64_t base_off;       // the chunk this one is a difference against, in the output space
    uint32_t len_a, len_b;
    uint32_t n;              // elements
    uint32_t piece0;
};
static_assert(sizeof(DeltaJob) == 48, "DeltaJob layout is shared with the host");

struct StreamArgs {
    const uint8_t *src;
    const FusedJob *jobs;       // SINK_BF16 jobs, or NULL
    const StreamJob *sjobs;     // plain stream jobs, or NULL
    const DeltaJob *djobs;      // SINK_DELTA: njobs counts streams, two per job
    const uint64_t *offs;       // neither: reference layout, (offset, length) pairs + plane
    uint32_t plane;
    uint32_t njobs;
    uint8_t *dst;
    uint32_t *status;
    uint32_t *any_bad;
    uint32_t *piece_crc;        // SINK_BF16 with checksums: R() per 64 KiB piece
    const CrcTables *tabs;
    const uint8_t *shared_hdr;  // CFN = -1: the 516-byte table every stream of the launch shares
    const uint8_t *tables;      // CFN = -1, or NULL: the 516-byte tables of a shared-table archive, F_TABLE_STRIDE
                                // bytes apart; a CTA's streams all use table number `flags` of its first job
    // Optional indirection, filled on the device by k_classify: the launch covers the
    // first *count entries of `order` (read from its end backwards when order_from_back),
    // each the index of a job; CTAs past the count leave at once.
    const uint32_t *order;
    const uint32_t *count;
    uint32_t order_from_back;
    // Streams per CTA (a multiple of 4, at most the instance's capacity; 0 = the capacity):
    // the launcher spreads a launch evenly over its waves of CTAs, so that a launch of 3.03
    // waves runs as four waves of three quarters the streams instead of three full waves
    // and one nearly empty one, and a small launch uses every SM.
    uint32_t per_cta;
};

constexpr uint32_t F_WIDE_BYTES = PROB_SCALE * 4;   // CFN = 0: one 16 KiB slot -> entry table per stream
constexpr int F_WIDE_GROUPS = 12;                   // three full warps; 13 tables would fit, but not their rings
__host__ __device__ constexpr uint32_t stream_group_bytes(int cfn)
{
    return (cfn > 0 ? 1024 + 4 * cfn : cfn == 0 ? F_WIDE_BYTES : 0) + F_RING_BYTES + F_STAGE + 32;   // 3008 / 2496 / 17344 / 960
}
constexpr int F_SHARED_WARPS = 16;                  // CFN = -1: one table per CTA, two CTAs per SM (64 registers a thread)
constexpr uint32_t F_TABLE_STRIDE = 528;            // 516 rounded up to 16
constexpr int F_SHARED_SINK_WARPS = 20;             // CFN = -1 with the BF16 sink: one CTA per SM, 80 chunks sharing its table
// Streams are carved from the bottom of the CTA's shared memory and the CRC tables
// from the top (slice tables 8 KiB aligned, row-advance tables above them), so the
// launch asks for everything the device lets one CTA have: 227 KiB that start
// F_SMEM_BASE bytes into the shared window (the launcher checks that reservation).
constexpr uint32_t F_SMEM_BASE = 1024, F_SMEM_DYN = 232448;
__host__ __device__ constexpr uint32_t stream_crc_adv(uint32_t top) { return (top - 4096u) & ~1023u; }
__host__ __device__ constexpr uint32_t stream_crc_slice(uint32_t top)
{
    return (stream_crc_adv(top) - (4096u << F_LOGS)) & ~((1024u << F_LOGS) - 1u);
}
// The BF16 sink's checksum needs no row-advance tables (see k_stream), so the 4 KiB they
// would take, above the slice tables, hold the level-1 tables of the CTA's last warp.
__host__ __device__ constexpr bool stream_top_l1(int sink, bool crc, int cfn) { return (sink == SINK_BF16 || sink == SINK_DELTA) && crc && cfn > 0; }
__host__ __device__ constexpr int stream_warps(int cfn, bool crc, int sink = SINK_BYTES)
{
    constexpr uint32_t top = F_SMEM_BASE + F_SMEM_DYN;
    if (cfn == 0) return F_WIDE_GROUPS / 4;
    if (cfn < 0) return sink == SINK_BF16 ? F_SHARED_SINK_WARPS : F_SHARED_WARPS;
    const uint32_t room = (crc ? stream_crc_slice(top) : top) - F_SMEM_BASE + (stream_top_l1(sink, crc, cfn) ? 4096u : 0u);
    int w = (int)(room / (4u * stream_group_bytes(cfn)));
    // Registers are shared per scheduler: a 21st warp would put six on one of the four and cut every
    // thread from 96 registers to 80 (which this kernel does not fit in), so 20 is the most.
    if (crc && w > 20) w = 20;
    return w;
}
__host__ __device__ constexpr unsigned stream_groups(int cfn, int warps) { return warps * 4; }
static_assert(F_LOGS == 3 && stream_crc_slice(F_SMEM_BASE + F_SMEM_DYN) % 32768u == 0,
              "crc_feed4q ORs a 32 KiB table's offsets onto its base");
static_assert(stream_warps(128, true) == 19 && stream_warps(256, true) == 16 &&
              stream_warps(128, false) == 23 && stream_warps(256, false) == 19 &&
              stream_warps(128, true, SINK_BF16) >= 19 && stream_warps(256, true, SINK_BF16) == 16, "shared memory budget");

__device__ __forceinline__ void bulk_g2s_sa(uint32_t dst_sa, const void *src, uint32_t bytes,
                                            uint32_t bar_sa)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_sa), "l"(src), "r"(bytes), "r"(bar_sa) : "memory");
}

// Input ring with a mirror of its head behind it.  Offsets are bytes from `abase`.
template <uint32_t NSLOT_, uint32_t MIRROR_>
struct MRingT {
    static constexpr uint32_t F_NSLOT = NSLOT_, F_RING = F_SLOT * NSLOT_, F_MIRROR = MIRROR_;
    uint32_t sa;           // shared address of the ring
    uint64_t *bars;
    const uint8_t *abase;
    uint32_t valid_slots, issued, ready;
    bool dead;

    // Every lane of the group keeps `issued` (so the usual "nothing to request" costs no
    // divergent branch); only the leader touches the barrier and starts the copies.
    __device__ __forceinline__ void issue(uint32_t cursor, bool leader)
    {
        uint32_t lim = cursor / F_SLOT + F_NSLOT;
        if (lim > valid_slots) lim = valid_slots;
        while (issued < lim) {
            if (leader) {
                uint32_t j = issued % F_NSLOT;
                uint32_t m = j * F_SLOT < F_MIRROR ? min(F_SLOT, F_MIRROR - j * F_SLOT) : 0u;
                const uint8_t *g = abase + (size_t)issued * F_SLOT;
                mbar_expect_tx(&bars[j], F_SLOT + m);
                bulk_g2s_sa(sa + j * F_SLOT, g, F_SLOT, smem_addr(&bars[j]));
                if (m) bulk_g2s_sa(sa + F_RING + j * F_SLOT, g, m, smem_addr(&bars[j]));
            }
            issued++;
        }
    }
    __device__ __forceinline__ void require(uint32_t upto)
    {
        uint32_t need = (upto + F_SLOT - 1) / F_SLOT;
        if (need > valid_slots) need = valid_slots;
        while (ready < need) {
            if (!dead && !mbar_wait(&bars[ready % F_NSLOT], (ready / F_NSLOT) & 1u)) dead = true;
            ready++;
        }
    }
    __device__ __forceinline__ uint32_t byte_at(uint32_t o) const { return lds_u8(sa + (o & (F_RING - 1))); }
    __device__ __forceinline__ uint32_t u16_at(uint32_t o) const { return byte_at(o) | (byte_at(o + 1) << 8); }
    __device__ __forceinline__ uint32_t u32_at(uint32_t o) const { return u16_at(o) | (u16_at(o + 2) << 16); }
};

// Table lookups and the state update of one decode step, before the refill.
// Returns the level-2 entry (its low byte is the symbol); x2 is the new state.
template <int CFN>
__device__ __forceinline__ uint32_t stream_advance(uint32_t x, uint32_t l1_sa, uint32_t cf_sa, uint32_t &x2)
{
    uint32_t e;
    if (CFN <= 0) {
        // wide table at l1_sa (the stream's own, or the CTA's shared one), 16 KiB aligned: one
        // lookup, the index OR-ed onto the base
        e = lds_u32(((x << 2) & 0x3ffcu) | l1_sa);
    } else {
        // level 1: the warp's four tables are interleaved word by word, so bucket b of
        // this group sits 16 * b bytes in -- the slot's bits 4-11, unshifted
        const uint32_t e1 = lds_u32((x & 0xff0u) | l1_sa);
        const uint32_t upto = 0xffffffffu >> ((~x) & 15u);             // bits 0 .. 16 + (slot & 15)
        const uint32_t pc = __popc(e1 & upto & 0xffff0000u);
        constexpr uint32_t IDX = 4u * (uint32_t)(CFN > 0 ? CFN : 1) - 4u;   // byte offset field of level 1
        e = lds_u32(((e1 & IDX) | cf_sa) + (pc << 2));
    }
    // f * (x >> 12) + slot - start  ==  x - (x >> 12) * (4096 - f) - start
    x2 = x - ((x >> PROB_BITS) * (e >> 20) + ((e >> 8) & 0xfffu));
    return e;
}

// One decode step, any lane mix.  `caddr` is the shared address of the cursor
// (linear within a tile thanks to the mirror).
template <int CFN>
__device__ __forceinline__ uint32_t stream_step(uint32_t &x, uint32_t &caddr, uint32_t l1_sa,
                                                uint32_t cf_sa, uint32_t lt_mask, uint32_t grp_mask,
                                                bool active)
{
    uint32_t x2;
    const uint32_t e = stream_advance<CFN>(x, l1_sa, cf_sa, x2);
    const bool need = active && x2 < RANS_LOW;
    const uint32_t vote = __ballot_sync(0xffffffffu, need);
    const uint32_t addr = caddr + 2 * __popc(vote & lt_mask);
    const uint32_t lo = lds_u8(addr), hi = lds_u8_1(addr);
    if (need) x2 = ((x2 << 8) + hi << 8) + lo;
    if (active) x = x2;
    caddr += 2 * __popc(vote & grp_mask);
    return e;
}

// One step of a full tile, four to a block.  `hist` collects the group's votes of
// the block, newest in byte 0 (vsel = 0x6540 + group picks this group's byte of
// the warp vote and shifts the older ones up); refills consumed before this
// lane's = bits of the older bytes plus the lanes below it in the newest, so one
// popcount of hist & below (= 0xffffff00 | lanes below) gives the offset from
// the block's cursor.  The caller adds 2 * popc(hist) to `cbase` after step 3.
template <int CFN, bool FIRST>
__device__ __forceinline__ uint32_t stream_step4(uint32_t &x, uint32_t &hist, uint32_t cbase,
                                                 uint32_t l1_sa, uint32_t cf_sa, uint32_t below,
                                                 uint32_t vsel)
{
    uint32_t x2;
    const uint32_t e = stream_advance<CFN>(x, l1_sa, cf_sa, x2);
    const bool need = x2 < RANS_LOW;
    const uint32_t vote = __ballot_sync(0xffffffffu, need);
    hist = __byte_perm(vote, FIRST ? 0u : hist, vsel);
    const uint32_t addr = cbase + 2 * __popc(hist & below);
    const uint32_t lo = lds_u8(addr), hi = lds_u8_1(addr);
    if (need) x2 = ((x2 << 8) + hi << 8) + lo;       // two predicated shift-adds, no select
    x = x2;
    return e;
}

template <int SINK, bool CRC, int WARPS, int CFN>
__global__ void __launch_bounds__(WARPS * 32, CFN < 0 && SINK == SINK_BYTES ? 2 : 1) k_stream(StreamArgs a)
{
    // SINK_BF16 checksums: lane k keeps one running value per word of its 32-byte unit,
    // ra[i] = sum over the piece's rows so far of word i * x^(2048 * rows since); a row
    // costs each of them one multiplication by x^2048 (the same four lookups as feeding a
    // word) with no chain between the eight and no per-row advance; the constants
    // word_mul[k][i] carry them to the piece's end.
    constexpr bool ROWMUL = (SINK == SINK_BF16 || SINK == SINK_DELTA) && CRC;
    constexpr int NRA = SINK == SINK_DELTA ? 4 : 8;        // running values per lane: words of its unit of a row
    constexpr bool TOPL1 = stream_top_l1(SINK, CRC, CFN);
    extern __shared__ __align__(16) uint8_t ssm[];
    constexpr bool WIDE = CFN <= 0, SHARED = CFN < 0;
    constexpr bool DIRECT = stream_direct(CFN, WARPS);
    static_assert(!DIRECT || SINK == SINK_BYTES, "the 13-stream instance writes bytes only");
    // SINK_DELTA with CFN = 192: the two planes of a chunk have level-2 tables of different sizes, 128
    // entries for the exponent differences (a handful of symbols) and 256 for the sign/mantissa
    // differences, 768 bytes a stream on average; the decode steps are those of the 256-entry instance.
    constexpr bool HYB = SINK == SINK_DELTA && CFN == F_HYBRID_CFN;
    constexpr int CFN_STEP = HYB ? 256 : CFN;
    constexpr uint32_t G = DIRECT ? F_DIRECT_GROUPS : stream_groups(CFN, WARPS), CFB = WIDE ? 16u : 4u * CFN;
    constexpr uint32_t CF_ALIGN = HYB ? 1024u : CFB;
    static_assert(CFN != F_HYBRID_CFN || SINK == SINK_DELTA, "mixed table sizes are the delta sink's");
    constexpr uint32_t LEAD = (SHARED ? 0u : HDR_BYTES) + STATE_BYTES;
    constexpr uint32_t MAX_LIVE = CFN > 0 && CFN < 256 ? (uint32_t)CFN - 24u : 256u;
    constexpr uint32_t TS = stream_tile(CFN, WARPS), NSL = stream_nslot(CFN, WARPS), RB = stream_ring_bytes(CFN, WARPS);
    constexpr uint32_t STG = stream_stage(CFN, WARPS), RINGB = F_SLOT * NSL;
    constexpr uint32_t HS = NSL != F_NSLOT ? 160u : 144u;     // header staging copy: four of them cover 548 + 15 bytes
    static_assert(CFN != 0 || !CRC, "the per-stream wide instance has no room for CRC tables");
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    // DIRECT: the fourth warp carries one stream; its other three groups shadow it (same tables,
    // ring and states, no copies requested, nothing stored) so that the warp decodes full tiles
    const uint32_t k = lane & 7u, g = lane >> 3, gi = DIRECT ? min(warp * 4 + g, G - 1) : warp * 4 + g;
    const bool shadow = DIRECT && warp * 4 + g > gi;
    const uint32_t grp_mask = 0xffu << (g * 8), lt_mask = ((1u << k) - 1u) << (g * 8);
    const uint32_t below = 0xffffff00u | ((1u << k) - 1u), vsel = 0x6540u + g;

    // ---- carve shared memory (addresses are 32-bit shared-space addresses) --------
    // small per-stream pieces from the bottom; level-1 tables (4 KiB per warp, the
    // four streams interleaved) end where the CRC tables begin, or at the top
    const uint32_t s0 = smem_addr(ssm), top = s0 + dynamic_smem_bytes();
    const uint32_t adv0 = stream_crc_adv(top), tab0 = stream_crc_slice(top);
    const uint32_t bars_0 = (s0 + 15u) & ~15u;
    const uint32_t stage_0 = bars_0 + G * 8 * NSL;
    const uint32_t ring_0 = stage_0 + G * STG;
    // DIRECT: thirteen 16 KiB tables leave 19 KiB of the window, some of it below the first 16 KiB
    // boundary and some above the last table: the tables sit on boundaries (an index is OR-ed onto the
    // base, which is what makes the step as short as the 12-stream instance's) and the rings fill both
    // remainders, `ring_below` of them under the tables.
    const uint32_t dl1_0 = (ring_0 + F_WIDE_BYTES - 1) & ~(F_WIDE_BYTES - 1);
    const uint32_t ring_below = DIRECT ? min(G, (dl1_0 - ring_0) / RB) : G;
    const uint32_t ring_above_0 = dl1_0 + G * F_WIDE_BYTES;
    auto ring_of = [&](uint32_t grp) { return DIRECT && grp >= ring_below ? ring_above_0 + (grp - ring_below) * RB : ring_0 + grp * RB; };
    const uint32_t cf_0 = (ring_0 + G * RB + CF_ALIGN - 1) & ~(CF_ALIGN - 1);
    // compact: level 1 at the top; wide: 16 KiB tables from the first 16 KiB boundary up
    const uint32_t l1_0 = DIRECT ? dl1_0 : WIDE ? (cf_0 + F_WIDE_BYTES - 1) & ~(F_WIDE_BYTES - 1)
                               : ((CRC ? tab0 : top) & ~4095u) - (WARPS - (TOPL1 ? 1 : 0)) * 4096u;
    // compact: this warp's 4 KiB of level 1 (the last warp's sits where the row-advance tables would)
    auto l1_of = [&](uint32_t w) { return TOPL1 && w == WARPS - 1 ? adv0 : l1_0 + w * 4096u; };
    const bool fits = DIRECT ? ring_above_0 + (G - ring_below) * RB <= top
                    : WIDE ? l1_0 + (SHARED ? 1u : G) * F_WIDE_BYTES <= (CRC ? tab0 : top)
                           : cf_0 + G * CFB <= l1_0 && (!TOPL1 || (adv0 & 4095u) == 0);
    auto gen = [&](uint32_t sa) { return ssm + (sa - s0); };
    const uint32_t l1_sa = SHARED ? l1_0 : WIDE ? l1_0 + gi * F_WIDE_BYTES : l1_of(warp) + g * 4;
    // (mixed sizes: the 1 KiB tables of the second planes first, then the half-KiB tables of the first planes)
    auto cf_of = [&](uint32_t grp) { return HYB ? ((grp & 1u) ? cf_0 + (grp >> 1) * 1024u : cf_0 + (G / 2) * 1024u + (grp >> 1) * 512u)
                                               : cf_0 + grp * CFB; };
    const uint32_t cf_sa = cf_of(gi);
    const uint32_t stage_sa = stage_0 + gi * STG;
    // byte (i + g) & 3 of a state word goes through slice table 3 - ((i + g) & 3)
    CrcQuarters cq;
#pragma unroll
    for (uint32_t i = 0; i < 4; i++) cq.b[i] = tab0 + 32u * (3u - ((i + g) & 3u)) + 4u * k;
    cq.rot = 8u * g;
    const uint32_t tla = adv0 - 4096u;                              // crc_advance<0> adds 4 .. 7 KiB

    MRingT<NSL, stream_mirror(CFN, WARPS)> ring;
    ring.sa = ring_of(gi);
    ring.bars = reinterpret_cast<uint64_t *>(gen(bars_0)) + gi * NSL;

    // ---- this group's stream ------------------------------------------------------
    const uint32_t per_cta = a.per_cta ? a.per_cta : G;
    const uint32_t idx = blockIdx.x * per_cta + gi;
    uint32_t limit = a.njobs;
    if (a.count) {
        limit = SINK == SINK_DELTA ? 2u * *a.count : *a.count;     // (delta: the count is of chunks, two streams each)
        if (blockIdx.x * per_cta >= limit) return;    // the whole CTA: nothing of this class is left
    }
    const bool have = gi < per_cta && idx < limit;
    // (SINK_DELTA: `order` lists chunks; stream 2c + p is plane p of chunk c)
    const uint32_t job = !(have && a.order) ? idx
                       : SINK == SINK_DELTA ? 2u * a.order[a.order_from_back ? a.njobs / 2 - 1 - (idx >> 1) : idx >> 1] + (idx & 1u)
                                            : a.order[a.order_from_back ? a.njobs - 1 - idx : idx];
    uint64_t soff = 0, doff = 0, moff = 0;
    uint32_t slen = 0, n = 0, piece0 = 0;
    if (have) {
        if (SINK == SINK_DELTA) {
            // groups 2c and 2c + 1 of the CTA take the two planes of its chunk c
            const DeltaJob j = a.djobs[job >> 1];
            soff = (job & 1u) ? j.src_b : j.src_a; slen = (job & 1u) ? j.len_b : j.len_a;
            doff = j.dst_off; moff = j.base_off; n = j.n; piece0 = j.piece0;
        } else if (a.jobs) {
            FusedJob j = a.jobs[job];
            soff = j.src_off; doff = j.dst_off; moff = j.mant_off;
            slen = j.src_len; n = j.n; piece0 = j.piece0;
        } else if (a.sjobs) {
            StreamJob j = a.sjobs[job];
            soff = j.src_off; doff = j.dst_off; slen = j.src_len; n = j.n;
        } else {
            soff = a.offs[2 * job]; slen = (uint32_t)a.offs[2 * job + 1];
            n = a.plane; doff = (uint64_t)job * a.plane;
        }
    }
    uint32_t st = ST_OK;
    if (!fits) { st = ST_BAD_SHAPE; n = 0; }          // the launch gave less shared memory than the layout needs
    if (n != 0 && slen < LEAD) { st = ST_BAD_HEADER; n = 0; }
    if (n == 0) slen = 0;
    const uint8_t *sbase = a.src + soff;
    const uint32_t skew = (uint32_t)(reinterpret_cast<uintptr_t>(sbase) & 15u);
    ring.abase = sbase - skew;
    ring.valid_slots = n ? (skew + slen + F_SLOT - 1) / F_SLOT : 0;
    ring.issued = 0; ring.ready = 0; ring.dead = false;

    if (k == 0 && !shadow)
        for (uint32_t j = 0; j < NSL; j++) mbar_init(&ring.bars[j], 1);
    mbar_fence_init();
    if (CRC && fits) {
        // slice-by-4 tables, eight copies in the bank-quartered layout of CrcQuarters; then
        // "advance by one row minus one lane unit"
        uint32_t *ts = reinterpret_cast<uint32_t *>(gen(tab0)), *ta = reinterpret_cast<uint32_t *>(gen(adv0));
        // (crc_feed4q sends byte m of a state through table 3 - m, crc_word's order; the
        // row multiplication is in crc_apply's order, byte m through table m)
        for (uint32_t i = threadIdx.x; i < 1024u << F_LOGS; i += WARPS * 32)
            ts[i] = ROWMUL ? a.tabs->mul_row[3u - ((i >> 3) & 3u)][i >> 5] : a.tabs->slice[(i >> 3) & 3u][i >> 5];
        const uint32_t *row_adv = SINK == SINK_F32 ? &a.tabs->adv_row4[0][0] : &a.tabs->adv_row[0][0];
        if (!ROWMUL)
            for (uint32_t i = threadIdx.x; i < 1024u; i += WARPS * 32) ta[i] = row_adv[i];
    }
    __syncthreads();

    if (SHARED) {
        // one table for the CTA, built by its first warp; a table that does not validate
        // fails every stream of the CTA
        uint32_t *poison = reinterpret_cast<uint32_t *>(gen(cf_0));
        if (warp == 0) {
            // one table for the launch, or the one this CTA's chunks name (a shared-table archive)
            const uint8_t *h = (a.tables && a.jobs) ? a.tables + (size_t)a.jobs[blockIdx.x * per_cta].flags * F_TABLE_STRIDE : a.shared_hdr;
            Tables tb{};
            tb.wide = reinterpret_cast<uint32_t *>(gen(l1_0));
            bool ok = fits && build_table<T_WIDE1>(
                [&](uint32_t s) { return (uint32_t)h[4 + 2 * s] | ((uint32_t)h[5 + 2 * s] << 8); }, tb, lane);
            if (lane == 0) *poison = (ok && h[0] == 'R' && h[1] == '1') ? 0u : 1u;
        }
        __syncthreads();
        if (*poison && n) { st = ST_BAD_HEADER; n = 0; }
        // the ring starts cold: slots 0..3 are requested the ordinary way
        ring.valid_slots = n ? ring.valid_slots : 0;
        __syncwarp();
        if (n) {
            ring.issue(0, k == 0);
            ring.require(skew + LEAD);
        }
    }
    // The stream's first 576 bytes or more (table + states, wherever the 16-byte
    // boundary falls) land linearly from the ring's start: four copies, one on each of
    // the first four slot barriers, which have then completed one phase -- as if ring
    // slots 0..3 had been filled and consumed -- when normal ring operation takes over.
    if (!SHARED && k == 0 && n && !shadow) {
        for (uint32_t j = 0; j < 4; j++) {
            mbar_expect_tx(&ring.bars[j], HS);
            bulk_g2s_sa(ring.sa + HS * j, ring.abase + HS * j, HS, smem_addr(&ring.bars[j]));
        }
    }
    __syncwarp();
    if (!SHARED) {
        if (n)
            for (uint32_t j = 0; j < 4; j++)
                if (!ring.dead && !mbar_wait(&ring.bars[j], 0)) ring.dead = true;
        // the bytes of ring slots 0..3 are in place and their barriers are one phase on; a
        // deeper ring's other slots and barriers are untouched
        ring.issued = ring.ready = 4;
    }

    // ---- per-stream tables, built by the whole warp one stream at a time ------------
#pragma unroll 1
    for (uint32_t gg = 0; !SHARED && gg < 4; gg++) {
        uint32_t on = __shfl_sync(0xffffffffu, n, gg * 8);
        if (!on || (DIRECT && warp * 4 + gg >= G)) continue;
        uint32_t sk = __shfl_sync(0xffffffffu, skew, gg * 8);
        const uint32_t rsa = ring_of(warp * 4 + gg);
        auto rd = [&](uint32_t o) { return lds_u8(rsa + o); };     // header sits in the first 548+15 bytes
        Tables tb{};
        auto freq_of = [&](uint32_t s) { return rd(sk + 4 + 2 * s) | (rd(sk + 5 + 2 * s) << 8); };
        uint32_t nlive = 0, max_live = MAX_LIVE;
        bool ok;
        if (WIDE) {
            tb.wide = reinterpret_cast<uint32_t *>(gen(l1_0 + (warp * 4 + gg) * F_WIDE_BYTES));
            ok = build_table<T_WIDE1>(freq_of, tb, lane);
        } else {
            tb.l1 = reinterpret_cast<uint32_t *>(gen(l1_of(warp) + gg * 4));
            tb.cf = reinterpret_cast<uint32_t *>(gen(cf_of(warp * 4 + gg)));
            max_live = HYB ? ((gg & 1u) ? 256u : F_SMALL_LIVE) : MAX_LIVE;
            ok = build_table<T_COMPACT, 4>(freq_of, tb, lane, (HYB ? !(gg & 1u) : CFN < 256) ? 8u * gg : 0u, &nlive, max_live);
        }
        ok = ok && rd(sk) == 'R' && rd(sk + 1) == '1';
        // an alphabet too large for this instance is the caller's mistake, not the stream's
        if (!ok && gi == warp * 4 + gg) { st = nlive > max_live ? ST_BAD_SHAPE : ST_BAD_HEADER; n = 0; }
    }
    __syncwarp();
    if (SINK == SINK_DELTA) {
        // The two groups of a chunk walk its tiles together (they share the merge, and the
        // checksum is folded over both with shuffles): when one plane has been refused, the
        // other is not decoded either.  The refused plane's status reports the chunk.
        const uint32_t partner_n = __shfl_xor_sync(0xffffffffu, n, 8);
        if (partner_n == 0) n = 0;
    }

    const uint32_t xo = ring.sa + skew + (SHARED ? 0u : HDR_BYTES) + 4 * k;
    uint32_t x = lds_u8(xo) | (lds_u8(xo + 1) << 8) | (lds_u8(xo + 2) << 16) | (lds_u8(xo + 3) << 24);
    uint32_t cursor = skew + LEAD;
    uint8_t *out = a.dst + doff;
    const uint32_t al = (uint32_t)(reinterpret_cast<uintptr_t>(out) & 15u);

    // SINK_BF16: the stored plane, read as aligned words and funnel-shifted.
    // SINK_DELTA: the base bytes in the output space, likewise; a tile of a chunk is 256 bytes
    // of output, of which lane k of the chunk's first group takes the 16 from 16 k and lane k
    // of its second group the 16 from 128 + 16 k.
    const uint32_t j16 = 8u * (g & 1u) + k;
    const uint8_t *mant = SINK == SINK_DELTA ? a.dst + moff + 16 * j16 : a.src + moff + 16 * k;
    const uint32_t msh = (uint32_t)(reinterpret_cast<uintptr_t>(mant) & 3u) * 8u;
    const uint32_t *mq = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(mant) & ~uintptr_t(3));
    uint32_t m[5] = {0, 0, 0, 0, 0};
    const uint32_t my_tiles = (n + TS - 1) / TS;
    const bool has_base = SINK == SINK_DELTA && moff != NONE64;      // (a plain two-plane chunk has none: m stays zero)
    if ((SINK == SINK_BF16 && my_tiles) || (has_base && n > 8 * j16)) {
#pragma unroll
        for (int i = 0; i < 5; i++) m[i] = __ldg(mq + i);
    }
    // SINK_BF16 checksum: the eight running values ra[] are multiplied by x^2048 while the
    // NEXT tile decodes (32 independent table lookups that hide behind the decode chain),
    // then that tile's words are XORed in.  SINK_F32 keeps one value, `acc`.
    uint32_t acc = 0, ra[8] = {0, 0, 0, 0, 0, 0, 0, 0};

    // ---- tiles of 128 symbols ---------------------------------------------------------
    const uint32_t warp_tiles = __reduce_max_sync(0xffffffffu, my_tiles);
#pragma unroll 1
    for (uint32_t t = 0; t < warp_tiles; t++) {
        const uint32_t done = t * TS;
        const uint32_t rem = n > done ? n - done : 0;
        __syncwarp();
        if (rem) {
            ring.issue(cursor, k == 0 && !shadow);
            ring.require(cursor + 2 * TS);         // every lane sees the completion itself
        }
        // SINK_F32: the tile's stored bytes are requested before the decode, which hides
        // their latency (lane k: elements 16k .. 16k+15 of each of the three planes)
        uint32_t pr[SINK == SINK_F32 ? 3 : 1][5];
        if (SINK == SINK_F32) {
            const bool mine = rem > 16 * k;
#pragma unroll
            for (int j = 0; j < 3; j++) {
                const uint8_t *pp = a.src + moff + (size_t)j * n + done + 16 * k;
                const uint32_t *pq = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(pp) & ~uintptr_t(3));
#pragma unroll
                for (int i = 0; i < 5; i++) pr[j][i] = mine ? __ldg(pq + i) : 0u;
            }
        }
        const uint32_t caddr0 = ring.sa + ((RINGB & (RINGB - 1)) == 0 ? cursor & (RINGB - 1) : cursor % RINGB);
        uint32_t caddr = caddr0;
        // (lanes that never had a stream run along in full tiles; nothing of theirs is kept)
        const bool full = __all_sync(0xffffffffu, rem >= TS);
        // a decoded symbol goes to the group's staging row, or (DIRECT) straight to its output byte
        uint8_t *const orow = out + done + k;
        auto put = [&](uint32_t step, uint32_t e) {
            if (DIRECT) { if (!shadow) orow[step * NLANES] = (uint8_t)e; }
            else sts_u8(stage_sa + step * NLANES + k, e);
        };
        if (full) {
#pragma unroll
            for (uint32_t s4 = 0; s4 < TS / NLANES; s4 += 4) {
                uint32_t hist = 0, e;
                e = stream_step4<CFN_STEP, true>(x, hist, caddr, l1_sa, cf_sa, below, vsel);
                put(s4, e);
                e = stream_step4<CFN_STEP, false>(x, hist, caddr, l1_sa, cf_sa, below, vsel);
                put(s4 + 1, e);
                if (ROWMUL && (s4 >> 1) < NRA) ra[s4 >> 1] = crc_feed4q(cq, ra[s4 >> 1]);
                e = stream_step4<CFN_STEP, false>(x, hist, caddr, l1_sa, cf_sa, below, vsel);
                put(s4 + 2, e);
                e = stream_step4<CFN_STEP, false>(x, hist, caddr, l1_sa, cf_sa, below, vsel);
                put(s4 + 3, e);
                if (ROWMUL && (s4 >> 1) < NRA) ra[(s4 >> 1) + 1] = crc_feed4q(cq, ra[(s4 >> 1) + 1]);
                caddr += 2 * __popc(hist);
            }
        } else {
            if (ROWMUL) {
#pragma unroll
                for (int i = 0; i < NRA; i++) ra[i] = crc_feed4q(cq, ra[i]);
            }
#pragma unroll 1
            for (uint32_t s = 0; s < TS / NLANES; s++) {
                bool active = s * NLANES + k < rem;
                uint32_t e = stream_step<CFN_STEP>(x, caddr, l1_sa, cf_sa, lt_mask, grp_mask, active);
                if (active) put(s, e);
            }
        }
        cursor += caddr - caddr0;
        __syncwarp();
        if (!rem || DIRECT) continue;
        if (SINK == SINK_DELTA) {
            // ---- both planes' symbols of this lane's eight elements, merge, XOR the base, write, checksum
            const uint32_t pair_sa = stage_0 + (gi & ~1u) * STG + 8u * j16;
            const uint2 ea = lds_u64(pair_sa), eb = lds_u64(pair_sa + STG);
            uint32_t w[4];
            bf16_merge4(ea.x, eb.x, w[0], w[1]);
            bf16_merge4(ea.y, eb.y, w[2], w[3]);
#pragma unroll
            for (int h = 0; h < 4; h++) w[h] ^= __funnelshift_r(m[h], m[h + 1], msh);
            if (has_base && n > (t + 1) * TS + 8u * j16) {         // next tile's base bytes, if this lane has any
#pragma unroll
                for (int i = 0; i < 5; i++) m[i] = __ldg(mq + (size_t)(t + 1) * (2 * TS / 4) + i);
            }
            uint8_t *d = out + (size_t)done * 2 + 16u * j16;
            const uint32_t ve = rem > 8u * j16 ? min(rem - 8u * j16, 8u) : 0u;   // valid elements of this lane
            if (ve == 8) {
                if (al == 0) *reinterpret_cast<uint4 *>(d) = make_uint4(w[0], w[1], w[2], w[3]);
                else if ((al & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
                }
            } else {
                const uint32_t vb = 2 * ve;
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if ((uint32_t)i < vb) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t keep = vb > 4u * i ? min(vb - 4u * i, 4u) : 0u;
                    w[i] = keep >= 4 ? w[i] : (keep ? w[i] & ((1u << (8 * keep)) - 1u) : 0u);
                }
            }
            if (CRC) {
#pragma unroll
                for (int i = 0; i < 4; i++) ra[i] ^= w[i];
                if ((t & 255u) == 255u || t + 1 == my_tiles) {
                    // close the 64 KiB piece: every running value to the row's end, XOR over the chunk's 16 lanes
                    uint32_t v = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        v ^= crc_mulmod(a.tabs->word_mul16[j16][i], ra[i]);
                        ra[i] = 0;
                    }
                    const uint32_t pair_mask = 0xffffu << (16u * (g >> 1));
                    v ^= __shfl_xor_sync(pair_mask, v, 1);
                    v ^= __shfl_xor_sync(pair_mask, v, 2);
                    v ^= __shfl_xor_sync(pair_mask, v, 4);
                    v ^= __shfl_xor_sync(pair_mask, v, 8);
                    if (j16 == 0) {
                        const uint32_t p = t >> 8, rows = (t & 255u) + 1;
                        const uint32_t plen = min(PIECE_BYTES, 2 * n - p * PIECE_BYTES);
                        if (rows * F_ROW != plen) v = crc_unshift(a.tabs->x2, v, rows * F_ROW - plen);
                        a.piece_crc[piece0 + p] = v;
                    }
                }
            }
            continue;
        }
        constexpr uint32_t PER = TS / NLANES;                  // this lane's symbols of the tile: 16 or 32
        uint4 evs[PER / 16];
#pragma unroll
        for (uint32_t q = 0; q < PER / 16; q++) evs[q] = lds_u128(stage_sa + PER * k + 16 * q);
        const uint4 ev = evs[0];

        if (SINK == SINK_BYTES) {
            if (rem >= TS && al == 0) {
#pragma unroll
                for (uint32_t q = 0; q < PER / 16; q++)
                    *reinterpret_cast<uint4 *>(out + done + k * PER + 16 * q) = evs[q];
            } else {
                const uint32_t cnt = rem < TS ? rem : TS;
#pragma unroll
                for (uint32_t q = 0; q < PER / 16; q++) {
                    const uint32_t ew[4] = {evs[q].x, evs[q].y, evs[q].z, evs[q].w};
#pragma unroll
                    for (uint32_t i = 0; i < 16; i++)
                        if (k * PER + 16 * q + i < cnt)
                            out[done + k * PER + 16 * q + i] = (uint8_t)(ew[i >> 2] >> (8 * (i & 3)));
                }
            }
            continue;
        }

        const uint32_t ew[4] = {ev.x, ev.y, ev.z, ev.w};
        if (SINK == SINK_F32) {
            // ---- interleave with the three stored planes, write, checksum ------------
            const uint32_t ve = rem > 16 * k ? min(rem - 16 * k, 16u) : 0u;   // valid elements of this lane
            uint32_t pw[3][4];
#pragma unroll
            for (int j = 0; j < 3; j++) {
                const uint32_t sh = (uint32_t)((reinterpret_cast<uintptr_t>(a.src) + moff + (size_t)j * n + done) & 3u) * 8u;
#pragma unroll
                for (int h = 0; h < 4; h++) pw[j][h] = __funnelshift_r(pr[j][h], pr[j][h + 1], sh);
            }
            uint32_t w[16];
#pragma unroll
            for (int h = 0; h < 4; h++) {
                const uint32_t u0 = __byte_perm(pw[0][h], pw[1][h], 0x5140), u1 = __byte_perm(pw[0][h], pw[1][h], 0x7362);
                const uint32_t v0 = __byte_perm(pw[2][h], ew[h], 0x5140), v1 = __byte_perm(pw[2][h], ew[h], 0x7362);
                w[4 * h + 0] = __byte_perm(u0, v0, 0x5410); w[4 * h + 1] = __byte_perm(u0, v0, 0x7632);
                w[4 * h + 2] = __byte_perm(u1, v1, 0x5410); w[4 * h + 3] = __byte_perm(u1, v1, 0x7632);
            }
            uint8_t *d = out + (size_t)done * 4 + k * 64;
            if (ve == 16) {
                if (al == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        reinterpret_cast<uint4 *>(d)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                } else if ((al & 7) == 0) {
#pragma unroll
                    for (int i = 0; i < 8; i++) reinterpret_cast<uint2 *>(d)[i] = make_uint2(w[2 * i], w[2 * i + 1]);
                } else if ((al & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 16; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 64; i++) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
                }
            } else {
                // whole elements only: a word is either kept or zero
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    if ((uint32_t)i < ve) {
                        if ((al & 3) == 0) reinterpret_cast<uint32_t *>(d)[i] = w[i];
                        else
                            for (int b = 0; b < 4; b++) d[4 * i + b] = (uint8_t)(w[i] >> (8 * b));
                    } else {
                        w[i] = 0u;
                    }
                }
            }
            if (CRC) {
                acc = crc_advance<0>(tla, acc);
#pragma unroll
                for (int i = 0; i < 16; i++) acc = crc_feed4q(cq, acc ^ w[i]);
                if ((t & 127u) == 127u || t + 1 == my_tiles) {
                    // close the 64 KiB piece: lane units -> row end, XOR over the group
                    uint32_t v = crc_mulmod(a.tabs->lane_mul8_4[k], acc);
                    v ^= __shfl_xor_sync(grp_mask, v, 1);
                    v ^= __shfl_xor_sync(grp_mask, v, 2);
                    v ^= __shfl_xor_sync(grp_mask, v, 4);
                    if (k == 0) {
                        const uint32_t p = t >> 7, rows = (t & 127u) + 1;
                        const uint32_t plen = min(PIECE_BYTES, 4 * n - p * PIECE_BYTES);
                        if (rows * 512u != plen) v = crc_unshift(a.tabs->x2, v, rows * 512u - plen);
                        a.piece_crc[piece0 + p] = v;
                    }
                    acc = 0;
                }
            }
            continue;
        }

        // ---- SINK_BF16: merge with the stored plane, write, checksum ------------------
        uint32_t w[8];
#pragma unroll
        for (int h = 0; h < 4; h++)
            bf16_merge4(ew[h], __funnelshift_r(m[h], m[h + 1], msh), w[2 * h], w[2 * h + 1]);
        if (t + 1 < my_tiles) {                                // next tile's stored bytes
#pragma unroll
            for (int i = 0; i < 5; i++) m[i] = __ldg(mq + (size_t)(t + 1) * (TILE / 4) + i);
        }
        uint8_t *d = out + (size_t)done * 2 + k * F_UNIT;
        const uint32_t ve = rem > 16 * k ? min(rem - 16 * k, 16u) : 0u;   // valid elements of this lane
        if (ve == 16) {
            if (al == 0) {
                reinterpret_cast<uint4 *>(d)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4 *>(d)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else if ((al & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) reinterpret_cast<uint2 *>(d)[i] = make_uint2(w[2 * i], w[2 * i + 1]);
            } else if ((al & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 8; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
            }
        } else {
            const uint32_t vb = 2 * ve;
#pragma unroll
            for (int i = 0; i < 32; i++)
                if ((uint32_t)i < vb) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t keep = vb > 4u * i ? min(vb - 4u * i, 4u) : 0u;
                w[i] = keep >= 4 ? w[i] : (keep ? w[i] & ((1u << (8 * keep)) - 1u) : 0u);
            }
        }
        if (CRC) {
#pragma unroll
            for (int i = 0; i < 8; i++) ra[i] ^= w[i];
            if ((t & 255u) == 255u || t + 1 == my_tiles) {
                // close the 64 KiB piece: every running value to the row's end, XOR over the group
                uint32_t v = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    v ^= crc_mulmod(a.tabs->word_mul[k][i], ra[i]);
                    ra[i] = 0;
                }
                v ^= __shfl_xor_sync(grp_mask, v, 1);
                v ^= __shfl_xor_sync(grp_mask, v, 2);
                v ^= __shfl_xor_sync(grp_mask, v, 4);
                if (k == 0) {
                    const uint32_t p = t >> 8, rows = (t & 255u) + 1;
                    const uint32_t plen = min(PIECE_BYTES, 2 * n - p * PIECE_BYTES);
                    if (rows * F_ROW != plen) v = crc_unshift(a.tabs->x2, v, rows * F_ROW - plen);
                    a.piece_crc[piece0 + p] = v;
                }
            }
        }
    }

    // ---- verdict -----------------------------------------------------------------------
    const uint32_t all_rest = __ballot_sync(0xffffffffu, x == RANS_LOW) & grp_mask;
    if (have && k == 0 && !shadow) {
        if (st == ST_OK && n) {
            const uint32_t used = cursor - skew;
            if (ring.dead) st = ST_TIMEOUT;
            else if (used > slen) st = ST_OVERRUN;
            else if (used != slen || all_rest != grp_mask) st = ST_SLACK;
        }
        if (a.status) a.status[job] = st;
        if (a.any_bad && st != ST_OK && st != ST_SLACK) atomicOr(a.any_bad, 1u);
    }
}

// Sort a launch's streams by alphabet size, on the device: one warp per stream counts the
// non-zero frequencies of its table; streams with at most `small_live` go to the front of
// `order` (counts[0] of them), the others to its back (counts[1]).
__global__ void k_classify(StreamArgs a, uint32_t small_live, uint32_t *order, uint32_t *counts)
{
    const uint32_t job = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (job >= a.njobs) return;
    // (delta jobs: njobs counts chunks here, and the first plane's alphabet decides: the instance for
    // small ones gives the second plane a full-size table)
    uint32_t live = 0;
    for (uint32_t plane = 0; plane < 1u; plane++) {
        uint64_t soff;
        uint32_t slen;
        if (a.djobs) { soff = plane ? a.djobs[job].src_b : a.djobs[job].src_a; slen = plane ? a.djobs[job].len_b : a.djobs[job].len_a; }
        else if (a.jobs) { soff = a.jobs[job].src_off; slen = a.jobs[job].src_len; }
        else if (a.sjobs) { soff = a.sjobs[job].src_off; slen = a.sjobs[job].src_len; }
        else { soff = a.offs[2 * job]; slen = (uint32_t)a.offs[2 * job + 1]; }
        uint32_t mine = 0;
        if (slen >= HDR_BYTES + STATE_BYTES) {
            // this lane's eight frequencies: 16 bytes at any alignment, as aligned words
            uint32_t w[4];
            load_words_nc<4>(a.src + soff + 4 + 16 * lane, w);
#pragma unroll
            for (int i = 0; i < 4; i++) mine += ((w[i] & 0xffffu) != 0) + ((w[i] >> 16) != 0);
            mine = __reduce_add_sync(0xffffffffu, mine);
        } else {
            mine = 257;                                // too short: the large instance reports it
        }
        live = max(live, mine);
    }
    if (lane == 0) {
        const bool small = live <= small_live;
        const uint32_t pos = atomicAdd(&counts[small ? 0 : 1], 1u);
        order[small ? pos : a.njobs - 1 - pos] = job;
    }
}

}  // namespace lmz
