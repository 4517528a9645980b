// Whole-chunk kernels: everything between "planes are decoded" and "the chunk's
// plaintext sits at its destination, checksummed".
//
//   k_finish      merge planes (BF16 field merge, byte-plane interleave, copy), XOR
//                 with a delta base, CRC-32 of the result; output written once,
//                 16 bytes a thread (conditioned chunks: k_cond_finish)
//   k_cond_hist   256-bin histogram of a decoded exponent plane
//   k_cond_plan   bucket map + bucket sizes from that histogram; sizes the
//                 sign/mantissa segment decodes
//   k_cond_count  per-piece bucket populations (ranks for the un-partition)
//   k_crc_check   combine piece checksums per chunk and compare with the record
//
// Reference behaviour: lmz/codec.py:1149-1230 (decode_chunk), :1075-1146
// (_decode_bf16c), :1045-1057 (decode_delta); lmz/native/lmzcore.c:439-447
// (BF16 merge), :289-347 (plane interleave), :525-543 (bucket map), :614-641
// (un-partition), :233-245 (xor).
#pragma once
#include "common.cuh"
#include "crc.cuh"
#include <type_traits>

namespace lmz {

constexpr uint64_t NONE64 = ~0ull;
constexpr uint32_t PIECE_ELEMS = PIECE_BYTES / 2;   // BF16 elements per piece
constexpr uint32_t COND_BUCKETS = 8;

enum : uint8_t { K_COPY = 0, K_BF16 = 1, K_SPLIT = 2, K_COND = 3 };

struct ChunkJob {
    uint64_t dst_off;        // chunk start in the output
    uint64_t base_off;       // delta source in the output, or NONE64
    uint64_t plane_off[8];   // plane k: payload offset, or scratch offset when bit k of scratch_mask
    uint32_t rlen;
    uint32_t crc;            // expected crc32, 0 = not recorded
    uint32_t piece0;         // first piece id of this chunk
    uint32_t aux;            // K_COND: index of its CondJob
    uint8_t kind, esize, scratch_mask, src_is_out;   // src_is_out: K_COPY reads the output (a ref)
    uint32_t record;         // archive record this chunk came from
};
static_assert(sizeof(ChunkJob) == 104, "ChunkJob layout is shared with the host");

struct CondJob {
    uint64_t exp_off;        // exponent plane: scratch offset, or payload offset when stored
    uint64_t seg_src[8];     // coded segment b in the payload
    uint64_t seg_scratch;    // where decoded rANS segments go (scratch)
    uint32_t seg_len[8];
    uint32_t nelem;
    uint32_t seg_job0;       // first of the chunk's 8 StreamJob slots
    uint32_t piece0;
    uint32_t chunk;
    uint8_t seg_method[8];
    uint8_t exp_in_scratch;
    uint8_t pad_[7];
};
static_assert(sizeof(CondJob) == 144, "CondJob layout is shared with the host");

struct CondState {           // written on the device
    uint64_t seg_ptr[8];     // plain bytes of segment b (payload or scratch offset)
    uint32_t counts[8];
    uint8_t lut[256];
    uint32_t seg_in_scratch;
    uint32_t status;
};
static_assert(sizeof(CondState) == 360, "CondState layout");

// ---- unaligned loads ---------------------------------------------------------
// N little-endian words starting at any byte address, from aligned 32-bit loads.
// Reads up to 3 bytes before and 4 after the range; buffers carry that slack.
template <int N>
__device__ __forceinline__ void load_words(const uint8_t *p, uint32_t (&w)[N])
{
    uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
    uint32_t sh = (uint32_t)(a & 3u) * 8u;
    uint32_t v[N + 1];
#pragma unroll
    for (int i = 0; i <= N; i++) v[i] = q[i];
#pragma unroll
    for (int i = 0; i < N; i++) w[i] = __funnelshift_r(v[i], v[i + 1], sh);
}

// The same through the read-only path, for data no thread of the kernel writes.
template <int N>
__device__ __forceinline__ void load_words_nc(const uint8_t *p, uint32_t (&w)[N])
{
    uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
    uint32_t sh = (uint32_t)(a & 3u) * 8u;
    uint32_t v[N + 1];
#pragma unroll
    for (int i = 0; i <= N; i++) v[i] = __ldg(q + i);
#pragma unroll
    for (int i = 0; i < N; i++) w[i] = __funnelshift_r(v[i], v[i + 1], sh);
}

__device__ __forceinline__ uint32_t smem_word(const uint8_t *base, uint32_t byte_index)
{
    return *reinterpret_cast<const uint32_t *>(base + byte_index);
}

// BF16 field merge of four elements at once (lmz/native/lmzcore.c:439-447): the low
// byte of an element is b's bits 0-6 under a's bit 0, the high byte b's sign over
// a >> 1; both are byte-wise selects on the packed words, then the bytes interleave.
__device__ __forceinline__ void bf16_merge4(uint32_t a4, uint32_t b4, uint32_t &w0, uint32_t &w1)
{
    const uint32_t lo4 = (b4 & 0x7f7f7f7fu) | ((a4 << 7) & 0x80808080u);
    const uint32_t hi4 = (b4 & 0x80808080u) | ((a4 >> 1) & 0x7f7f7f7fu);
    w0 = __byte_perm(lo4, hi4, 0x5140);
    w1 = __byte_perm(lo4, hi4, 0x7362);
}

__device__ __forceinline__ void bf16_merge8(const uint32_t (&a)[2], const uint32_t (&b)[2],
                                            uint32_t (&w)[4])
{
#pragma unroll
    for (int h = 0; h < 2; h++) bf16_merge4(a[h], b[h], w[2 * h], w[2 * h + 1]);
}

// Padded shared-memory layout for per-thread runs of 128 bytes: 4 bytes of
// padding per 128 keep a warp's accesses on distinct banks.
__device__ __forceinline__ uint32_t pad128(uint32_t i) { return i + ((i >> 7) << 2); }
constexpr uint32_t PADDED_PIECE = PIECE_ELEMS + (PIECE_ELEMS >> 7) * 4;

// CRC tables in the bank-quartered layout (k_stream, k_cond_finish), laid out so that the warp's 32 lookups of one load never
// share a bank: entry i of table j, copy r sits at word 32 i + 8 j + r -- a table owns a
// quarter of the banks and each of its eight copies one bank of that quarter.  Lane k of
// group g uses copy k, and the groups take the four bytes of a state word in rotated order
// (group g starts at byte g), so in each of the four loads the groups are in four different
// tables, i.e. bank quarters.  b[i] = table base + this lane's word for load i; rot = 8 g.
struct CrcQuarters {
    uint32_t b[4], rot;
};
__device__ __forceinline__ uint32_t crc_feed4q(const CrcQuarters &q, uint32_t s)
{
    const uint32_t r = __funnelshift_r(s, s, q.rot);     // byte i of r = byte (i + g) & 3 of s
    return lds_u32(((r << 7) & 0x7f80u) | q.b[0]) ^ lds_u32(((r >> 1) & 0x7f80u) | q.b[1]) ^
           lds_u32(((r >> 9) & 0x7f80u) | q.b[2]) ^ lds_u32(((r >> 17) & 0x7f80u) | q.b[3]);
}

struct FinishArgs {
    const ChunkJob *chunks;
    const uint32_t *piece_chunk;   // piece id -> chunk index
    uint32_t piece_begin, piece_end;
    const uint8_t *payload;
    const uint8_t *scratch;
    uint8_t *out;
    uint32_t *piece_crc;           // R() of each piece, or NULL to skip checksums
    const CrcTables *tabs;
    const CondJob *cond_jobs;
    const CondState *cond_state;
    const uint32_t *piece_cnt;     // per piece of a K_COND chunk: 8 bucket populations, 8 running totals
    const uint16_t *piece_wcnt;    // per piece of a K_COND chunk: the populations of its eight 4096-element runs
    const uint32_t *piece_lcnt;    // per conditioned piece, in the order of the conditioned-piece list: the
                                   // populations of every lane's 32 elements (k_cond_count, k_cond_finish)
    uint32_t lcnt_first;           // place of piece_begin in that list
};

constexpr uint32_t FINISH_THREADS = 256;   // threads that finish one piece together

// Shared memory of k_finish: the "multiply by x^(8 * 4096)" tables (one 4 KiB row of a piece
// further on) in the bank-quartered layout of CrcQuarters, 32 KiB on a 32 KiB boundary of
// the shared window; then, per 256-thread sub-block, 2 KiB of reduction scratch.
constexpr uint32_t FINISH_TABLE_BYTES = 32768;
__host__ __device__ constexpr uint32_t finish_sub_bytes() { return 2048; }
__host__ __device__ constexpr uint32_t finish_smem(int subs)
{
    return 2 * FINISH_TABLE_BYTES /*the tables, wherever their boundary falls*/ + subs * finish_sub_bytes();
}

// Replicated-table CRC steps.  `tl` = shared address of this lane's copy of table 0;
// table j lives j table-sizes further on.
// Byte `b` of s (0 = least significant) as a table offset, OR-ed onto the lane's base.
template <int LOGR, int B>
__device__ __forceinline__ uint32_t crc_index(uint32_t tl, uint32_t s)
{
    constexpr int SH = 2 + LOGR;
    constexpr uint32_t MASK = 0xffu << SH;
    constexpr int RIGHT = 8 * B - SH;          // shift that moves byte B's bits to SH..SH+7
    uint32_t v;
    if constexpr (RIGHT >= 0) v = s >> RIGHT;
    else v = s << (-RIGHT);
    return (v & MASK) | tl;
}

// One slice-by-4 step over the replicated tables: the state after feeding the four
// bytes already XOR-ed into s (tables 0..3 = CrcTables::slice).
template <int LOGR>
__device__ __forceinline__ uint32_t crc_feed4(uint32_t tl, uint32_t s)
{
    constexpr uint32_t TS = 1024u << LOGR;
    return lds_u32(crc_index<LOGR, 0>(tl, s) + 3 * TS) ^ lds_u32(crc_index<LOGR, 1>(tl, s) + 2 * TS) ^
           lds_u32(crc_index<LOGR, 2>(tl, s) + 1 * TS) ^ lds_u32(crc_index<LOGR, 3>(tl, s));
}

// The state advanced by a row minus 16 bytes of zeros (tables 4..7 = CrcTables::adv).
template <int LOGR>
__device__ __forceinline__ uint32_t crc_advance(uint32_t tl, uint32_t s)
{
    constexpr uint32_t TS = 1024u << LOGR;
    return lds_u32(crc_index<LOGR, 0>(tl, s) + 4 * TS) ^ lds_u32(crc_index<LOGR, 1>(tl, s) + 5 * TS) ^
           lds_u32(crc_index<LOGR, 2>(tl, s) + 6 * TS) ^ lds_u32(crc_index<LOGR, 3>(tl, s) + 7 * TS);
}

// SUBS = 256-thread sub-blocks per CTA sharing one table set.  Exponent-conditioned chunks
// go to k_cond_finish instead.
//
// Checksum: a thread writes the same 16 bytes of every 4 KiB row of a piece.  It keeps one
// running value per word of them, ra[i] = sum over the rows so far of word i * x^(32768 *
// rows since): a row costs each of the four one multiplication by x^32768 -- four table
// lookups with no chain between the four values and no separate advance step -- and at the
// piece's end the four are joined as if they were a 16-byte message of their own.
template <int SUBS>
__global__ void __launch_bounds__(FINISH_THREADS * SUBS) k_finish(FinishArgs a)
{
    extern __shared__ __align__(16) uint8_t fsm[];
    const uint32_t sub = threadIdx.x / FINISH_THREADS, t = threadIdx.x % FINISH_THREADS;
    const uint32_t lane = t & 31, warp = t >> 5;
    const uint32_t tab0 = (smem_addr(fsm) + FINISH_TABLE_BYTES - 1) & ~(FINISH_TABLE_BYTES - 1);
    uint8_t *after = fsm + (tab0 - smem_addr(fsm)) + FINISH_TABLE_BYTES;
    uint8_t *sb = after + sub * finish_sub_bytes();
    uint32_t *s_red = reinterpret_cast<uint32_t *>(sb);               // 512 words of scratch
    const bool do_crc = a.piece_crc != nullptr;
    // byte m of a running value goes through table m, which crc_feed4q looks for in slot 3 - m
    CrcQuarters cq;
    {
        const uint32_t k = lane & 7u, g = lane >> 3;
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) cq.b[i] = tab0 + 32u * (3u - ((i + g) & 3u)) + 4u * k;
        cq.rot = 8u * g;
    }
    auto sub_sync = [&]() {
        if (SUBS == 1) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(sub + 1), "n"(FINISH_THREADS) : "memory");
    };
    // one row into the running values
    auto crc_row = [&](uint32_t (&ra)[4], const uint32_t (&w)[4]) {
#pragma unroll
        for (int i = 0; i < 4; i++) ra[i] = crc_feed4q(cq, ra[i]) ^ w[i];
    };

    if (do_crc) {
        uint32_t *tw = reinterpret_cast<uint32_t *>(fsm + (tab0 - smem_addr(fsm)));
        for (uint32_t i = threadIdx.x; i < FINISH_TABLE_BYTES / 4; i += FINISH_THREADS * SUBS)
            tw[i] = a.tabs->mul_row4096[3u - ((i >> 3) & 3u)][i >> 5];
    }
    __syncthreads();

    for (uint32_t q = a.piece_begin + blockIdx.x * SUBS + sub; q < a.piece_end;
         q += gridDim.x * SUBS) {
        const ChunkJob &c = a.chunks[a.piece_chunk[q]];
        const uint32_t pbase = (q - c.piece0) * PIECE_BYTES;          // chunk-relative
        const uint32_t plen = min(PIECE_BYTES, c.rlen - pbase);
        const uint8_t kind = c.kind, esize = c.esize;
        uint8_t *dst = a.out + c.dst_off + pbase;
        const uint8_t *base = c.base_off == NONE64 ? nullptr : a.out + c.base_off + pbase;
        const uint32_t al = (uint32_t)(reinterpret_cast<uintptr_t>(a.out + c.dst_off) & 15u);

        const uint8_t *pl[8];
#pragma unroll
        for (int k = 0; k < 8; k++)
            pl[k] = (c.scratch_mask >> k & 1 ? a.scratch : a.payload) + c.plane_off[k];
        if (kind == K_COPY && c.src_is_out) pl[0] = a.out + c.plane_off[0];

        // ---- rows: every thread produces 16 output bytes per row ----------------
        uint32_t ra[4] = {0, 0, 0, 0};
        // Fast path for the overwhelmingly common piece: full, 16-byte aligned, no delta
        // base, copy or BF16 merge.  No per-row dispatch, loads on the read-only path and
        // four rows unrolled so the loads of later rows overlap the CRC chain of earlier ones.
        const bool fast = plen == PIECE_BYTES && al == 0 && base == nullptr &&
                          (kind == K_COPY || kind == K_BF16) && !(kind == K_COPY && c.src_is_out);
        if (fast) {
            auto rows = [&](auto kind_c) {
                constexpr int KIND = decltype(kind_c)::value;
#pragma unroll 4
                for (uint32_t row = 0; row < PIECE_BYTES / ROW_BYTES; row++) {
                    const uint32_t r = row * ROW_BYTES + t * 16;
                    uint32_t w[4];
                    if (KIND == K_COPY) {
                        load_words_nc<4>(pl[0] + pbase + r, w);
                    } else {
                        uint32_t pa[2], pb[2];
                        load_words_nc<2>(pl[0] + (pbase + r) / 2, pa);
                        load_words_nc<2>(pl[1] + (pbase + r) / 2, pb);
                        bf16_merge8(pa, pb, w);
                    }
                    *reinterpret_cast<uint4 *>(dst + r) = make_uint4(w[0], w[1], w[2], w[3]);
                    if (do_crc) crc_row(ra, w);
                }
            };
            if (kind == K_COPY) rows(std::integral_constant<int, K_COPY>{});
            else rows(std::integral_constant<int, K_BF16>{});
        }
#pragma unroll 1
        for (uint32_t row = 0; !fast && row < PIECE_BYTES / ROW_BYTES; row++) {
            const uint32_t r = row * ROW_BYTES + t * 16;    // piece-relative
            uint32_t w[4] = {0, 0, 0, 0};
            if (r < plen) {
                const uint32_t cr = pbase + r;              // chunk-relative
                if (kind == K_COPY) {
                    load_words<4>(pl[0] + cr, w);
                } else if (kind == K_BF16) {
                    uint32_t pa[2], pb[2];
                    load_words<2>(pl[0] + cr / 2, pa);
                    load_words<2>(pl[1] + cr / 2, pb);
                    bf16_merge8(pa, pb, w);
                } else if (esize == 4) {
                    uint32_t p0[1], p1[1], p2[1], p3[1];
                    load_words<1>(pl[0] + cr / 4, p0);
                    load_words<1>(pl[1] + cr / 4, p1);
                    load_words<1>(pl[2] + cr / 4, p2);
                    load_words<1>(pl[3] + cr / 4, p3);
                    uint32_t t0 = __byte_perm(p0[0], p1[0], 0x5140), t1 = __byte_perm(p2[0], p3[0], 0x5140);
                    uint32_t t2 = __byte_perm(p0[0], p1[0], 0x7362), t3 = __byte_perm(p2[0], p3[0], 0x7362);
                    w[0] = __byte_perm(t0, t1, 0x5410); w[1] = __byte_perm(t0, t1, 0x7632);
                    w[2] = __byte_perm(t2, t3, 0x5410); w[3] = __byte_perm(t2, t3, 0x7632);
                } else if (esize == 2) {
                    uint32_t p0[2], p1[2];
                    load_words<2>(pl[0] + cr / 2, p0);
                    load_words<2>(pl[1] + cr / 2, p1);
                    w[0] = __byte_perm(p0[0], p1[0], 0x5140); w[1] = __byte_perm(p0[0], p1[0], 0x7362);
                    w[2] = __byte_perm(p0[1], p1[1], 0x5140); w[3] = __byte_perm(p0[1], p1[1], 0x7362);
                } else {   // esize 8: two elements, one byte from each of eight planes
                    uint32_t e = cr / 8;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        uint32_t b0 = pl[k][e], b1 = pl[k][e + 1];
                        w[k >> 2] |= b0 << (8 * (k & 3));
                        w[2 + (k >> 2)] |= b1 << (8 * (k & 3));
                    }
                }
                if (base) {
                    uint32_t bw[4];
                    load_words<4>(base + r, bw);
#pragma unroll
                    for (int i = 0; i < 4; i++) w[i] ^= bw[i];
                }
                const uint32_t left = plen - r;
                if (left >= 16) {
                    uint8_t *d = dst + r;
                    if (al == 0) *reinterpret_cast<uint4 *>(d) = make_uint4(w[0], w[1], w[2], w[3]);
                    else if ((al & 7) == 0) {
                        reinterpret_cast<uint2 *>(d)[0] = make_uint2(w[0], w[1]);
                        reinterpret_cast<uint2 *>(d)[1] = make_uint2(w[2], w[3]);
                    } else if ((al & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if ((uint32_t)i < left) dst[r + i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t keep = left > 4u * i ? min(left - 4u * i, 4u) : 0u;
                        w[i] = keep >= 4 ? w[i] : (keep ? w[i] & ((1u << (8 * keep)) - 1u) : 0u);
                    }
                }
            }
            if (do_crc) crc_row(ra, w);
        }
        if (do_crc) {
            // the four running values as one 16-byte message (tables in global memory: once per piece)
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) acc = crc_word(a.tabs->slice, acc, ra[i]);
            uint32_t v = crc_mulmod(a.tabs->lane_mul[t], acc);
#pragma unroll
            for (int d = 16; d; d >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, d);
            sub_sync();
            if (lane == 0) s_red[300 + warp] = v;
            sub_sync();
            if (t == 0) {
                uint32_t r = 0;
                for (int i = 0; i < 8; i++) r ^= s_red[300 + i];
                if (plen < PIECE_BYTES) r = crc_unshift(a.tabs->x2, r, PIECE_BYTES - plen);
                a.piece_crc[q] = r;
            }
        }
        sub_sync();
    }
}

}  // namespace lmz
