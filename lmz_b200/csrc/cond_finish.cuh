// k_cond_finish: the last pass of an exponent-conditioned BF16 chunk
// (lmz/codec.py:1144-1146: un-partition, then the BF16 field merge), one 64 KiB piece
// of output per 256 threads, four pieces in flight per CTA.
//
// The stable 8-way un-partition (lmz/native/lmzcore.c:614-641) gives element i the next
// unread byte of its bucket's segment.  Here a warp owns a run of 4096 consecutive elements
// and walks it in four blocks of 1024, lane l holding the 32 consecutive elements
// 32 l .. 32 l + 31 of the block:
//
//   * how many elements of each bucket every lane's 32 hold is known before the kernel
//     starts (k_cond_count wrote it, 8 bytes per lane and block), so ONE warp scan per
//     block tells each lane where its first element of every bucket sits in the piece's
//     share of that bucket's segment, which is staged in shared memory;
//   * the lane keeps those eight read positions in a table of its own in shared memory
//     ([bucket][lane]: its words are all in its own bank); an element is then: its bucket
//     (one 16-bit table lookup by its exponent byte), the bucket's position, the byte
//     there, the position + 1 written back -- no ranks, no one-hot arithmetic;
//   * the lane merges eight exponents and eight bytes to 16 bytes of BF16, XORs the
//     delta base if there is one, stores them and feeds them to a CRC-32 of its own 64
//     contiguous bytes per block (tables in the bank-quartered layout: no conflicts); from
//     one block to the next the lane's value is multiplied by x^(8 * 1984), the bytes of
//     other lanes in between, through a second small table.
//
// What a warp needs to know before it starts -- where its run begins in each segment --
// comes from k_cond_count (populations of every 4096-element run) and k_cond_scan
// (where the piece begins).
#pragma once
#include "chunk_kernels.cuh"

namespace lmz {

constexpr uint32_t CF_SUB = 256, CF_SUBS = 4, CF_THREADS = CF_SUB * CF_SUBS;
constexpr uint32_t CF_RUN = PIECE_ELEMS / 8;                  // elements one warp walks
constexpr uint32_t CF_BLOCK = 1024, CF_LANE = CF_BLOCK / 32;  // elements per warp step, per lane of it
constexpr uint32_t CF_BLOCKS = CF_RUN / CF_BLOCK;
constexpr uint32_t CF_LCNT_WORDS = 8 * CF_BLOCKS * 32 * 2;    // piece_lcnt: [warp][block][lane] x {even buckets, odd buckets}
constexpr uint32_t CF_STAGE = PIECE_ELEMS + 8 * 32;           // eight ranges, each copied from its 16-byte boundary
constexpr uint32_t CF_PTR_BYTES = 8 * 8 * 32 * 4;             // read positions: [warp][bucket][lane]
constexpr uint32_t CF_LUT_BYTES = 512;                        // symbol -> 128 * bucket, 16 bits
constexpr uint32_t CF_SUB_BYTES = CF_STAGE + CF_LUT_BYTES + 256 /*misc*/;
constexpr uint32_t CF_TABLE_BYTES = 32768;                    // four tables x 256 entries x eight copies
constexpr uint32_t CF_GAP_BYTES = 4096;                       // four tables x 256 entries, once
// The slice tables must start on a 32 KiB boundary of the shared window, wherever the
// block's own memory starts in it; as many of the four position tables as fit go below
// that boundary, everything else above the tables.  210 KiB covers every case.
__host__ __device__ constexpr uint32_t cond_finish_smem() { return 215040; }

// Per conditioned chunk and bucket: running totals of the piece populations, so a
// piece knows where its share of every segment starts (piece_cnt[q][8 + b]).
__global__ void k_cond_scan(const ChunkJob *chunks, const CondJob *cond_jobs, uint32_t ncond,
                            uint32_t *piece_cnt)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= ncond * 8) return;
    const ChunkJob &c = chunks[cond_jobs[i >> 3].chunk];
    const uint32_t b = i & 7, np = (c.rlen + PIECE_BYTES - 1) / PIECE_BYTES;
    uint32_t run = 0;
    for (uint32_t p = 0; p < np; p++) {
        uint32_t *row = piece_cnt + (size_t)(c.piece0 + p) * 16;
        row[8 + b] = run;
        run += row[b];
    }
}

struct CfShared {
    uint32_t stage_sa, lut_sa, ptr_sa, gap_sa, sub;
    uint32_t *s_misc;
    uint8_t *s_stage;
    CrcQuarters cq;
};

__device__ __forceinline__ void cf_sync(uint32_t sub)
{
    asm volatile("bar.sync %0, %1;" ::"r"(sub + 1), "n"(CF_SUB) : "memory");
}

// One piece.  FULL: the piece has all 32768 elements, so no thread checks a tail.
template <bool FULL>
__device__ __forceinline__ void cf_piece(const FinishArgs &a, const CfShared &sh, uint32_t q,
                                         const ChunkJob &c, const CondJob &cj, const CondState &cs)
{
    const uint32_t t = threadIdx.x % CF_SUB, lane = t & 31, warp = t >> 5;
    const bool do_crc = a.piece_crc != nullptr;
    const uint32_t p = q - c.piece0;
    const uint32_t pbase = p * PIECE_BYTES;
    const uint32_t plen = FULL ? PIECE_BYTES : min(PIECE_BYTES, c.rlen - pbase), ne = plen / 2;
    uint8_t *dst = a.out + c.dst_off + pbase;
    const uint8_t *base = c.base_off == NONE64 ? nullptr : a.out + c.base_off + pbase;
    const uint32_t al = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u);
    const uint8_t *exp = (cj.exp_in_scratch ? a.scratch : a.payload) + cj.exp_off + pbase / 2;
    const bool exp_al16 = (reinterpret_cast<uintptr_t>(exp) & 15u) == 0;
    const uint32_t *cnt_row = a.piece_cnt + (size_t)q * 16;
    const uint16_t *wcnt = a.piece_wcnt + (size_t)q * 64;
    const uint2 *lcnt = reinterpret_cast<const uint2 *>(a.piece_lcnt) +
                        ((size_t)(a.lcnt_first + (q - a.piece_begin)) * 8 + warp) * (CF_BLOCKS * 32) + lane;

    // ---- the piece's range of each segment -> shared memory, whole 16-byte units -------
    // s_misc[b] = offset in the staging buffer of the range's first byte
    if (t < 8) {
        const uint32_t b = t;
        uint32_t pos = 0;
        for (uint32_t j = 0; j < b; j++) pos += (cnt_row[j] + 30u) & ~15u;      // room for any skew, whole units
        const uint8_t *sp = (cs.seg_in_scratch >> b & 1 ? a.scratch : a.payload) + cs.seg_ptr[b] + cnt_row[8 + b];
        sh.s_misc[b] = pos + (uint32_t)(reinterpret_cast<uintptr_t>(sp) & 15u);
    }
    cf_sync(sh.sub);
#pragma unroll 1
    for (int b = 0; b < 8; b++) {
        const uint32_t cnt = cnt_row[b];
        if (!cnt) continue;
        const uint8_t *sp = (cs.seg_in_scratch >> b & 1 ? a.scratch : a.payload) + cs.seg_ptr[b] + cnt_row[8 + b];
        const uint32_t skew = (uint32_t)(reinterpret_cast<uintptr_t>(sp) & 15u);
        const uint4 *s4 = reinterpret_cast<const uint4 *>(sp - skew);
        uint4 *d4 = reinterpret_cast<uint4 *>(sh.s_stage + (sh.s_misc[b] - skew));
        const uint32_t nvec = (skew + cnt + 15u) >> 4;
        for (uint32_t i = t; i < nvec; i += CF_SUB) d4[i] = __ldg(s4 + i);
    }
    // Where this warp's run begins in every range (offset in the staging buffer): the range's
    // start plus the populations of the runs before it.  Kept as four words of 16-bit
    // fields, in the order the lane counts arrive in: buckets (0,4) (2,6) (1,5) (3,7).
    uint32_t W[4];
    {
        uint32_t v = 0;
        if (lane < 8) {
            v = sh.s_misc[lane];
            for (uint32_t w = 0; w < warp; w++) v += wcnt[w * 8 + lane];
        }
        W[0] = __shfl_sync(0xffffffffu, v, 0) | (__shfl_sync(0xffffffffu, v, 4) << 16);
        W[1] = __shfl_sync(0xffffffffu, v, 2) | (__shfl_sync(0xffffffffu, v, 6) << 16);
        W[2] = __shfl_sync(0xffffffffu, v, 1) | (__shfl_sync(0xffffffffu, v, 5) << 16);
        W[3] = __shfl_sync(0xffffffffu, v, 3) | (__shfl_sync(0xffffffffu, v, 7) << 16);
    }
    cf_sync(sh.sub);

    // ---- walk the run: four blocks of 1024 elements, 32 consecutive ones per lane -----------
    const uint32_t my_ptr = sh.ptr_sa + warp * 1024 + lane * 4;        // + 128 * bucket
    uint32_t acc = 0;
    auto fetch = [&](uint32_t j, uint32_t (&e)[8], uint2 &lc) {        // block j: this lane's exponents and counts
        const uint32_t at = warp * CF_RUN + j * CF_BLOCK + lane * CF_LANE;
        lc = __ldg(lcnt + j * 32);
        if (FULL && exp_al16) {
            const uint4 v0 = __ldg(reinterpret_cast<const uint4 *>(exp + at)), v1 = __ldg(reinterpret_cast<const uint4 *>(exp + at) + 1);
            e[0] = v0.x; e[1] = v0.y; e[2] = v0.z; e[3] = v0.w;
            e[4] = v1.x; e[5] = v1.y; e[6] = v1.z; e[7] = v1.w;
        } else {
#pragma unroll
            for (int k = 0; k < 8; k++) {
                uint32_t v[1] = {0};
                if (FULL || at + 4 * k < ne) load_words_nc<1>(exp + at + 4 * k, v);     // (reads at most 3 bytes past ne)
                e[k] = v[0];
            }
        }
    };
    uint32_t nx[8];
    uint2 nlc;
    fetch(0, nx, nlc);
#pragma unroll 1
    for (uint32_t j = 0; j < CF_BLOCKS; j++) {
        uint32_t ex[8];
#pragma unroll
        for (int k = 0; k < 8; k++) ex[k] = nx[k];
        const uint2 lc = nlc;
        if (j + 1 < CF_BLOCKS) fetch(j + 1, nx, nlc);                  // the next block's, under this block's work
        // this lane's first element of every bucket: an exclusive scan of the lanes' counts
        const uint32_t f[4] = {lc.x & 0x00ff00ffu, (lc.x >> 8) & 0x00ff00ffu, lc.y & 0x00ff00ffu, (lc.y >> 8) & 0x00ff00ffu};
        uint32_t inc[4] = {f[0], f[1], f[2], f[3]};
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, inc[i], d);
                if (lane >= (uint32_t)d) inc[i] += v;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t first = W[i] + inc[i] - f[i];               // staging offsets: below 2^16, no carries between fields
            W[i] += __shfl_sync(0xffffffffu, inc[i], 31);
            // word i holds buckets B and B + 4, B = 0, 2, 1, 3
            const uint32_t B = i == 0 ? 0u : i == 1 ? 2u : i == 2 ? 1u : 3u;
            sts_u32(my_ptr + 128u * B, sh.stage_sa + (first & 0xffffu));
            sts_u32(my_ptr + 128u * (B + 4u), sh.stage_sa + (first >> 16));
        }
        if (do_crc && j) {
            // the other lanes' bytes between this lane's blocks: x^(8 * (2048 - 64))
            acc = lds_u32(sh.gap_sa + 4u * (acc & 0xffu)) ^ lds_u32(sh.gap_sa + 1024u + 4u * ((acc >> 8) & 0xffu)) ^
                  lds_u32(sh.gap_sa + 2048u + 4u * ((acc >> 16) & 0xffu)) ^ lds_u32(sh.gap_sa + 3072u + 4u * (acc >> 24));
        }
#pragma unroll
        for (uint32_t it = 0; it < CF_LANE / 8; it++) {
            const uint32_t i0 = warp * CF_RUN + j * CF_BLOCK + lane * CF_LANE + it * 8;   // first of these eight elements
            const uint32_t valid = FULL ? 8u : (ne > i0 ? min(ne - i0, 8u) : 0u);
            const uint32_t e2[2] = {ex[2 * it], ex[2 * it + 1]};
            uint32_t sm[2] = {0, 0};
#pragma unroll
            for (int z = 0; z < 8; z++) {
                if (FULL || (uint32_t)z < valid) {
                    const uint32_t w = e2[z >> 2];
                    const int zz = z & 3;
                    // the bucket table is 512-byte aligned: twice the symbol is OR-ed on
                    const uint32_t ix = zz == 0 ? (w << 1) & 0x1feu : (w >> (8 * zz - 1)) & 0x1feu;
                    const uint32_t pa = my_ptr + lds_u16(ix | sh.lut_sa);
                    const uint32_t at = lds_u32(pa);
                    constexpr uint32_t SEL[4] = {0x3214u, 0x3240u, 0x3410u, 0x4210u};   // the byte into place z & 3
                    sm[z >> 2] = __byte_perm(sm[z >> 2], lds_u8(at), SEL[zz]);
                    sts_u32(pa, at + 1u);
                }
            }
            uint32_t w[4];
            bf16_merge8(e2, sm, w);
            const uint32_t r = 2 * i0;                                      // piece-relative output offset
            if (base) {
                if (valid) {
                    uint32_t bw[4];
                    load_words<4>(base + r, bw);
#pragma unroll
                    for (int i = 0; i < 4; i++) w[i] ^= bw[i];
                }
            }
            if (FULL || valid == 8) {
                uint8_t *d = dst + r;
                if (al == 0) *reinterpret_cast<uint4 *>(d) = make_uint4(w[0], w[1], w[2], w[3]);
                else if ((al & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) d[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
                }
            } else {
                const uint32_t left = 2 * valid;                            // bytes of this lane that exist
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if ((uint32_t)i < left) dst[r + i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t keep = left > 4u * i ? min(left - 4u * i, 4u) : 0u;
                    w[i] = keep >= 4 ? w[i] : (keep ? w[i] & ((1u << (8 * keep)) - 1u) : 0u);
                }
            }
            if (do_crc) {
#pragma unroll
                for (int i = 0; i < 4; i++) acc = crc_feed4q(sh.cq, acc ^ w[i]);
            }
        }
    }
    if (do_crc) {
        // the lane's value to the end of the warp's 8 KiB, XOR over the warp, then to the piece's end
        uint32_t v = crc_mulmod(a.tabs->lane_mul64[lane], acc);
#pragma unroll
        for (int d = 16; d; d >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, d);
        if (lane == 0) sh.s_misc[16 + warp] = crc_mulmod(a.tabs->warp_mul8k[warp], v);
        cf_sync(sh.sub);
        if (t == 0) {
            uint32_t r = 0;
            for (int i = 0; i < 8; i++) r ^= sh.s_misc[16 + i];
            if (plen < PIECE_BYTES) r = crc_unshift(a.tabs->x2, r, PIECE_BYTES - plen);
            a.piece_crc[q] = r;
        }
    }
}

__global__ void __launch_bounds__(CF_THREADS, 1) k_cond_finish(FinishArgs a)
{
    extern __shared__ __align__(16) uint8_t csm[];
    const uint32_t sub = threadIdx.x / CF_SUB, t = threadIdx.x % CF_SUB, lane = t & 31;
    const uint32_t s0 = smem_addr(csm);
    // [s0, tab0): position tables of the first sub-blocks; [tab0, +32 KiB): slice tables;
    // then the gap table, the other position tables, and every sub-block's own part
    const uint32_t tab0 = (s0 + CF_TABLE_BYTES - 1) & ~(CF_TABLE_BYTES - 1);
    const uint32_t below = min(CF_SUBS, (tab0 - ((s0 + 15u) & ~15u)) / CF_PTR_BYTES);
    const uint32_t gap0 = tab0 + CF_TABLE_BYTES;
    const uint32_t own0 = gap0 + CF_GAP_BYTES + (CF_SUBS - below) * CF_PTR_BYTES;
    uint8_t *mine = csm + (own0 - s0) + sub * CF_SUB_BYTES;
    CfShared sh;
    sh.sub = sub;
    sh.ptr_sa = sub < below ? ((s0 + 15u) & ~15u) + sub * CF_PTR_BYTES : gap0 + CF_GAP_BYTES + (sub - below) * CF_PTR_BYTES;
    sh.gap_sa = gap0;
    uint16_t *s_lut = reinterpret_cast<uint16_t *>(mine);                        // 512-byte aligned
    sh.s_misc = reinterpret_cast<uint32_t *>(mine + CF_LUT_BYTES);               // 64 words
    sh.s_stage = mine + CF_LUT_BYTES + 256;
    sh.stage_sa = smem_addr(sh.s_stage); sh.lut_sa = smem_addr(s_lut);
    const bool fits = own0 + CF_SUBS * CF_SUB_BYTES <= s0 + dynamic_smem_bytes() && (sh.lut_sa & 511u) == 0;
    // slice tables in the bank-quartered layout (see CrcQuarters): byte m of a state goes
    // through table 3 - m, which crc_feed4q looks for in slot m
    const uint32_t k = lane & 7u, g = lane >> 3;
#pragma unroll
    for (uint32_t i = 0; i < 4; i++) sh.cq.b[i] = tab0 + 32u * (3u - ((i + g) & 3u)) + 4u * k;
    sh.cq.rot = 8u * g;
    if (a.piece_crc && fits) {
        uint32_t *tw = reinterpret_cast<uint32_t *>(csm + (tab0 - s0));
        for (uint32_t i = threadIdx.x; i < CF_TABLE_BYTES / 4; i += CF_THREADS)
            tw[i] = a.tabs->slice[(i >> 3) & 3u][i >> 5];
        uint32_t *gw = reinterpret_cast<uint32_t *>(csm + (gap0 - s0));
        for (uint32_t i = threadIdx.x; i < CF_GAP_BYTES / 4; i += CF_THREADS) gw[i] = (&a.tabs->mul_gap1984[0][0])[i];
    }
    __syncthreads();
    if (!fits) return;                                     // (the launcher asks for enough: every piece stays unwritten and fails its checksum)
    uint32_t have_lut = 0xffffffffu;
    for (uint32_t q = a.piece_begin + blockIdx.x * CF_SUBS + sub; q < a.piece_end; q += gridDim.x * CF_SUBS) {
        const ChunkJob &c = a.chunks[a.piece_chunk[q]];
        const CondJob &cj = a.cond_jobs[c.aux];
        const CondState &cs = a.cond_state[c.aux];
        cf_sync(sub);                                      // the previous piece is done with shared memory
        // A chunk whose bucket sizes contradict its stored segment lengths (k_cond_plan's
        // verdict) is reported, not decoded: its counts would index past its segments.
        if (cs.status != ST_OK) continue;
        if (have_lut != c.aux) {                           // bucket table of this chunk
            s_lut[t] = (uint16_t)(128u * cs.lut[t]);
            have_lut = c.aux;
        }
        const uint32_t pbase = (q - c.piece0) * PIECE_BYTES;
        if (c.rlen - pbase >= PIECE_BYTES) cf_piece<true>(a, sh, q, c, cj, cs);
        else cf_piece<false>(a, sh, q, c, cj, cs);
    }
}

}  // namespace lmz
