// k_cond_finish: the last pass of an exponent-conditioned BF16 chunk
// (lmz/codec.py:1144-1146: un-partition, then the BF16 field merge), one 64 KiB piece
// of output per 256 threads, three pieces in flight per CTA.
//
// The stable 8-way un-partition (lmz/native/lmzcore.c:614-641) gives element i the next
// unread byte of its bucket's segment; "next" is the number of earlier elements of the
// same bucket.  Here a warp owns a run of 4096 consecutive elements and walks it in
// blocks of 256, lane l holding elements 8l .. 8l+7 of the block:
//
//   * every element's bucket comes from its exponent byte through one 16-byte table entry:
//     a pair of one-hot words (8 bits per bucket), the bucket number, and four times it;
//   * the lane's eight one-hot pairs are summed, one warp scan of the sums gives the
//     lane its first rank in every bucket, and a running copy of that pair of words,
//     advanced by each element's one-hot, gives every element its rank -- one byte
//     permute, no chain through memory;
//   * the rank is added to the warp's position in that bucket's segment (eight words of
//     shared memory per warp, advanced once per block) and the byte is read from the
//     piece's share of the segment, staged in shared memory: consecutive elements of a
//     bucket read consecutive bytes, so a warp's 32 reads fall in a few words;
//   * the lane merges its eight exponents and eight bytes to 16 bytes of BF16, XORs the
//     delta base if there is one, stores them (a warp writes 512 contiguous bytes) and
//     folds them into the piece's CRC-32: four running values per lane, each multiplied
//     by x^4096 per block through tables in the bank-quartered layout (no conflicts).
//
// What a warp needs to know before it starts -- where its run begins in each segment --
// comes from k_cond_count (populations of every 4096-element run) and k_cond_scan
// (where the piece begins).
#pragma once
#include "chunk_kernels.cuh"

namespace lmz {

constexpr uint32_t CF_SUB = 256, CF_SUBS = 3, CF_THREADS = CF_SUB * CF_SUBS;
constexpr uint32_t CF_RUN = PIECE_ELEMS / 8;                  // elements one warp walks
constexpr uint32_t CF_BLOCK = 256;                            // elements per warp step
constexpr uint32_t CF_STAGE = PIECE_ELEMS + 8 * 32;           // eight ranges, each copied from its 16-byte boundary
constexpr uint32_t CF_LUT_BYTES = 256 * 16;                   // symbol -> {one-hot low, one-hot high, bucket, 4 * bucket}
constexpr uint32_t CF_SUB_BYTES = (CF_LUT_BYTES + CF_STAGE + 8 * 8 * 4 /*warp positions*/ + 256 /*misc*/ + 4095u) & ~4095u;
constexpr uint32_t CF_TABLE_BYTES = 32768;                    // four tables x 256 entries x eight copies
__host__ __device__ constexpr uint32_t cond_finish_smem()
{
    return 2 * CF_TABLE_BYTES /*the tables, wherever their 32 KiB boundary falls*/ + CF_SUBS * CF_SUB_BYTES;
}

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
    uint32_t stage_sa, lut_sa, wpos_sa, sub;
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
    const bool exp_al8 = (reinterpret_cast<uintptr_t>(exp) & 7u) == 0;
    const uint32_t *cnt_row = a.piece_cnt + (size_t)q * 16;
    const uint16_t *wcnt = a.piece_wcnt + (size_t)q * 64;

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
    // where this warp's run begins in every range: the range's start plus the populations
    // of the runs before it (shared address of the byte, one word per bucket)
    const uint32_t my_wpos = sh.wpos_sa + warp * 32;
    if (lane < 8) {
        uint32_t before = 0;
        for (uint32_t w = 0; w < warp; w++) before += wcnt[w * 8 + lane];
        sts_u32(my_wpos + 4 * lane, sh.stage_sa + sh.s_misc[lane] + before);
    }
    cf_sync(sh.sub);

    // ---- walk the run: 16 blocks of 256 elements, 8 per lane -------------------------------
    uint32_t ra[4] = {0, 0, 0, 0};
    auto fetch = [&](uint32_t j, uint32_t (&e)[2]) {                   // block j's exponents of this lane
        const uint32_t at = warp * CF_RUN + j * CF_BLOCK + lane * 8;
        e[0] = e[1] = 0;
        if (FULL || at < ne) {                                         // (the plane is padded past ne)
            if (exp_al8) {
                const uint2 v = __ldg(reinterpret_cast<const uint2 *>(exp + at));
                e[0] = v.x; e[1] = v.y;
            } else {
                load_words_nc<2>(exp + at, e);
            }
        }
    };
    uint32_t nx[2];
    fetch(0, nx);
#pragma unroll 1
    for (uint32_t j = 0; j < CF_RUN / CF_BLOCK; j++) {
        const uint32_t i0 = warp * CF_RUN + j * CF_BLOCK + lane * 8;   // first of this lane's eight elements
        const uint32_t valid = FULL ? 8u : (ne > i0 ? min(ne - i0, 8u) : 0u);
        const uint32_t ex[2] = {nx[0], nx[1]};
        if (j + 1 < CF_RUN / CF_BLOCK) fetch(j + 1, nx);               // the next block's, under this block's work
        // buckets: one table entry per element (the table is 4 KiB aligned: an index is OR-ed on)
        uint4 en[8];
        uint32_t slo = 0, shi = 0;
#pragma unroll
        for (int z = 0; z < 8; z++) {
            const uint32_t w = ex[z >> 2];
            const int zz = z & 3;
            const uint32_t ix = zz == 0 ? (w << 4) & 0xff0u : (w >> (8 * zz - 4)) & 0xff0u;
            en[z] = lds_u128(ix | sh.lut_sa);
            if (!FULL && (uint32_t)z >= valid) en[z].x = en[z].y = 0u;
            slo += en[z].x;
            shi += en[z].y;
        }
        // exclusive scan over the lanes: fields stay below 256 (31 lanes x 8 elements)
        uint32_t ilo = slo, ihi = shi;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t vlo = __shfl_up_sync(0xffffffffu, ilo, d), vhi = __shfl_up_sync(0xffffffffu, ihi, d);
            if (lane >= (uint32_t)d) { ilo += vlo; ihi += vhi; }
        }
        // (a field of the inclusive sums can reach 256 and spill into its neighbour; the
        // differences below are exact all the same, and the block totals are taken in two parts)
        uint32_t qlo = ilo - slo, qhi = ihi - shi;                     // ranks of this lane's first elements
        const uint32_t t1lo = __shfl_sync(0xffffffffu, qlo, 31), t1hi = __shfl_sync(0xffffffffu, qhi, 31);
        const uint32_t t2lo = __shfl_sync(0xffffffffu, slo, 31), t2hi = __shfl_sync(0xffffffffu, shi, 31);
        // every element's byte: warp position of its bucket + its rank within the block
        uint32_t sm[2] = {0, 0};
#pragma unroll
        for (int z = 0; z < 8; z++) {
            const uint32_t rank = __byte_perm(qlo, qhi, en[z].z) & 0xffu;
            const uint32_t at = lds_u32(my_wpos + en[z].w) + rank;
            qlo += en[z].x;
            qhi += en[z].y;
            if (FULL || (uint32_t)z < valid) {
                // the byte into place z & 3 of its word
                constexpr uint32_t SEL[4] = {0x3214u, 0x3240u, 0x3410u, 0x4210u};
                sm[z >> 2] = __byte_perm(sm[z >> 2], lds_u8(at), SEL[z & 3]);
            }
        }
        __syncwarp();
        if (lane < 8)                                                   // the block's populations move the warp on
            sts_u32(my_wpos + 4 * lane, lds_u32(my_wpos + 4 * lane) + (__byte_perm(t1lo, t1hi, lane) & 0xffu) +
                                            (__byte_perm(t2lo, t2hi, lane) & 0xffu));
        __syncwarp();

        uint32_t w[4];
        bf16_merge8(ex, sm, w);
        const uint32_t r = 2 * i0;                                      // piece-relative output offset
        if (base && valid) {
            uint32_t bw[4];
            load_words<4>(base + r, bw);
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] ^= bw[i];
        }
        if (FULL || valid == 8) {
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
            for (int i = 0; i < 4; i++) ra[i] = crc_feed4q(sh.cq, ra[i]) ^ w[i];
        }
    }
    if (do_crc) {
        // every running value to the end of the warp's 8 KiB, XOR over the warp, then to the piece's end
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) v ^= crc_mulmod(a.tabs->word_mul512[lane][i], ra[i]);
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
    const uint32_t tab0 = (s0 + CF_TABLE_BYTES - 1) & ~(CF_TABLE_BYTES - 1);
    uint8_t *mine = csm + (tab0 - s0) + CF_TABLE_BYTES + sub * CF_SUB_BYTES;
    CfShared sh;
    sh.sub = sub;
    uint4 *s_lut = reinterpret_cast<uint4 *>(mine);                              // 4 KiB aligned
    sh.s_stage = mine + CF_LUT_BYTES;
    uint32_t *s_wpos = reinterpret_cast<uint32_t *>(sh.s_stage + CF_STAGE);      // [warp][bucket]
    sh.s_misc = s_wpos + 64;                                                     // 64 words
    sh.stage_sa = smem_addr(sh.s_stage); sh.lut_sa = smem_addr(s_lut);
    sh.wpos_sa = smem_addr(s_wpos);
    // the x^4096 multiplication tables in the bank-quartered layout (see CrcQuarters): byte m of a
    // state goes through table m, which crc_feed4q looks for in slot 3 - m
    const uint32_t k = lane & 7u, g = lane >> 3;
#pragma unroll
    for (uint32_t i = 0; i < 4; i++) sh.cq.b[i] = tab0 + 32u * (3u - ((i + g) & 3u)) + 4u * k;
    sh.cq.rot = 8u * g;
    if (a.piece_crc) {
        uint32_t *tw = reinterpret_cast<uint32_t *>(csm + (tab0 - s0));
        for (uint32_t i = threadIdx.x; i < CF_TABLE_BYTES / 4; i += CF_THREADS)
            tw[i] = a.tabs->mul_row512[3u - ((i >> 3) & 3u)][i >> 5];
    }
    __syncthreads();
    uint32_t have_lut = 0xffffffffu;
    for (uint32_t q = a.piece_begin + blockIdx.x * CF_SUBS + sub; q < a.piece_end; q += gridDim.x * CF_SUBS) {
        const ChunkJob &c = a.chunks[a.piece_chunk[q]];
        const CondJob &cj = a.cond_jobs[c.aux];
        const CondState &cs = a.cond_state[c.aux];
        cf_sync(sub);                                      // the previous piece is done with shared memory
        // A chunk whose bucket sizes contradict its stored segment lengths (k_cond_plan's
        // verdict) is reported, not decoded: its counts would index past its segments.
        if (cs.status != ST_OK) continue;
        if (have_lut != c.aux) {                           // bucket tables of this chunk
            const uint32_t b = cs.lut[t];
            s_lut[t] = make_uint4(b < 4 ? 1u << (8 * b) : 0u, b < 4 ? 0u : 1u << (8 * (b - 4)), b, 4u * b);
            have_lut = c.aux;
        }
        const uint32_t pbase = (q - c.piece0) * PIECE_BYTES;
        if (c.rlen - pbase >= PIECE_BYTES) cf_piece<true>(a, sh, q, c, cj, cs);
        else cf_piece<false>(a, sh, q, c, cj, cs);
    }
}

}  // namespace lmz
