// k_cond_finish: the last pass of an exponent-conditioned BF16 chunk
// (lmz/codec.py:1144-1146: un-partition, then the BF16 field merge), one 64 KiB piece
// of output per 256 threads.
//
// Thread t owns elements [128 t, 128 t + 128) of the piece: it deals each element's
// sign/mantissa byte back from its bucket's segment in order (the stable 8-way
// un-partition of lmz/native/lmzcore.c:614-641), merges it with the exponent, XORs
// a delta base if there is one, writes its 256 contiguous output bytes and folds them
// into the piece's CRC-32.
//
// The piece's share of every segment is one contiguous range (ranks are stable), so
// the eight ranges are first copied into shared memory with coalesced loads; the
// (whole 16-byte units from each range's 16-byte boundary, so the loads vectorise); the
// per-element gather then reads shared memory.  A thread keeps its 128 exponent bytes
// in registers: it counts its buckets from them (one-hot words, as k_cond_count does),
// a scan over the threads turns the counts into each thread's first position in every
// range, and the walk then costs three dependent shared accesses per element: bucket
// row, running position (read, advance), byte.
#pragma once
#include "chunk_kernels.cuh"

namespace lmz {

constexpr uint32_t CF_THREADS = 256, CF_RUN = PIECE_ELEMS / CF_THREADS;   // 128 elements per thread
constexpr uint32_t CF_LOGR = 2;                               // CRC slice tables replicated 4x
constexpr uint32_t CF_STAGE = PIECE_ELEMS + 8 * 32;           // eight ranges, each copied from its 16-byte boundary
constexpr uint32_t CF_POS_ROW = CF_THREADS * 4;               // one word per thread and bucket: no two lanes share a bank
__host__ __device__ constexpr uint32_t cond_finish_smem()
{
    return 4 * (1024u << CF_LOGR) + (1024u << CF_LOGR) /*alignment*/ + CF_STAGE + 256 * 8 /*one-hot*/ +
           256 * 2 /*bucket rows*/ + 8 * CF_POS_ROW + 512 /*misc*/;
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
    uint32_t stage_sa, hot_sa, row_sa, mypos_sa, tl;
    uint32_t *s_pos;
    uint32_t *s_misc;
    uint8_t *s_stage;
};

// One piece.  FULL: the piece has all 32768 elements, so no thread checks a tail.
template <bool FULL>
__device__ __forceinline__ void cf_piece(const FinishArgs &a, const CfShared &sh, uint32_t q,
                                         const ChunkJob &c, const CondJob &cj, const CondState &cs)
{
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const bool do_crc = a.piece_crc != nullptr;
    const uint32_t p = q - c.piece0;
    const uint32_t pbase = p * PIECE_BYTES;
    const uint32_t plen = FULL ? PIECE_BYTES : min(PIECE_BYTES, c.rlen - pbase), ne = plen / 2;
    uint8_t *dst = a.out + c.dst_off + pbase;
    const uint8_t *base = c.base_off == NONE64 ? nullptr : a.out + c.base_off + pbase;
    const uint32_t al = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u);
    const uint8_t *exp = (cj.exp_in_scratch ? a.scratch : a.payload) + cj.exp_off + pbase / 2;
    const uint32_t my0 = t * CF_RUN;
    const uint32_t mine = FULL ? CF_RUN : (ne > my0 ? min(ne - my0, CF_RUN) : 0u);   // live elements
    const uint32_t *cnt_row = a.piece_cnt + (size_t)q * 16;

    // ---- this thread's exponents (the plane is padded past ne) -----------------------
    uint32_t ex[CF_RUN / 4];
    if ((reinterpret_cast<uintptr_t>(exp) & 15u) == 0) {
        const uint4 *e4 = reinterpret_cast<const uint4 *>(exp + my0);
#pragma unroll
        for (int j = 0; j < (int)CF_RUN / 16; j++) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (FULL || my0 + 16 * j < ne) v = __ldg(e4 + j);
            ex[4 * j] = v.x; ex[4 * j + 1] = v.y; ex[4 * j + 2] = v.z; ex[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < (int)CF_RUN / 4; j += 4) {
            uint32_t v[4] = {0, 0, 0, 0};
            if (FULL || my0 + 4 * j < ne) load_words_nc<4>(exp + my0 + 4 * j, v);
#pragma unroll
            for (int i = 0; i < 4; i++) ex[j + i] = v[i];
        }
    }
    // ---- the piece's range of each segment -> shared memory, whole 16-byte units -------
    // s_misc[b] = offset in the staging buffer of the range's first byte
    if (t < 8) {
        const uint32_t b = t;
        uint32_t pos = 0;
        for (uint32_t j = 0; j < b; j++) pos += (cnt_row[j] + 30u) & ~15u;      // room for any skew, whole units
        const uint8_t *sp = (cs.seg_in_scratch >> b & 1 ? a.scratch : a.payload) + cs.seg_ptr[b] + cnt_row[8 + b];
        sh.s_misc[b] = pos + (uint32_t)(reinterpret_cast<uintptr_t>(sp) & 15u);
    }
    __syncthreads();
#pragma unroll 1
    for (int b = 0; b < 8; b++) {
        const uint32_t cnt = cnt_row[b];
        if (!cnt) continue;
        const uint8_t *sp = (cs.seg_in_scratch >> b & 1 ? a.scratch : a.payload) + cs.seg_ptr[b] + cnt_row[8 + b];
        const uint32_t skew = (uint32_t)(reinterpret_cast<uintptr_t>(sp) & 15u);
        const uint4 *s4 = reinterpret_cast<const uint4 *>(sp - skew);
        uint4 *d4 = reinterpret_cast<uint4 *>(sh.s_stage + (sh.s_misc[b] - skew));
        const uint32_t nvec = (skew + cnt + 15u) >> 4;
        for (uint32_t i = t; i < nvec; i += CF_THREADS) d4[i] = __ldg(s4 + i);
    }
    // ---- this thread's bucket counts (8-bit fields), then an exclusive scan over threads ----
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < (int)CF_RUN / 4; j++) {
        const uint32_t w = ex[j];
        const uint32_t ix[4] = {(w << 3) & 0x7f8u, (w >> 5) & 0x7f8u, (w >> 13) & 0x7f8u, (w >> 21) & 0x7f8u};
#pragma unroll
        for (int z = 0; z < 4; z++) {
            if (FULL || (uint32_t)(4 * j + z) < mine) {
                const uint2 h = lds_u64(sh.hot_sa + ix[z]);
                lo += h.x;
                hi += h.y;
            }
        }
    }
    // 16-bit fields: f[0] = buckets 0,2  f[1] = buckets 1,3  f[2] = buckets 4,6  f[3] = buckets 5,7
    uint32_t f[4] = {lo & 0x00ff00ffu, (lo >> 8) & 0x00ff00ffu, hi & 0x00ff00ffu, (hi >> 8) & 0x00ff00ffu};
    uint32_t inc[4] = {f[0], f[1], f[2], f[3]};
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, inc[j], d);
            if (lane >= (uint32_t)d) inc[j] += v;
        }
    }
    uint32_t *s_w = sh.s_misc + 32;                                      // 8 warps x 4
    if (lane == 31) {
#pragma unroll
        for (int j = 0; j < 4; j++) s_w[warp * 4 + j] = inc[j];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t before = 0;
        for (uint32_t wv = 0; wv < warp; wv++) before += s_w[wv * 4 + j];
        inc[j] += before - f[j];                                        // exclusive, over the whole piece
    }
    // running position of each bucket for this thread, as an offset into the staging buffer
    // (own slots only: nobody else reads them)
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const uint32_t field = (inc[(b >> 2) * 2 + (b & 1)] >> (16 * ((b >> 1) & 1))) & 0xffffu;
        sh.s_pos[b * CF_THREADS + t] = sh.s_misc[b] + field;
    }

    // ---- walk: 16 groups of 8 elements = 16 bytes of output each -----------------------
    uint32_t acc = 0;
#pragma unroll
    for (int g = 0; g < (int)CF_RUN / 8; g++) {
        if (!FULL && 8u * g >= mine) {
            if (do_crc) {
#pragma unroll
                for (int i = 0; i < 4; i++) acc = crc_feed4<CF_LOGR>(sh.tl, acc);
            }
            continue;
        }
        const uint32_t exg[2] = {ex[2 * g], ex[2 * g + 1]};
        // bucket rows first (independent loads), then the running positions in element
        // order (two elements of one bucket must see each other's update), bytes last
        uint32_t pa[8], idx[8];
#pragma unroll
        for (int z = 0; z < 8; z++) {
            const uint32_t w = exg[z >> 2];
            const int zz = z & 3;
            const uint32_t ri = zz == 0 ? (w << 1) & 0x1feu : (w >> (8 * zz - 1)) & 0x1feu;
            pa[z] = sh.mypos_sa + lds_u16(sh.row_sa + ri);
        }
#pragma unroll
        for (int z = 0; z < 8; z++) {
            idx[z] = 0;
            if (FULL || (uint32_t)(8 * g + z) < mine) {
                idx[z] = lds_u32(pa[z]);
                sts_u32(pa[z], idx[z] + 1);
            }
        }
        uint32_t sm[2] = {0, 0};
#pragma unroll
        for (int z = 0; z < 8; z++) sm[z >> 2] |= lds_u8(sh.stage_sa + idx[z]) << (8 * (z & 3));
        uint32_t w[4];
        bf16_merge8(exg, sm, w);
        const uint32_t r = 2 * (my0 + 8 * g);              // piece-relative output offset
        if (base) {
            uint32_t bw[4];
            load_words<4>(base + r, bw);
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] ^= bw[i];
        }
        const uint32_t left = plen - r;
        if ((FULL || left >= 16) && (al & 3) == 0) {
            uint8_t *d = dst + r;
            if (al == 0) *reinterpret_cast<uint4 *>(d) = make_uint4(w[0], w[1], w[2], w[3]);
            else if ((al & 7) == 0) {
                reinterpret_cast<uint2 *>(d)[0] = make_uint2(w[0], w[1]);
                reinterpret_cast<uint2 *>(d)[1] = make_uint2(w[2], w[3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(d)[i] = w[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++)
                if ((uint32_t)i < left) dst[r + i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t keep = left > 4u * i ? min(left - 4u * i, 4u) : 0u;
                w[i] = keep >= 4 ? w[i] : (keep ? w[i] & ((1u << (8 * keep)) - 1u) : 0u);
            }
        }
        if (do_crc) {
#pragma unroll
            for (int i = 0; i < 4; i++) acc = crc_feed4<CF_LOGR>(sh.tl, acc ^ w[i]);
        }
    }
    if (do_crc) {
        uint32_t v = crc_mulmod(a.tabs->run_mul[t], acc);
#pragma unroll
        for (int d = 16; d; d >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, d);
        if (lane == 0) sh.s_misc[64 + warp] = v;
        __syncthreads();
        if (t == 0) {
            uint32_t r = 0;
            for (int i = 0; i < 8; i++) r ^= sh.s_misc[64 + i];
            if (plen < PIECE_BYTES) r = crc_unshift(a.tabs->x2, r, PIECE_BYTES - plen);
            a.piece_crc[q] = r;
        }
    }
}

__global__ void __launch_bounds__(CF_THREADS, 3) k_cond_finish(FinishArgs a)
{
    extern __shared__ __align__(16) uint8_t csm[];
    constexpr uint32_t TS = 1024u << CF_LOGR;
    const uint32_t t = threadIdx.x, lane = t & 31;
    const uint32_t tab0 = (smem_addr(csm) + TS - 1) & ~(TS - 1);
    uint8_t *after = csm + (tab0 - smem_addr(csm)) + 4 * TS;
    CfShared sh;
    sh.s_stage = after;
    uint2 *s_hot = reinterpret_cast<uint2 *>(sh.s_stage + CF_STAGE);             // symbol -> one-hot bucket words
    uint16_t *s_row = reinterpret_cast<uint16_t *>(s_hot + 256);                 // symbol -> bucket * CF_POS_ROW
    sh.s_pos = reinterpret_cast<uint32_t *>(s_row + 256);                        // [bucket][thread]
    sh.s_misc = sh.s_pos + 8 * CF_THREADS;                                       // 128 words
    sh.stage_sa = smem_addr(sh.s_stage); sh.hot_sa = smem_addr(s_hot); sh.row_sa = smem_addr(s_row);
    sh.mypos_sa = smem_addr(sh.s_pos) + 4 * t;
    sh.tl = tab0 + 4 * (lane & ((1u << CF_LOGR) - 1));

    if (a.piece_crc) {
        uint32_t *tw = reinterpret_cast<uint32_t *>(csm + (tab0 - smem_addr(csm)));
        const uint32_t *src = &a.tabs->slice[0][0];
        for (uint32_t i = t; i < (4u * 256u) << CF_LOGR; i += CF_THREADS) tw[i] = src[i >> CF_LOGR];
    }
    uint32_t have_lut = 0xffffffffu;
    for (uint32_t q = a.piece_begin + blockIdx.x; q < a.piece_end; q += gridDim.x) {
        const ChunkJob &c = a.chunks[a.piece_chunk[q]];
        const CondJob &cj = a.cond_jobs[c.aux];
        const CondState &cs = a.cond_state[c.aux];
        __syncthreads();                                   // the previous piece is done with shared memory
        // A chunk whose bucket sizes contradict its stored segment lengths (k_cond_plan's
        // verdict) is reported, not decoded: its counts would index past its segments.
        if (cs.status != ST_OK) continue;
        if (have_lut != c.aux) {                           // bucket tables of this chunk
            const uint32_t b = cs.lut[t];
            s_hot[t] = make_uint2(b < 4 ? 1u << (8 * b) : 0u, b < 4 ? 0u : 1u << (8 * (b - 4)));
            s_row[t] = (uint16_t)(b * CF_POS_ROW);
            have_lut = c.aux;
        }
        const uint32_t pbase = (q - c.piece0) * PIECE_BYTES;
        if (c.rlen - pbase >= PIECE_BYTES) cf_piece<true>(a, sh, q, c, cj, cs);
        else cf_piece<false>(a, sh, q, c, cj, cs);
    }
}

}  // namespace lmz
