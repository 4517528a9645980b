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
// per-element gather then reads shared memory.  Gathering straight from global memory
// made every byte pull a 32-byte sector through an L1 that the shared-memory carve-out
// leaves almost empty.
#pragma once
#include "chunk_kernels.cuh"

namespace lmz {

constexpr uint32_t CF_THREADS = 256;
constexpr uint32_t CF_LOGR = 2;                               // CRC slice tables replicated 4x
constexpr uint32_t CF_STAGE = PIECE_ELEMS + 8 * 16;           // eight ranges, each 16-byte aligned
__host__ __device__ constexpr uint32_t cond_finish_smem()
{
    return 4 * (1024u << CF_LOGR) + (1024u << CF_LOGR) /*alignment*/ + PADDED_PIECE + CF_STAGE +
           256 /*lut*/ + 8 * CF_THREADS * 2 /*ranks*/ + 512 /*misc*/;
}

__global__ void __launch_bounds__(CF_THREADS) k_cond_finish(FinishArgs a)
{
    extern __shared__ __align__(16) uint8_t csm[];
    constexpr uint32_t TS = 1024u << CF_LOGR;
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t tab0 = (smem_addr(csm) + TS - 1) & ~(TS - 1);
    uint8_t *after = csm + (tab0 - smem_addr(csm)) + 4 * TS;
    uint8_t *s_exp = after;                                   // padded: 4 bytes per 128
    uint8_t *s_stage = s_exp + PADDED_PIECE;
    uint8_t *s_lut = s_stage + CF_STAGE;
    uint16_t *s_rank = reinterpret_cast<uint16_t *>(s_lut + 256);         // [bucket][thread]
    uint32_t *s_misc = reinterpret_cast<uint32_t *>(s_rank + 8 * CF_THREADS);   // 128 words
    const bool do_crc = a.piece_crc != nullptr;
    const uint32_t tl = tab0 + 4 * (lane & ((1u << CF_LOGR) - 1));

    if (do_crc) {
        uint32_t *tw = reinterpret_cast<uint32_t *>(csm + (tab0 - smem_addr(csm)));
        const uint32_t *src = &a.tabs->slice[0][0];
        for (uint32_t i = t; i < (4u * 256u) << CF_LOGR; i += CF_THREADS) tw[i] = src[i >> CF_LOGR];
    }
    __syncthreads();

    for (uint32_t q = a.piece_begin + blockIdx.x; q < a.piece_end; q += gridDim.x) {
        const ChunkJob &c = a.chunks[a.piece_chunk[q]];
        const CondJob &cj = a.cond_jobs[c.aux];
        const CondState &cs = a.cond_state[c.aux];
        const uint32_t p = q - c.piece0;
        const uint32_t pbase = p * PIECE_BYTES;
        const uint32_t plen = min(PIECE_BYTES, c.rlen - pbase), ne = plen / 2;
        uint8_t *dst = a.out + c.dst_off + pbase;
        const uint8_t *base = c.base_off == NONE64 ? nullptr : a.out + c.base_off + pbase;
        const uint32_t al = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u);
        const uint8_t *exp = (cj.exp_in_scratch ? a.scratch : a.payload) + cj.exp_off + pbase / 2;

        // ---- stage the exponent piece; bucket map; rank of the piece's first element ----
        s_lut[t] = cs.lut[t];
        for (uint32_t i0 = t * 4; i0 < PIECE_ELEMS; i0 += CF_THREADS * 4 * 8) {
            uint32_t w[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                uint32_t i = i0 + u * CF_THREADS * 4, v[1] = {0};
                if (i < ne) load_words_nc<1>(exp + i, v);
                w[u] = v[0];
            }
#pragma unroll
            for (int u = 0; u < 8; u++)
                *reinterpret_cast<uint32_t *>(s_exp + pad128(i0 + u * CF_THREADS * 4)) = w[u];
        }
        if (t < 8) s_misc[t] = 0;
        __syncthreads();
        {
            const uint32_t b = t & 7;
            uint32_t sum = 0;
            for (uint32_t j = t >> 3; j < p; j += CF_THREADS / 8)
                sum += a.piece_cnt[(size_t)(c.piece0 + j) * 8 + b];
            if (sum) atomicAdd(&s_misc[b], sum);
        }
        __syncthreads();
        // s_misc[8+b] = where bucket b's range starts in the staging buffer
        if (t == 0) {
            uint32_t pos = 0;
            for (int b = 0; b < 8; b++) {
                s_misc[8 + b] = pos;
                pos += (a.piece_cnt[(size_t)q * 8 + b] + 15u) & ~15u;
            }
        }
        __syncthreads();
        // ---- copy the piece's range of each segment into shared memory -----------------
        for (int b = 0; b < 8; b++) {
            const uint32_t cnt = a.piece_cnt[(size_t)q * 8 + b];
            const uint8_t *sp = (cs.seg_in_scratch >> b & 1 ? a.scratch : a.payload) + cs.seg_ptr[b] +
                                s_misc[b];
            uint8_t *dp = s_stage + s_misc[8 + b];
            for (uint32_t i = t * 4; i < cnt; i += CF_THREADS * 4) {
                uint32_t v[1];
                load_words_nc<1>(sp + i, v);
                *reinterpret_cast<uint32_t *>(dp + i) = v[0];
            }
        }
        // ---- phase A: this thread's bucket counts, then an exclusive scan over threads ----
        const uint32_t my0 = t * 128;
        uint64_t lo = 0, hi = 0;
        for (uint32_t j = 0; j < 128; j += 4) {
            uint32_t w = smem_word(s_exp, pad128(my0 + j));
#pragma unroll
            for (int z = 0; z < 4; z++) {
                if (my0 + j + z < ne) {
                    uint32_t b = s_lut[(w >> (8 * z)) & 0xff];
                    uint64_t one = 1ull << (16 * (b & 3));
                    if (b & 4) hi += one; else lo += one;
                }
            }
        }
        uint64_t ilo = lo, ihi = hi;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint64_t vl = __shfl_up_sync(0xffffffffu, ilo, d);
            uint64_t vh = __shfl_up_sync(0xffffffffu, ihi, d);
            if (lane >= (uint32_t)d) { ilo += vl; ihi += vh; }
        }
        uint64_t *s_w = reinterpret_cast<uint64_t *>(s_misc + 32);          // 8 warps x 2
        if (lane == 31) { s_w[warp * 2] = ilo; s_w[warp * 2 + 1] = ihi; }
        __syncthreads();
        uint64_t blo = 0, bhi = 0;
        for (uint32_t wv = 0; wv < warp; wv++) { blo += s_w[wv * 2]; bhi += s_w[wv * 2 + 1]; }
        const uint64_t xlo = ilo - lo + blo, xhi = ihi - hi + bhi;
        // running position of each bucket for this thread, as an index into the staging buffer
#pragma unroll
        for (int b = 0; b < 8; b++)
            s_rank[b * CF_THREADS + t] =
                (uint16_t)(s_misc[8 + b] + ((uint32_t)((b & 4 ? xhi : xlo) >> (16 * (b & 3))) & 0xffffu));
        // (own slots only: no barrier needed before the walk; the staging copy needs one)
        __syncthreads();

        // ---- walk: 16 groups of 8 elements = 16 bytes of output each -----------------------
        uint32_t acc = 0;
#pragma unroll 2
        for (uint32_t g = 0; g < 16; g++) {
            const uint32_t e0 = my0 + 8 * g;                 // first element of the group
            if (e0 >= ne) {
                if (do_crc) {
#pragma unroll
                    for (int i = 0; i < 4; i++) acc = crc_feed4<CF_LOGR>(tl, acc);
                }
                continue;
            }
            uint32_t ex[2] = {smem_word(s_exp, pad128(e0)), smem_word(s_exp, pad128(e0) + 4)};
            uint32_t sm[2] = {0, 0};
#pragma unroll
            for (int z = 0; z < 8; z++) {
                const uint32_t b = s_lut[(ex[z >> 2] >> (8 * (z & 3))) & 0xff];
                uint16_t *rk = s_rank + b * CF_THREADS + t;
                const uint32_t idx = *rk;
                const bool live = e0 + z < ne;
                if (live) *rk = (uint16_t)(idx + 1);
                sm[z >> 2] |= (uint32_t)s_stage[live ? idx : 0] << (8 * (z & 3));
            }
            uint32_t w[4];
            bf16_merge8(ex, sm, w);
            const uint32_t r = 2 * e0;                        // piece-relative output offset
            if (base) {
                uint32_t bw[4];
                load_words<4>(base + r, bw);
#pragma unroll
                for (int i = 0; i < 4; i++) w[i] ^= bw[i];
            }
            const uint32_t left = plen - r;
            if (left >= 16 && (al & 3) == 0) {
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
                for (int i = 0; i < 4; i++) acc = crc_feed4<CF_LOGR>(tl, acc ^ w[i]);
            }
        }
        if (do_crc) {
            uint32_t v = crc_mulmod(a.tabs->run_mul[t], acc);
#pragma unroll
            for (int d = 16; d; d >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0) s_misc[64 + warp] = v;
            __syncthreads();
            if (t == 0) {
                uint32_t r = 0;
                for (int i = 0; i < 8; i++) r ^= s_misc[64 + i];
                if (plen < PIECE_BYTES) r = crc_unshift(a.tabs->x2, r, PIECE_BYTES - plen);
                a.piece_crc[q] = r;
            }
        }
        __syncthreads();
    }
}

}  // namespace lmz
