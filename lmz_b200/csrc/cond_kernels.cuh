// Support kernels for exponent-conditioned BF16 chunks (reference
// lmz/codec.py:1116-1142) and the per-chunk checksum verdict.
#pragma once
#include "chunk_kernels.cuh"

namespace lmz {

struct CondArgs {
    const ChunkJob *chunks;
    const uint32_t *piece_chunk;
    const uint32_t *cond_pieces;   // piece ids that belong to K_COND chunks
    uint32_t ncond_pieces;
    const CondJob *cond_jobs;
    CondState *cond_state;
    uint32_t ncond;
    uint32_t *hist;                // ncond x 256, zeroed by the caller
    uint32_t *piece_cnt;           // npieces x 16: 8 populations, then 8 running totals (k_cond_scan)
    uint16_t *piece_wcnt;          // npieces x 8 x 8: the populations of each 4096-element run of a piece
    uint32_t *piece_lcnt;          // ncond_pieces x 8 runs x 4 blocks x 32 lanes x 2 words: the populations of the
                                   // 32 consecutive elements one lane of k_cond_finish takes, as 8-bit fields
                                   // (buckets 0, 2, 4, 6 in the first word, 1, 3, 5, 7 in the second)
    StreamJob *seg_jobs;           // one slot per rANS-coded segment, sized by k_cond_plan
    const uint8_t *payload;
    const uint8_t *scratch;
};

__device__ __forceinline__ const uint8_t *cond_exp_piece(const CondArgs &a, uint32_t q,
                                                         uint32_t &ci, uint32_t &ne)
{
    const ChunkJob &c = a.chunks[a.piece_chunk[q]];
    ci = c.aux;
    const CondJob &cj = a.cond_jobs[ci];
    uint32_t e0 = (q - c.piece0) * PIECE_ELEMS;
    ne = min(PIECE_ELEMS, cj.nelem - e0);
    return (cj.exp_in_scratch ? a.scratch : a.payload) + cj.exp_off + e0;
}

// 256-bin histogram of one exponent piece (lmz/native/lmzcore.c:385-397), accumulated in
// shared memory, then added to the chunk's histogram.  Exponent planes have a handful of
// popular symbols, so the lanes of a warp keep asking for the same counter; every lane
// therefore has its own copy of the histogram, laid out [bin][lane]: whatever the bins, the
// 32 additions of a warp go to 32 different banks, and only warps meet on a counter.
__global__ void __launch_bounds__(256) k_cond_hist(CondArgs a)
{
    __shared__ uint32_t h[256][32];
    const uint32_t t = threadIdx.x, lane = t & 31;
    for (uint32_t i = t; i < 32 * 256; i += 256) (&h[0][0])[i] = 0;
    __syncthreads();
    uint32_t ci, ne;
    const uint8_t *exp = cond_exp_piece(a, a.cond_pieces[blockIdx.x], ci, ne);
    uint32_t *mine = &h[0][lane];
    auto add4 = [&](uint32_t w) {
        atomicAdd(mine + 32u * (w & 0xffu), 1u);
        atomicAdd(mine + 32u * __byte_perm(w, 0u, 0x4441u), 1u);
        atomicAdd(mine + 32u * __byte_perm(w, 0u, 0x4442u), 1u);
        atomicAdd(mine + 32u * (w >> 24), 1u);
    };
    if (ne == PIECE_ELEMS && (reinterpret_cast<uintptr_t>(exp) & 15u) == 0) {
        // a whole piece, aligned: 128 bytes per thread as eight 16-byte loads, all in flight
        const uint4 *e4 = reinterpret_cast<const uint4 *>(exp) + t;
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = e4[u * 256];
#pragma unroll
        for (int u = 0; u < 8; u++) { add4(v[u].x); add4(v[u].y); add4(v[u].z); add4(v[u].w); }
    } else {
        for (uint32_t i0 = t * 4; i0 < ne; i0 += 256 * 4 * 8) {
            uint32_t w[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                uint32_t i = i0 + u * 256 * 4, v[1] = {0};
                if (i < ne) load_words<1>(exp + i, v);
                w[u] = v[0];
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                uint32_t i = i0 + u * 256 * 4;
                if (i + 4 <= ne) add4(w[u]);
                else
                    for (uint32_t z = 0; i + z < ne; z++) atomicAdd(mine + 32u * ((w[u] >> (8 * z)) & 0xffu), 1u);
            }
        }
    }
    __syncthreads();
    // bin t: its 32 copies, each thread starting at a different one (different banks)
    uint32_t s = 0;
#pragma unroll
    for (uint32_t l = 0; l < 32; l++) s += h[t][(l + t) & 31u];
    if (s) atomicAdd(&a.hist[(size_t)ci * 256 + t], s);
}

// One thread per conditioned chunk: the bucket map (lmz/native/lmzcore.c:525-543,
// same 64-bit products), the bucket sizes (lmz/kernels.py:481-486), the checks
// of lmz/codec.py:1120-1142, and the sizes/destinations of the segment decodes.
__global__ void k_cond_plan(CondArgs a)
{
    uint32_t ci = blockIdx.x * blockDim.x + threadIdx.x;
    if (ci >= a.ncond) return;
    const CondJob &cj = a.cond_jobs[ci];
    CondState &cs = a.cond_state[ci];
    const uint32_t *hist = a.hist + (size_t)ci * 256;
    uint64_t total = 0;
    for (int s = 0; s < 256; s++) total += hist[s];
    uint32_t counts[COND_BUCKETS] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint64_t acc = 0, b = 0;
    for (int s = 0; s < 256; s++) {
        cs.lut[s] = (uint8_t)b;
        uint32_t hs = hist[s];
        // counts[b] with a dynamic b would go to local memory; select instead
#pragma unroll
        for (int j = 0; j < COND_BUCKETS; j++) counts[j] += (b == (uint64_t)j) ? hs : 0u;
        acc += hs;
        while (b + 1 < COND_BUCKETS && acc * COND_BUCKETS >= (b + 1) * total) b++;
    }
    uint32_t status = total == cj.nelem ? ST_OK : ST_BAD_SHAPE;
    uint64_t run = 0;
    uint32_t in_scratch = 0, nj = 0;      // nj: this chunk's rANS segments seen so far
#pragma unroll
    for (int j = 0; j < COND_BUCKETS; j++) {
        uint32_t want = counts[j], ln = cj.seg_len[j], m = cj.seg_method[j];
        cs.counts[j] = want;
        cs.seg_ptr[j] = cj.seg_src[j];
        // the host made one job slot per rANS-coded, non-empty segment, in bucket order
        const bool slot = m == 3 && ln != 0;
        if (slot) a.seg_jobs[cj.seg_job0 + nj].n = 0;
        if (want == 0) {
            if (ln) status = ST_BAD_SHAPE;
        } else if (m == 0) {
            if (ln != want) status = ST_BAD_SHAPE;
        } else if (slot) {
            StreamJob &sj = a.seg_jobs[cj.seg_job0 + nj];
            cs.seg_ptr[j] = cj.seg_scratch + run;
            in_scratch |= 1u << j;
            sj.dst_off = cj.seg_scratch + run;
            sj.n = want;
            run += want;
        } else {
            status = ST_BAD_SHAPE;
        }
        nj += slot;
    }
    if (status != ST_OK)
        for (uint32_t j = 0; j < nj; j++) a.seg_jobs[cj.seg_job0 + j].n = 0;
    cs.seg_in_scratch = in_scratch;
    cs.status = status;
}

// Bucket populations of one exponent piece, for the stable un-partition's read positions: of
// the piece (piece_cnt), of each of its eight 4096-element runs (piece_wcnt; one run per
// warp, which is how k_cond_finish walks the piece) and of the 32 consecutive elements every
// lane of that kernel takes in each of a run's four blocks (piece_lcnt).  A symbol's bucket
// is looked up as a byte (four times the bucket number) and counted as a one-hot word of
// 4-bit fields: a byte extract, one shared load, a shift and an add per element; every
// twelve elements the nibbles are spread into 8-bit fields (buckets 0, 2, 4, 6 in one word,
// 1, 3, 5, 7 in the other).  Half a KiB of shared memory: with the KiB the system reserves
// per block that still fits beside the segment decodes that run at the same time and leave
// under 2 KiB of an SM free.
__global__ void __launch_bounds__(256) k_cond_count(CondArgs a)
{
    __shared__ uint8_t hot[256];                          // symbol -> 4 * bucket
    __shared__ uint32_t cnt[8][COND_BUCKETS];
    const uint32_t t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t q = a.cond_pieces[blockIdx.x];
    uint32_t ci, ne;
    const uint8_t *exp = cond_exp_piece(a, q, ci, ne);
    hot[t] = (uint8_t)(4 * a.cond_state[ci].lut[t]);
    __syncthreads();
    uint32_t lo = 0, hi = 0, nib = 0;
    auto flush = [&]() {
        lo += nib & 0x0f0f0f0fu;
        hi += (nib >> 4) & 0x0f0f0f0fu;
        nib = 0;
    };
    auto add4 = [&](uint32_t w) {
        nib += 1u << hot[w & 0xffu];
        nib += 1u << hot[__byte_perm(w, 0u, 0x4441u)];
        nib += 1u << hot[__byte_perm(w, 0u, 0x4442u)];
        nib += 1u << hot[w >> 24];
    };
    // warp w takes elements [4096 w, 4096 w + 4096) in four blocks of 1024, lane l the 32
    // elements from 32 l of each
    const uint32_t w0 = warp * (PIECE_ELEMS / 8) + lane * 32;
    uint2 *lc = reinterpret_cast<uint2 *>(a.piece_lcnt) + ((size_t)blockIdx.x * 8 + warp) * 128 + lane;
    uint32_t run_lo = 0, run_hi = 0;
    if (ne == PIECE_ELEMS && (reinterpret_cast<uintptr_t>(exp) & 15u) == 0) {
        // a whole piece, aligned: eight 16-byte loads per lane, all in flight
        const uint4 *e4 = reinterpret_cast<const uint4 *>(exp + w0);
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 4; j++) { v[2 * j] = e4[j * 64]; v[2 * j + 1] = e4[j * 64 + 1]; }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t w[8] = {v[2 * j].x, v[2 * j].y, v[2 * j].z, v[2 * j].w,
                                   v[2 * j + 1].x, v[2 * j + 1].y, v[2 * j + 1].z, v[2 * j + 1].w};
#pragma unroll
            for (int c = 0; c < 8; c++) {
                add4(w[c]);
                if (c % 3 == 2) flush();                   // twelve additions at most
            }
            flush();
            lc[j * 32] = make_uint2(lo, hi);
            run_lo += lo; run_hi += hi;
            lo = hi = 0;
        }
    } else {
        for (uint32_t j = 0; j < 4; j++) {
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint32_t i = w0 + j * 1024 + 4 * c;
                if (i < ne) {
                    uint32_t v[1];
                    load_words<1>(exp + i, v);
                    if (i + 4 <= ne) add4(v[0]);
                    else
                        for (uint32_t z = 0; i + z < ne; z++) nib += 1u << hot[(v[0] >> (8 * z)) & 0xffu];
                }
                if (c % 3 == 2) flush();
            }
            flush();
            lc[j * 32] = make_uint2(lo, hi);
            run_lo += lo; run_hi += hi;
            lo = hi = 0;
        }
    }
    // 8-bit fields -> 16-bit fields (a warp sees at most 4096 elements), then a butterfly
    uint32_t f[4] = {run_lo & 0x00ff00ffu, (run_lo >> 8) & 0x00ff00ffu, run_hi & 0x00ff00ffu, (run_hi >> 8) & 0x00ff00ffu};
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int d = 16; d; d >>= 1) f[j] += __shfl_xor_sync(0xffffffffu, f[j], d);
    }
    if (lane == 0) {
        // lo bytes = buckets 0, 2, 4, 6 and hi bytes = buckets 1, 3, 5, 7:
        // f[0] = buckets 0,4  f[1] = buckets 2,6  f[2] = buckets 1,5  f[3] = buckets 3,7
        cnt[warp][0] = f[0] & 0xffffu; cnt[warp][4] = f[0] >> 16;
        cnt[warp][2] = f[1] & 0xffffu; cnt[warp][6] = f[1] >> 16;
        cnt[warp][1] = f[2] & 0xffffu; cnt[warp][5] = f[2] >> 16;
        cnt[warp][3] = f[3] & 0xffffu; cnt[warp][7] = f[3] >> 16;
    }
    __syncthreads();
    if (t < COND_BUCKETS) {
        uint32_t s = 0;
        for (int w = 0; w < 8; w++) s += cnt[w][t];
        a.piece_cnt[(size_t)q * 16 + t] = s;
    }
    if (t < 64) a.piece_wcnt[(size_t)q * 64 + t] = (uint16_t)cnt[t >> 3][t & 7];
}

struct CheckArgs {
    const ChunkJob *chunks;
    uint32_t nchunks;
    const uint32_t *piece_crc;
    const CrcTables *tabs;
    const CondState *cond_state;
    uint32_t *chunk_status;        // one word per chunk
    uint32_t *chunk_crc;           // computed crc32 per chunk (may be NULL)
    uint32_t *any_bad;
};

// One thread per chunk: crc32 = shift(~0, rlen) ^ XOR_j shift(R_j, bytes after piece j) ^ ~0.
__global__ void k_crc_check(CheckArgs a)
{
    uint32_t ci = blockIdx.x * blockDim.x + threadIdx.x;
    if (ci >= a.nchunks) return;
    const ChunkJob &c = a.chunks[ci];
    uint32_t status = ST_OK;
    if (c.kind == K_COND) status = a.cond_state[c.aux].status;
    if (a.piece_crc && (c.crc || a.chunk_crc)) {
        const uint32_t *x2 = a.tabs->x2;
        uint32_t np = (c.rlen + PIECE_BYTES - 1) / PIECE_BYTES;
        uint32_t acc = crc_shift(x2, 0xffffffffu, c.rlen);
        // Horner over the pieces: all but the last are PIECE_BYTES long.
        uint32_t r = 0;
        const uint32_t full = crc_xpow(x2, 8ull * PIECE_BYTES);
        for (uint32_t j = 0; j < np; j++) {
            uint32_t len = min(PIECE_BYTES, c.rlen - j * PIECE_BYTES);
            r = (len == PIECE_BYTES ? crc_mulmod(full, r) : crc_shift(x2, r, len)) ^
                a.piece_crc[c.piece0 + j];
        }
        uint32_t crc = acc ^ r ^ 0xffffffffu;
        if (a.chunk_crc) a.chunk_crc[ci] = crc;
        if (c.crc && crc != c.crc && status == ST_OK) status = ST_BAD_CRC;
    }
    a.chunk_status[ci] = status;
    if (status != ST_OK && a.any_bad) atomicOr(a.any_bad, 2u);
}

}  // namespace lmz
