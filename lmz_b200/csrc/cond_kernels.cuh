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
// popular symbols, so lanes of a warp keep hitting the same counter: every warp has four
// copies of the histogram (one per lane & 3) to spread those collisions.
__global__ void __launch_bounds__(256) k_cond_hist(CondArgs a)
{
    __shared__ uint32_t h[32][256];
    const uint32_t t = threadIdx.x, warp = t >> 5, mine = warp * 4 + (t & 3u);
    for (uint32_t i = t; i < 32 * 256; i += 256) (&h[0][0])[i] = 0;
    __syncthreads();
    uint32_t ci, ne;
    const uint8_t *exp = cond_exp_piece(a, a.cond_pieces[blockIdx.x], ci, ne);
    // 32 KiB per piece = 32 words per thread; loaded 8 at a time so the reads overlap
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
#pragma unroll
            for (int z = 0; z < 4; z++)
                if (i + z < ne) atomicAdd(&h[mine][(w[u] >> (8 * z)) & 0xff], 1u);
        }
    }
    __syncthreads();
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < 32; w++) s += h[w][t];
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

// Bucket populations of one exponent piece, for the stable un-partition's ranks: of the
// piece (piece_cnt) and of each of its eight 4096-element runs (piece_wcnt), one run per
// warp, which is how k_cond_finish walks the piece.  A symbol's bucket is looked up as a
// byte (four times the bucket number) and counted as a one-hot word of 4-bit fields, one
// shared load, a shift and an add per element; every twelve elements the nibbles are spread
// into 8-bit fields (buckets 0, 2, 4, 6 in one word, 1, 3, 5, 7 in the other), which hold the
// 128 elements a thread sees.  Half a KiB of shared memory: with the KiB the system reserves
// per block that still fits beside the segment decodes that run at the same time and leave
// under 2 KiB of an SM free.
__global__ void __launch_bounds__(256) k_cond_count(CondArgs a)
{
    __shared__ __align__(256) uint32_t both[64 + 8 * COND_BUCKETS];     // one array: no padding between the two
    uint8_t *hot = reinterpret_cast<uint8_t *>(both);                   // symbol -> 4 * bucket
    uint32_t (*cnt)[COND_BUCKETS] = reinterpret_cast<uint32_t (*)[COND_BUCKETS]>(both + 64);
    const uint32_t t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t q = a.cond_pieces[blockIdx.x];
    uint32_t ci, ne;
    const uint8_t *exp = cond_exp_piece(a, q, ci, ne);
    hot[t] = (uint8_t)(4 * a.cond_state[ci].lut[t]);
    __syncthreads();
    const uint32_t hot_sa = smem_addr(hot);               // 256-byte aligned: an index is OR-ed on
    uint32_t lo = 0, hi = 0, nib = 0;
    auto flush = [&]() {
        lo += nib & 0x0f0f0f0fu;
        hi += (nib >> 4) & 0x0f0f0f0fu;
        nib = 0;
    };
    // warp w takes elements [4096 w, 4096 w + 4096): 32 words per lane, loaded 8 at a time
    const uint32_t w0 = warp * (PIECE_ELEMS / 8);
    for (uint32_t j0 = 0; j0 < 32; j0 += 8) {
        uint32_t w[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            uint32_t i = w0 + (j0 + u) * 128 + lane * 4, v[1] = {0};
            if (i < ne) load_words<1>(exp + i, v);
            w[u] = v[0];
        }
        const bool whole = w0 + (j0 + 7) * 128 + lane * 4 + 4 <= ne;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint32_t i = w0 + (j0 + u) * 128 + lane * 4;
            const uint32_t valid = whole ? 4u : (i < ne ? min(ne - i, 4u) : 0u);
            const uint32_t ix[4] = {w[u] & 0xffu, (w[u] >> 8) & 0xffu, (w[u] >> 16) & 0xffu, w[u] >> 24};
#pragma unroll
            for (int z = 0; z < 4; z++)
                if (whole || (uint32_t)z < valid) nib += 1u << lds_u8(ix[z] | hot_sa);
            if (u % 3 == 2) flush();                       // at most twelve additions between flushes
        }
        flush();
    }
    // 8-bit fields -> 16-bit fields (a warp sees at most 4096 elements), then a butterfly
    uint32_t f[4] = {lo & 0x00ff00ffu, (lo >> 8) & 0x00ff00ffu, hi & 0x00ff00ffu, (hi >> 8) & 0x00ff00ffu};
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
