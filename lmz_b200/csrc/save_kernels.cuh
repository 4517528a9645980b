// The way back at chunk level: from BF16 bytes in HBM to the chunk payloads of an lmz archive.
// The reference does all of this on the CPU (lmz/codec.py:914-1009 encode_chunk); the plane
// coder itself is k_encode (encode_kernel.cuh).
//
//   k_split_bf16    every chunk into its exponent plane and its sign/mantissa plane
//                   (lmz/native/lmzcore.c:430-437), the two planes of a chunk back to back
//   k_frame_decide  per chunk: which coded planes pay (a stream must save max(1024, n >> 8)
//                   bytes, lmz/codec.py:385-398), the chunk's codec, flags and payload length
//                   (a chunk with no coded plane, or one that would not shrink, is stored,
//                   lmz/codec.py:997-1003)
//   k_frame_pack    the payload bytes: two plane lengths, then each plane as its stream or as it is
//   k_crc32_chunks  zlib's crc32 of every chunk's plaintext (lmz/codec.py:931)
#pragma once
#include "chunk_kernels.cuh"
#include "encode_kernel.cuh"

namespace lmz {

constexpr uint32_t CODEC_ID_STORED = 0, CODEC_ID_BF16 = 3, METHOD_ID_RANS = 3;

struct FrameMeta {           // one per chunk, written by k_frame_decide (crc by k_crc32_chunks)
    uint32_t clen, codec, flags, crc;
};

__device__ __forceinline__ uint32_t chunk_bytes_of(uint64_t nbytes, uint32_t chunk, uint32_t c)
{
    const uint64_t at = (uint64_t)c * chunk;
    return (uint32_t)min((uint64_t)chunk, nbytes - at);
}

// 256 threads per chunk; a thread turns 8 elements (16 bytes) into 8 + 8 plane bytes at a time.
__global__ void __launch_bounds__(256) k_split_bf16(const uint8_t *src, uint64_t nbytes, uint32_t chunk, uint8_t *planes)
{
    const uint32_t c = blockIdx.x, len = chunk_bytes_of(nbytes, chunk, c), n = len / 2;
    const uint8_t *s = src + (uint64_t)c * chunk;
    uint8_t *pa = planes + (uint64_t)c * chunk, *pb = pa + n;
    const bool fast = ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(pa) | reinterpret_cast<uintptr_t>(pb)) & 15u) == 0 &&
                      (n & 7u) == 0;
    if (fast) {
        for (uint32_t i = threadIdx.x * 8; i < n; i += 256 * 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(s + 2 * i));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t a[2] = {0, 0}, b[2] = {0, 0};
#pragma unroll
            for (int h = 0; h < 4; h++) {
                // two elements per word: exponent byte = bits 7..14, the other = sign over the low 7 bits
                const uint32_t lo = w[h] & 0xffffu, hi = w[h] >> 16;
                const uint32_t e0 = (lo >> 7) & 0xffu, e1 = (hi >> 7) & 0xffu;
                const uint32_t m0 = ((lo >> 8) & 0x80u) | (lo & 0x7fu), m1 = ((hi >> 8) & 0x80u) | (hi & 0x7fu);
                a[h >> 1] |= (e0 | (e1 << 8)) << (16 * (h & 1));
                b[h >> 1] |= (m0 | (m1 << 8)) << (16 * (h & 1));
            }
            *reinterpret_cast<uint2 *>(pa + i) = make_uint2(a[0], a[1]);
            *reinterpret_cast<uint2 *>(pb + i) = make_uint2(b[0], b[1]);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += 256) {
            const uint32_t w = (uint32_t)s[2 * i] | ((uint32_t)s[2 * i + 1] << 8);
            pa[i] = (uint8_t)((w >> 7) & 0xffu);
            pb[i] = (uint8_t)(((w >> 8) & 0x80u) | (w & 0x7fu));
        }
    }
}

__global__ void k_frame_decide(uint64_t nbytes, uint32_t chunk, uint32_t nchunks, const uint32_t *lens, FrameMeta *meta)
{
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= nchunks) return;
    const uint32_t len = chunk_bytes_of(nbytes, chunk, c), n = len / 2;
    const uint32_t gain = max(1024u, n >> 8);
    uint32_t total = 0, flags = 0;
    for (int p = 0; p < 2; p++) {
        const uint32_t coded = lens[2 * c + p];
        const bool keep = coded != 0 && coded + gain < n;
        total += keep ? coded : n;
        flags |= (keep ? METHOD_ID_RANS : 0u) << (2 * p);
    }
    const bool split = flags != 0 && total + 8 < len;
    meta[c].clen = split ? total + 8 : len;
    meta[c].codec = split ? CODEC_ID_BF16 : CODEC_ID_STORED;
    meta[c].flags = split ? flags : 0u;
}

// One CTA per chunk.  Streams end at the ends of their slots (k_encode's layout): full chunks
// use slots of `slot` bytes, the last, shorter chunk slots of `slot_tail` bytes after them.
__global__ void __launch_bounds__(256) k_frame_pack(const uint8_t *src, uint64_t nbytes, uint32_t chunk, const uint32_t *lens,
                                                    const FrameMeta *meta, const uint8_t *planes, const uint8_t *slots,
                                                    uint32_t slot, uint32_t slot_tail, uint32_t nfull,
                                                    const uint64_t *offs, uint8_t *out)
{
    const uint32_t c = blockIdx.x, len = chunk_bytes_of(nbytes, chunk, c), n = len / 2;
    uint8_t *d = out + offs[c];
    const FrameMeta m = meta[c];
    if (m.codec == CODEC_ID_STORED) {
        const uint8_t *s = src + (uint64_t)c * chunk;
        for (uint32_t i = threadIdx.x; i < len; i += 256) d[i] = s[i];
        return;
    }
    uint32_t plen[2];
    const uint8_t *from[2];
    for (int p = 0; p < 2; p++) {
        const bool coded = (m.flags >> (2 * p) & 3u) == METHOD_ID_RANS;
        plen[p] = coded ? lens[2 * c + p] : n;
        const uint8_t *slot_end = c < nfull ? slots + (uint64_t)(2 * c + p + 1) * slot
                                            : slots + (uint64_t)2 * nfull * slot + (uint64_t)(p + 1) * slot_tail;
        from[p] = coded ? slot_end - plen[p] : planes + (uint64_t)c * chunk + (uint64_t)p * n;
    }
    if (threadIdx.x < 8) {
        const uint32_t v = plen[threadIdx.x >> 2];
        d[threadIdx.x] = (uint8_t)(v >> (8 * (threadIdx.x & 3)));
    }
    for (uint32_t i = threadIdx.x; i < plen[0]; i += 256) d[8 + i] = from[0][i];
    for (uint32_t i = threadIdx.x; i < plen[1]; i += 256) d[8 + plen[0] + i] = from[1][i];
}

// crc32 of every chunk: 256 threads per chunk, each over its own contiguous run (table lookups
// through a 16-fold replicated copy of the slice tables, as k_finish), runs joined by
// x^(8 * bytes after the run) (crc.cuh).
__global__ void __launch_bounds__(256) k_crc32_chunks(const uint8_t *src, uint64_t nbytes, uint32_t chunk,
                                                      const CrcTables *tabs, FrameMeta *meta)
{
    constexpr int LOGR = 4;
    constexpr uint32_t TS = 1024u << LOGR;
    extern __shared__ __align__(16) uint8_t qsm[];
    __shared__ uint32_t part[8];
    const uint32_t tab0 = (smem_addr(qsm) + TS - 1) & ~(TS - 1);
    uint32_t *tw = reinterpret_cast<uint32_t *>(qsm + (tab0 - smem_addr(qsm)));
    for (uint32_t i = threadIdx.x; i < 4u * 256u << LOGR; i += 256) tw[i] = (&tabs->slice[0][0])[i >> LOGR];
    __syncthreads();
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t tl = tab0 + 4 * (lane & ((1u << LOGR) - 1));
    const uint32_t c = blockIdx.x, len = chunk_bytes_of(nbytes, chunk, c);
    const uint8_t *s = src + (uint64_t)c * chunk;
    // thread t takes bytes [t * run, (t + 1) * run), run a multiple of 4
    const uint32_t run = ((len + 255u) / 256u + 3u) & ~3u;
    const uint32_t lo = min(t * run, len), hi = min(lo + run, len);
    uint32_t acc = 0;
    uint32_t i = lo;
    for (; i + 4 <= hi; i += 4) {
        uint32_t w[1];
        load_words_nc<1>(s + i, w);
        acc = crc_feed4<LOGR>(tl, acc ^ w[0]);
    }
    for (; i < hi; i++) acc = (acc >> 8) ^ tabs->slice[0][(acc ^ s[i]) & 0xffu];
    // to the chunk's end, XOR over the chunk
    uint32_t v = crc_shift(tabs->x2, acc, len - hi);
#pragma unroll
    for (int d = 16; d; d >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0) part[warp] = v;
    __syncthreads();
    if (t == 0) {
        uint32_t r = 0;
        for (int w = 0; w < 8; w++) r ^= part[w];
        meta[c].crc = crc_shift(tabs->x2, 0xffffffffu, len) ^ r ^ 0xffffffffu;
    }
}

}  // namespace lmz
