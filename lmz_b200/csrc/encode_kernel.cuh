// k_encode: the 8-lane interleaved rANS *encoder* for a batch of byte planes, the
// inverse of the batch decode.  Stream i is byte-identical to what the reference's
// CPU encoder writes for plane i with the plane's own histogram
// (lmz/native/lmzcore.c:882-937 rans_normalize, :808-841 rans_enc_put, :958-979
// rans_enc_body, :1318-1383 rans_encode_impl).
//
// One 8-lane group per stream, four streams per warp:
//   1. histogram of the plane in shared memory;
//   2. the reference's normalisation to 12-bit frequencies, by the whole warp for one
//      stream at a time (floor(c * 4096 / n) at least 1, the remainder given to the most
//      common symbol, an overshoot taken back from the largest frequency, first index
//      winning every tie);
//   3. the walk from the last symbol to the first.  Lane k owns state k.  Within a group
//      of eight symbols the reference visits lane 7 first, so a lane's 16-bit word lands
//      below those of the lanes above it: one vote and a popcount give its place.  Words
//      go into a 512-byte ring that mirrors the stream's slot in global memory modulo 512
//      and leave it in whole, aligned 128-byte pieces;
//   4. the eight states (lane 0 lowest) and the 516-byte table in front of the words.
// The stream ends exactly at the end of its slot; its length is reported, so it starts
// at slot_bytes - length.
#pragma once
#include "common.cuh"

namespace lmz {

struct EncodeArgs {
    const uint8_t *src;     // nstr planes of `plane` bytes, back to back
    uint32_t plane;
    uint32_t nstr;
    uint8_t *slots;         // nstr slots of slot_bytes each, 512-byte aligned
    uint32_t slot_bytes;    // multiple of 512, at least HDR + 32 + 2 * plane
    uint32_t *lengths;      // per stream: bytes written at the end of its slot, 0 = failed
};

constexpr uint32_t E_RING = 512;
constexpr uint32_t E_GROUP_BYTES = 1024 /*counts, then f | start << 16*/ + 1024 /*reciprocals*/ + E_RING + 128 /*input tile*/;
__host__ __device__ constexpr uint32_t encode_smem_bytes(int warps) { return warps * 4 * E_GROUP_BYTES; }
__host__ __device__ constexpr uint32_t encode_slot_bytes(uint32_t plane)
{
    return (HDR_BYTES + STATE_BYTES + 2u * plane + 64u + 511u) & ~511u;
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) k_encode(EncodeArgs a)
{
    extern __shared__ __align__(512) uint8_t esm[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t k = lane & 7u, g = lane >> 3, gi = warp * 4 + g;
    uint8_t *gp = esm + (size_t)gi * E_GROUP_BYTES;
    uint32_t *tab = reinterpret_cast<uint32_t *>(gp);
    uint32_t *rcp = tab + 256;
    uint8_t *ring = gp + 2048;
    uint8_t *tile = ring + E_RING;
    const uint32_t ring_sa = smem_addr(ring);

    const uint32_t job = (blockIdx.x * WARPS + warp) * 4 + g;
    const bool have = job < a.nstr;
    const uint32_t n = have ? a.plane : 0;
    const uint8_t *src = a.src + (size_t)job * a.plane;

    // ---- 1. histogram ------------------------------------------------------------------
    for (uint32_t i = k; i < 256; i += 8) tab[i] = 0;
    __syncwarp();
    {
        // bytes up to the first 16-byte boundary, whole 16-byte units (two per lane in
        // flight), then the tail
        const uint32_t head = min(n, (uint32_t)((16u - (reinterpret_cast<uintptr_t>(src) & 15u)) & 15u));
        const uint32_t units = (n - head) / 16;
        for (uint32_t i = k; i < head; i += 8) atomicAdd(&tab[src[i]], 1u);
        const uint4 *u4 = reinterpret_cast<const uint4 *>(src + head);
        auto count16 = [&](const uint4 &v) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                atomicAdd(&tab[w[j] & 0xffu], 1u);
                atomicAdd(&tab[(w[j] >> 8) & 0xffu], 1u);
                atomicAdd(&tab[(w[j] >> 16) & 0xffu], 1u);
                atomicAdd(&tab[w[j] >> 24], 1u);
            }
        };
        uint32_t u = k;
        for (; u + 8 < units; u += 16) {
            const uint4 v0 = __ldg(u4 + u), v1 = __ldg(u4 + u + 8);
            count16(v0);
            count16(v1);
        }
        for (; u < units; u += 8) count16(__ldg(u4 + u));
        for (uint32_t i = head + units * 16 + k; i < n; i += 8) atomicAdd(&tab[src[i]], 1u);
    }
    __syncwarp();

    // ---- 2. frequencies, one stream at a time by the whole warp ---------------------------
    bool ok = n != 0;
#pragma unroll 1
    for (uint32_t gg = 0; gg < 4; gg++) {
        const uint32_t nn = __shfl_sync(0xffffffffu, n, gg * 8);
        if (!nn) continue;
        uint32_t *t = reinterpret_cast<uint32_t *>(esm + (size_t)(warp * 4 + gg) * E_GROUP_BYTES);
        uint32_t c[8], f[8], sum = 0;
        uint64_t best = 0;                              // (count << 8) | (255 - symbol): first index wins
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t s = lane * 8 + j;
            c[j] = t[s];
            uint64_t q = c[j] ? (uint64_t)c[j] * PROB_SCALE / nn : 0;
            if (c[j] && q < 1) q = 1;
            if (q > PROB_SCALE) q = PROB_SCALE;
            f[j] = (uint32_t)q;
            sum += f[j];
            const uint64_t key = ((uint64_t)c[j] << 8) | (255u - s);
            if (c[j] && key > best) best = key;
        }
        sum = __reduce_add_sync(0xffffffffu, sum);
#pragma unroll
        for (int d = 16; d; d >>= 1) {
            const uint64_t o = __shfl_xor_sync(0xffffffffu, best, d);
            if (o > best) best = o;
        }
        const uint32_t top = 255u - (uint32_t)(best & 0xffu);
        bool good = true;
        if (sum < PROB_SCALE) {
            if (top / 8 == lane) {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if ((uint32_t)j == (top & 7u)) f[j] += PROB_SCALE - sum;
            }
        } else {
            uint32_t excess = sum - PROB_SCALE;
            for (uint32_t it = 0; excess && it < 512; it++) {
                uint32_t bk = 0;                        // (freq << 8) | (255 - symbol), freq > 1 only
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t key = (f[j] << 8) | (255u - (lane * 8 + j));
                    if (f[j] > 1 && key > bk) bk = key;
                }
                bk = __reduce_max_sync(0xffffffffu, bk);
                if (!bk) { good = false; break; }
                const uint32_t bi = 255u - (bk & 0xffu), bf = bk >> 8;
                const uint32_t take = bf - 1 < excess ? bf - 1 : excess;
                if (bi / 8 == lane) {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        if ((uint32_t)j == (bi & 7u)) f[j] -= take;
                }
                excess -= take;
            }
            if (excess) good = false;
        }
        // cumulative starts, then the tables the walk reads: f | start << 16 and floor((2^32-1)/f)
        uint32_t mine = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) mine += f[j];
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= (uint32_t)d) incl += v;
        }
        if (__shfl_sync(0xffffffffu, incl, 31) != PROB_SCALE) good = false;
        uint32_t start = incl - mine;
        uint32_t *r = t + 256;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t s = lane * 8 + j;
            if ((c[j] != 0) != (f[j] != 0)) good = false;
            t[s] = f[j] | (start << 16);
            r[s] = f[j] ? 0xffffffffu / f[j] : 0u;
            start += f[j];
        }
        good = __all_sync(0xffffffffu, good);
        if (!good && g == gg) ok = false;
    }
    __syncwarp();

    // ---- 3. the walk, last symbol first ---------------------------------------------------
    uint8_t *slot = a.slots + (size_t)job * a.slot_bytes;
    const uint32_t T = ok ? (n + 7) / 8 : 0;            // groups of eight symbols
    const uint32_t tiles = (T + 15) / 16;
    const uint32_t warp_tiles = __reduce_max_sync(0xffffffffu, tiles);
    uint32_t x = RANS_LOW, emitted = 0, flushed = 0;    // bytes, counted back from the slot's end
#pragma unroll 1
    for (uint32_t tt = warp_tiles; tt-- > 0;) {
        const bool mine_tile = tt < tiles;
        // this tile's 128 symbols into shared memory (lane k: bytes 16 k .. 16 k + 15)
        __syncwarp();
        if (mine_tile) {
            const uint8_t *tp = src + tt * 128 + 16 * k;
            if ((reinterpret_cast<uintptr_t>(tp) & 15u) == 0 && tt * 128 + 16 * k + 16 <= n) {
                *reinterpret_cast<uint4 *>(tile + 16 * k) = __ldg(reinterpret_cast<const uint4 *>(tp));
            } else {
#pragma unroll
                for (uint32_t j = 0; j < 16; j++) {
                    const uint32_t i = tt * 128 + 16 * k + j;
                    tile[16 * k + j] = i < n ? src[i] : 0;
                }
            }
        }
        __syncwarp();
#pragma unroll 4
        for (uint32_t s = 16; s-- > 0;) {
            const uint32_t i = tt * 128 + s * 8 + k;
            const bool active = mine_tile && i < n;
            const uint32_t sym = tile[s * 8 + k];
            const uint32_t e = tab[sym], f = e & 0xffffu, st = e >> 16;
            uint32_t v = x;
            const bool need = active && f < PROB_SCALE && v >= (f << 20);
            const uint32_t vote = (__ballot_sync(0xffffffffu, need) >> (8 * g)) & 0xffu;
            if (need) {
                const uint32_t before = emitted + 2 * __popc(vote >> (k + 1));   // lanes above go first
                sts_u16(ring_sa + ((0u - before - 2u) & (E_RING - 1)), v & 0xffffu);
                v >>= 16;
            }
            emitted += 2 * __popc(vote);
            if (active) {
                uint32_t q = __umulhi(v, rcp[sym]);
                uint32_t rem = v - q * f;
                if (rem >= f) { q++; rem -= f; }
                if (rem >= f) { q++; rem -= f; }
                x = v + st + q * (PROB_SCALE - f);
            }
        }
        // whole 128-byte pieces leave the ring (at most 127 + 256 bytes are ever pending)
        __syncwarp();
        while (flushed + 128 <= emitted) {
            const uint32_t at = flushed + 128;          // piece = [end - at, end - at + 128)
            const uint4 v = lds_u128(ring_sa + ((0u - at) & (E_RING - 1)) + 16 * k);
            *reinterpret_cast<uint4 *>(slot + a.slot_bytes - at + 16 * k) = v;
            flushed = at;
        }
    }
    __syncwarp();
    if (ok) {
        // the pending tail of the words, byte by byte
        for (uint32_t j = flushed + k; j < emitted; j += 8)
            slot[a.slot_bytes - 1 - j] = ring[(0u - 1u - j) & (E_RING - 1)];
        // ---- 4. states (lane 0 lowest) and the table, in front of the words -------------
        uint8_t *p = slot + a.slot_bytes - emitted - STATE_BYTES;
#pragma unroll
        for (int b = 0; b < 4; b++) p[4 * k + b] = (uint8_t)(x >> (8 * b));
        uint8_t *h = p - HDR_BYTES;
        if (k == 0) { h[0] = 'R'; h[1] = '1'; h[2] = 0; h[3] = 0; }
        for (uint32_t s = k; s < 256; s += 8) {
            const uint32_t f = tab[s] & 0xffffu;
            h[4 + 2 * s] = (uint8_t)f;
            h[5 + 2 * s] = (uint8_t)(f >> 8);
        }
    }
    if (have && k == 0) a.lengths[job] = ok ? HDR_BYTES + STATE_BYTES + emitted : 0u;
}

// Streams out of their slots into one buffer, stream i at offs[2 i] (the layout the batch
// decode reads): one CTA per stream.  offs[2 i + 1] must hold the length.
__global__ void k_pack_streams(const uint8_t *slots, uint32_t slot_bytes, const uint64_t *offs,
                               uint32_t nstr, uint8_t *out)
{
    const uint32_t i = blockIdx.x;
    if (i >= nstr) return;
    uint64_t len = offs[2 * i + 1];
    if (len > slot_bytes) len = slot_bytes;        // a stream never outgrows its slot
    const uint8_t *s = slots + (size_t)(i + 1) * slot_bytes - len;
    uint8_t *d = out + offs[2 * i];
    for (uint64_t j = threadIdx.x; j < len; j += blockDim.x) d[j] = s[j];
}

}  // namespace lmz
