// CRC-32 (zlib / ISO-HDLC, reflected 0xEDB88320) for chunks decoded in pieces.
//
// The reference checks every chunk with zlib.crc32 (lmz/codec.py:931,
// 1191-1194, 1227-1229).  On the GPU a chunk is produced by many threads, so
// the checksum is assembled from linear parts:
//
//   R(D)      state after feeding D from state 0, no final xor   (linear in D)
//   shift(s,n) state after feeding n zero bytes from state s = s * x^(8n) mod P
//   R(A|B)    = shift(R(A), |B|) ^ R(B)
//   crc32(D)  = shift(0xFFFFFFFF, |D|) ^ R(D) ^ 0xFFFFFFFF
//
// Polynomial arithmetic follows zlib's published crc32_combine construction
// (multiplication modulo P on bit-reflected 32-bit values, powers of x by
// repeated squaring).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace lmz {

constexpr uint32_t CRC_POLY = 0xEDB88320u;

// a * b mod P, bit-reflected representation (bit 31 is x^0).
__host__ __device__ inline uint32_t crc_mulmod(uint32_t a, uint32_t b)
{
    uint32_t p = 0;
    for (int i = 0; i < 32; i++) {
        if (a & (0x80000000u >> i)) p ^= b;
        b = (b >> 1) ^ (CRC_POLY & (0u - (b & 1u)));
    }
    return p;
}

struct CrcTables {
    uint32_t slice[4][256];   // slice-by-4 byte tables
    uint32_t adv[4][256];     // advance a state by ADV_BYTES zero bytes, per state byte
    uint32_t lane_mul[256];   // x^(8 * 16 * (255 - t)): thread t's unit to the row's end
    uint32_t x2[32];          // x^(2^k)
    uint32_t adv_row[4][256]; // advance by a 256-byte group row minus one 32-byte lane unit
    uint32_t lane_mul8[8];    // x^(8 * 32 * (7 - k)): lane k's unit to the group row's end
    uint32_t run_mul[256];    // x^(8 * 256 * (255 - t)): thread t's 256-byte run to the piece's end
    uint32_t adv_row4[4][256];// advance by a 512-byte group row minus one 64-byte lane unit (4-byte elements)
    uint32_t lane_mul8_4[8];  // x^(8 * 64 * (7 - k))
    uint32_t mul_row[4][256]; // multiply a state by x^(8 * 256), one 256-byte group row, per state byte
    uint32_t word_mul[8][8];  // x^(32 * (64 - 8k - i)): word i of lane k's 32-byte unit to the row's end
    uint32_t mul_row512[4][256];  // multiply a state by x^(8 * 512): one 512-byte warp row (k_cond_finish)
    uint32_t word_mul512[32][4];  // x^(32 * (128 - 4l - i)): word i of lane l's 16-byte unit to that row's end
    uint32_t warp_mul8k[8];       // x^(8 * 8192 * (7 - w)): warp w's 8 KiB run to the piece's end
    uint32_t word_mul16[16][4];   // x^(32 * (64 - 4j - i)): word i of the j-th 16-byte unit of a 256-byte row to the row's end (delta sink)
    uint32_t mul_row4096[4][256]; // multiply a state by x^(8 * 4096): one row of a piece (k_finish)
    uint32_t mul_gap1984[4][256]; // multiply a state by x^(8 * 1984): from the end of a lane's 64 bytes of one
                                  // 2 KiB warp block to the start of its 64 bytes of the next (k_cond_finish)
    uint32_t lane_mul64[32];      // x^(8 * 64 * (31 - l)): the end of lane l's 64 bytes to the end of the block
};

// Rows of the piece layout: 256 threads x 16 bytes.
constexpr uint32_t ROW_BYTES = 4096;
constexpr uint32_t PIECE_BYTES = 65536;
constexpr uint32_t ADV_BYTES = ROW_BYTES - 16;

// x^e mod P for any exponent (x has order dividing 2^32 - 1, so x2[] wraps).
__host__ __device__ inline uint32_t crc_xpow(const uint32_t *x2, uint64_t e)
{
    uint32_t p = 0x80000000u;
    for (int k = 0; e; e >>= 1, k++)
        if (e & 1) p = crc_mulmod(x2[k & 31], p);
    return p;
}

// State after feeding n zero bytes.
__host__ __device__ inline uint32_t crc_shift(const uint32_t *x2, uint32_t s, uint64_t n)
{
    return crc_mulmod(crc_xpow(x2, 8 * n), s);
}

// Inverse of crc_shift: the state that n zero bytes would turn into s.
__host__ __device__ inline uint32_t crc_unshift(const uint32_t *x2, uint32_t s, uint64_t n)
{
    const uint64_t M = 0xFFFFFFFFull;
    uint64_t e = (8 * n) % M;
    return crc_mulmod(crc_xpow(x2, (M - e) % M), s);
}

inline void crc_build_tables(CrcTables &t)
{
    for (uint32_t i = 0; i < 256; i++) {
        uint32_t c = i;
        for (int k = 0; k < 8; k++) c = (c >> 1) ^ (CRC_POLY & (0u - (c & 1u)));
        t.slice[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; i++)
        for (int j = 1; j < 4; j++)
            t.slice[j][i] = (t.slice[j - 1][i] >> 8) ^ t.slice[0][t.slice[j - 1][i] & 0xff];
    uint32_t p = 0x40000000u;   // x^1
    t.x2[0] = p;
    for (int k = 1; k < 32; k++) t.x2[k] = p = crc_mulmod(p, p);
    uint32_t adv = crc_xpow(t.x2, 8ull * ADV_BYTES);
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.adv[j][i] = crc_mulmod(adv, i << (8 * j));
    for (uint32_t th = 0; th < 256; th++) t.lane_mul[th] = crc_xpow(t.x2, 8ull * 16 * (255 - th));
    uint32_t adv2 = crc_xpow(t.x2, 8ull * (256 - 32));
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.adv_row[j][i] = crc_mulmod(adv2, i << (8 * j));
    for (uint32_t k = 0; k < 8; k++) t.lane_mul8[k] = crc_xpow(t.x2, 8ull * 32 * (7 - k));
    for (uint32_t th = 0; th < 256; th++) t.run_mul[th] = crc_xpow(t.x2, 8ull * 256 * (255 - th));
    uint32_t adv4 = crc_xpow(t.x2, 8ull * (512 - 64));
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.adv_row4[j][i] = crc_mulmod(adv4, i << (8 * j));
    for (uint32_t k = 0; k < 8; k++) t.lane_mul8_4[k] = crc_xpow(t.x2, 8ull * 64 * (7 - k));
    uint32_t row = crc_xpow(t.x2, 8ull * 256);
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.mul_row[j][i] = crc_mulmod(row, i << (8 * j));
    for (uint32_t k = 0; k < 8; k++)
        for (uint32_t i = 0; i < 8; i++) t.word_mul[k][i] = crc_xpow(t.x2, 32ull * (64 - 8 * k - i));
    uint32_t row512 = crc_xpow(t.x2, 8ull * 512);
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.mul_row512[j][i] = crc_mulmod(row512, i << (8 * j));
    for (uint32_t l = 0; l < 32; l++)
        for (uint32_t i = 0; i < 4; i++) t.word_mul512[l][i] = crc_xpow(t.x2, 32ull * (128 - 4 * l - i));
    for (uint32_t w = 0; w < 8; w++) t.warp_mul8k[w] = crc_xpow(t.x2, 8ull * 8192 * (7 - w));
    for (uint32_t j = 0; j < 16; j++)
        for (uint32_t i = 0; i < 4; i++) t.word_mul16[j][i] = crc_xpow(t.x2, 32ull * (64 - 4 * j - i));
    uint32_t row4096 = crc_xpow(t.x2, 8ull * ROW_BYTES);
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.mul_row4096[j][i] = crc_mulmod(row4096, i << (8 * j));
    uint32_t gap = crc_xpow(t.x2, 8ull * 1984);
    for (int j = 0; j < 4; j++)
        for (uint32_t i = 0; i < 256; i++) t.mul_gap1984[j][i] = crc_mulmod(gap, i << (8 * j));
    for (uint32_t l = 0; l < 32; l++) t.lane_mul64[l] = crc_xpow(t.x2, 8ull * 64 * (31 - l));
}

// Feed one little-endian 32-bit word: four table lookups.
__device__ __forceinline__ uint32_t crc_word(const uint32_t (*sl)[256], uint32_t s, uint32_t w)
{
    s ^= w;
    return sl[3][s & 0xff] ^ sl[2][(s >> 8) & 0xff] ^ sl[1][(s >> 16) & 0xff] ^ sl[0][s >> 24];
}

// Apply a per-state-byte linear map (the advance tables).
__device__ __forceinline__ uint32_t crc_apply(const uint32_t (*tb)[256], uint32_t s)
{
    return tb[0][s & 0xff] ^ tb[1][(s >> 8) & 0xff] ^ tb[2][(s >> 16) & 0xff] ^ tb[3][s >> 24];
}

}  // namespace lmz
