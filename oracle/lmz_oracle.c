/*
 * CPU oracle for the lmz checkpoint-decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain scalar restatement of the arithmetic the reference's decoder
 * performs on an archive's byte-plane streams, written from the reference's
 * behaviour, one function per reference function, each citing the file:line it
 * follows.  It exists so the CUDA library's output can be compared with
 * something that (a) travels with this repository and (b) is simple enough to
 * audit.  Nothing in the product (the lmz_b200 package, the C-ABI library)
 * may link, import or call this file; only tests, the smoke check and the
 * benchmark's CPU-baseline leg do.
 *
 * Parity of this restatement is pinned three ways by the test-suite: against
 * streams and archives written by the reference's own encoder (committed
 * under tests/golden/), against the reference's compiled C core when it has
 * been built into oracle/_ref/ (see oracle/Makefile), and by exhaustive
 * round trips over the shapes the reference's own tests use.
 *
 * The small encoder at the bottom (normalise + backwards 8-state walk) is
 * here because parity inputs have to be *written* somewhere the reference's
 * Python cannot travel to; it must emit byte-for-byte what the reference's
 * portable encoder emits, and the tests hold it to that.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

enum {
    PROB_BITS = 12,
    PROB_SCALE = 1 << PROB_BITS,   /* lmz/native/lmzcore.c:755-756 */
    NLANES = 8,                    /* :766 RANS_STREAMS */
    HDR_BYTES = 516,               /* :767 magic(2) reserved(2) 256*u16 */
};
#define RANS_LOW (1u << 16)        /* :765 renormalisation floor */

ORC_API int orc_abi_version(void) { return 1; }

/* ------------------------------------------------------------------ helpers */

static uint32_t rd16(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }
static uint32_t rd32(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) |
           ((uint32_t)p[3] << 24);
}

/* ----------------------------------------------------------------- rANS decode */

/*
 * Decode with an explicit frequency table and the lane states starting at
 * `body`.  This is the common core of the per-stream form (table read from the
 * stream's own header) and of the shared-table form (table handed in; the
 * stream starts at its 8 states -- scratchpad/gpu/shared_enc.c:1-13).
 *
 * Semantics: lmz/native/lmzcore.c:1409-1530.  Symbol i is produced by lane
 * i & 7; a lane whose state falls below 2^16 pulls the next little-endian
 * u16 from the shared cursor, lanes refilling in lane order within a group of
 * eight.  A refill that would read past `len` is malformed (-1), exactly as
 * rans_dec_advance_safe (:858-872) reports it; the reference's fast loop only
 * runs while 16 bytes remain so it never reads past the end either, which
 * makes this byte-at-a-time restatement equivalent on every input.
 *
 * `end_state` (may be NULL) receives the 8 final states then the final cursor
 * offset relative to `body`, for the end-of-stream invariant tests.
 */
static int decode_core(const uint16_t *freqs, const uint8_t *body, size_t body_len,
                       uint8_t *dst, size_t n, uint32_t *end_state)
{
    /* slot -> symbol, and per-symbol start; the reference packs these into one
     * 32-bit LUT entry (:1432-1441), which is a speed matter only. */
    static __thread uint8_t slot_sym[PROB_SCALE];
    uint32_t start[257];
    uint32_t acc = 0;
    for (int s = 0; s < 256; s++) {
        start[s] = acc;
        uint32_t f = freqs[s];
        if (acc + f > PROB_SCALE) return -1;
        for (uint32_t j = 0; j < f; j++) slot_sym[acc + j] = (uint8_t)s;
        acc += f;
    }
    if (acc != PROB_SCALE) return -1;            /* :1421, :1442 */
    if (body_len < 4 * NLANES) return -1;        /* :1412 */

    uint32_t x[NLANES];
    for (int k = 0; k < NLANES; k++) x[k] = rd32(body + 4 * k);   /* :843-849 */
    size_t p = 4 * NLANES;

    for (size_t i = 0; i < n; i++) {
        int k = (int)(i & (NLANES - 1));
        uint32_t slot = x[k] & (PROB_SCALE - 1);
        uint32_t s = slot_sym[slot];
        dst[i] = (uint8_t)s;
        uint32_t v = (uint32_t)freqs[s] * (x[k] >> PROB_BITS) + slot - start[s];  /* :866 */
        if (v < RANS_LOW) {
            if (p + 2 > body_len) return -1;     /* :869 */
            v = (v << 16) | rd16(body + p);
            p += 2;
        }
        x[k] = v;
    }
    if (end_state) {
        for (int k = 0; k < NLANES; k++) end_state[k] = x[k];
        end_state[NLANES] = (uint32_t)p;
    }
    return 0;
}

/* lmz_rans_decode, lmz/native/lmzcore.c:1409-1530. 0 ok, -1 malformed. */
ORC_API int orc_rans_decode_ex(const uint8_t *src, size_t src_len, uint8_t *dst,
                               size_t n, uint32_t *end_state)
{
    if (n == 0) return src_len == 0 ? 0 : -1;                    /* :1411 */
    if (src_len < HDR_BYTES + 4 * NLANES) return -1;             /* :1412 */
    if (src[0] != 'R' || src[1] != '1') return -1;               /* :1413 */
    uint16_t freqs[256];
    for (int s = 0; s < 256; s++) freqs[s] = (uint16_t)rd16(src + 4 + 2 * s);
    int rc = decode_core(freqs, src + HDR_BYTES, src_len - HDR_BYTES, dst, n, end_state);
    if (rc == 0 && end_state) end_state[NLANES] += HDR_BYTES;
    return rc;
}

ORC_API int orc_rans_decode(const uint8_t *src, size_t src_len, uint8_t *dst, size_t n)
{
    return orc_rans_decode_ex(src, src_len, dst, n, NULL);
}

/* Shared-table stream: `hdr` is the 516-byte table, `src` starts at the lane
 * states.  Equivalent to prepending hdr to src and calling orc_rans_decode
 * (scratchpad/gpu/prep_shared.py:101-112 verifies its streams that way). */
ORC_API int orc_rans_decode_shared(const uint8_t *hdr, const uint8_t *src, size_t src_len,
                                   uint8_t *dst, size_t n)
{
    if (n == 0) return 0;
    if (hdr[0] != 'R' || hdr[1] != '1') return -1;
    uint16_t freqs[256];
    for (int s = 0; s < 256; s++) freqs[s] = (uint16_t)rd16(hdr + 4 + 2 * s);
    return decode_core(freqs, src, src_len, dst, n, NULL);
}

/* --------------------------------------------------------- planes and fields */

/* lmz_hist, lmz/native/lmzcore.c:385-397. */
ORC_API void orc_hist(const uint8_t *p, size_t n, uint64_t *hist)
{
    memset(hist, 0, 256 * sizeof *hist);
    for (size_t i = 0; i < n; i++) hist[p[i]]++;
}

/* split_bf16_scalar, lmz/native/lmzcore.c:430-437: plane A is the 8 exponent
 * bits, plane B the sign in bit 7 over the 7 mantissa bits. */
ORC_API void orc_split_bf16(const uint8_t *src, uint8_t *pa, uint8_t *pb, size_t nelem)
{
    for (size_t i = 0; i < nelem; i++) {
        uint32_t w = rd16(src + 2 * i);
        pa[i] = (uint8_t)((w >> 7) & 0xFF);
        pb[i] = (uint8_t)(((w >> 8) & 0x80) | (w & 0x7F));
    }
}

/* merge_bf16_scalar, lmz/native/lmzcore.c:439-447. */
ORC_API void orc_merge_bf16(const uint8_t *pa, const uint8_t *pb, uint8_t *dst, size_t nelem)
{
    for (size_t i = 0; i < nelem; i++) {
        uint32_t a = pa[i], b = pb[i];
        uint32_t w = ((b & 0x80u) << 8) | (a << 7) | (b & 0x7Fu);
        dst[2 * i] = (uint8_t)(w & 0xFF);
        dst[2 * i + 1] = (uint8_t)(w >> 8);
    }
}

/* Byte-plane split: plane j holds byte j of every element.  The reference
 * reaches the same layout by recursive halving (lmz/native/lmzcore.c:252-347);
 * the result, out[i*esize + j] = plane_j[i], is what its tests pin. */
ORC_API void orc_split_planes(const uint8_t *src, uint8_t *out, size_t nelem, size_t esize)
{
    for (size_t i = 0; i < nelem; i++)
        for (size_t j = 0; j < esize; j++) out[j * nelem + i] = src[i * esize + j];
}

/* lmz_merge_planes, lmz/native/lmzcore.c:338-347 (via merge_rec :289-318). */
ORC_API void orc_merge_planes(const uint8_t *const *planes, uint8_t *dst, size_t nelem,
                              size_t esize)
{
    for (size_t i = 0; i < nelem; i++)
        for (size_t j = 0; j < esize; j++) dst[i * esize + j] = planes[j][i];
}

/* lmz_xor, lmz/native/lmzcore.c:233-245. */
ORC_API void orc_xor(const uint8_t *a, const uint8_t *b, size_t n, uint8_t *out)
{
    for (size_t i = 0; i < n; i++) out[i] = (uint8_t)(a[i] ^ b[i]);
}

/* CRC-32 as zlib.crc32 computes it (reflected 0xEDB88320, init and final
 * xor 0xFFFFFFFF); the reference checks chunks with it at
 * lmz/codec.py:931,1191-1194,1227-1229. */
ORC_API uint32_t orc_crc32(uint32_t crc, const uint8_t *p, size_t n)
{
    static uint32_t table[256];
    static int ready;
    if (!ready) {
        for (uint32_t i = 0; i < 256; i++) {
            uint32_t c = i;
            for (int k = 0; k < 8; k++) c = (c >> 1) ^ (0xEDB88320u & (0u - (c & 1u)));
            table[i] = c;
        }
        ready = 1;
    }
    crc = ~crc;
    for (size_t i = 0; i < n; i++) crc = table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
    return ~crc;
}

/* ------------------------------------------------------ exponent conditioning */

/* lmz_bucket_lut, lmz/native/lmzcore.c:525-543: contiguous equal-mass buckets
 * over the alphabet; 64-bit products, as there. */
ORC_API int orc_bucket_lut(const uint64_t *hist, size_t k, uint8_t *lut)
{
    if (k == 0 || k > 32) return -1;
    uint64_t total = 0;
    for (int s = 0; s < 256; s++) total += hist[s];
    if (total == 0) {
        memset(lut, 0, 256);
        return 0;
    }
    uint64_t acc = 0, b = 0;
    for (int s = 0; s < 256; s++) {
        lut[s] = (uint8_t)b;
        acc += hist[s];
        while (b + 1 < k && acc * k >= (b + 1) * total) b++;
    }
    return 0;
}

/* bucket_counts, lmz/kernels.py:481-486. */
ORC_API void orc_bucket_counts(const uint64_t *hist, const uint8_t *lut, size_t k,
                               uint64_t *counts)
{
    for (size_t b = 0; b < k; b++) counts[b] = 0;
    for (int s = 0; s < 256; s++) counts[lut[s]] += hist[s];
}

/* lmz_bucket_partition, lmz/native/lmzcore.c:552-609 (stable per bucket). */
ORC_API int orc_bucket_partition(const uint8_t *ctx, const uint8_t *val, size_t n,
                                 const uint8_t *lut, size_t k, uint8_t *out,
                                 uint64_t *counts)
{
    if (k == 0 || k > 32) return -1;
    uint64_t hist[256];
    orc_hist(ctx, n, hist);
    orc_bucket_counts(hist, lut, k, counts);
    uint8_t *cur[32];
    uint8_t *p = out;
    for (size_t b = 0; b < k; b++) {
        cur[b] = p;
        p += counts[b];
    }
    for (size_t i = 0; i < n; i++) *cur[lut[ctx[i]]]++ = val[i];
    return 0;
}

/* lmz_bucket_unpartition, lmz/native/lmzcore.c:614-641. */
ORC_API int orc_bucket_unpartition(const uint8_t *ctx, const uint8_t *const *segs, size_t n,
                                   const uint8_t *lut, size_t k, uint8_t *val_out)
{
    if (k == 0 || k > 32) return -1;
    const uint8_t *cur[32];
    for (size_t b = 0; b < k; b++) cur[b] = segs[b];
    for (size_t i = 0; i < n; i++) val_out[i] = *cur[lut[ctx[i]]]++;
    return 0;
}

/* ------------------------------------------------------ whole-chunk plane decode */

/*
 * lmz_decode_planes, lmz/native/lmzcore.c:1553-1598: `nplanes` u32 lengths,
 * the planes back to back, plane k coded by method (methods >> 2k) & 3 where
 * 0 is stored and 3 is rANS.  Returns 0, -1 (malformed) or -2 (a plane coded
 * some other way, which the caller decodes elsewhere).  `scratch` must hold
 * nplanes * nelem bytes.
 */
ORC_API int orc_decode_planes(const uint8_t *payload, size_t plen, size_t nplanes,
                              size_t nelem, uint32_t methods, int bf16, uint8_t *dst,
                              uint8_t *scratch)
{
    if (nplanes == 0 || nplanes > 16 || nelem == 0) return -1;
    if (bf16 && nplanes != 2) return -1;
    size_t hdr = 4 * nplanes;
    if (plen < hdr) return -1;
    uint32_t lens[16];
    size_t total = hdr;
    for (size_t k = 0; k < nplanes; k++) {
        lens[k] = rd32(payload + 4 * k);
        total += lens[k];
        if (total > plen) return -1;
    }
    const uint8_t *p = payload + hdr;
    const uint8_t *planes[16];
    for (size_t k = 0; k < nplanes; k++) {
        uint32_t m = (methods >> (2 * k)) & 3u;
        if (m == 0) {
            if (lens[k] != nelem) return -1;
            planes[k] = p;
        } else if (m == 3) {
            uint8_t *d = scratch + k * nelem;
            if (orc_rans_decode(p, lens[k], d, nelem) != 0) return -1;
            planes[k] = d;
        } else {
            return -2;
        }
        p += lens[k];
    }
    if (bf16) orc_merge_bf16(planes[0], planes[1], dst, nelem);
    else orc_merge_planes(planes, dst, nelem, nplanes);
    return 0;
}

/* ------------------------------------------------------------------ encoder */

/* rans_normalize, lmz/native/lmzcore.c:882-937: counts -> 12-bit frequencies
 * summing to 4096, no occurring symbol at zero. */
ORC_API int orc_rans_normalize(const uint64_t *counts, uint16_t *freqs)
{
    uint64_t total = 0;
    for (int i = 0; i < 256; i++) total += counts[i];
    if (total == 0) return -1;
    uint32_t sum = 0;
    int top = -1;
    uint64_t top_count = 0;
    for (int i = 0; i < 256; i++) {
        freqs[i] = 0;
        if (!counts[i]) continue;
        uint64_t f = counts[i] * PROB_SCALE / total;
        if (f < 1) f = 1;
        if (f > PROB_SCALE) f = PROB_SCALE;
        freqs[i] = (uint16_t)f;
        sum += (uint32_t)f;
        if (counts[i] > top_count) {
            top_count = counts[i];
            top = i;
        }
    }
    if (top < 0) return -1;
    if (sum < PROB_SCALE) {
        freqs[top] = (uint16_t)(freqs[top] + (PROB_SCALE - sum));
    } else {
        /* overshoot is taken back from the currently largest frequency, first
         * index winning ties, never below one (:912-925) */
        uint32_t excess = sum - PROB_SCALE;
        while (excess) {
            int bi = -1;
            uint32_t bf = 1;
            for (int i = 0; i < 256; i++)
                if (freqs[i] > bf) {
                    bf = freqs[i];
                    bi = i;
                }
            if (bi < 0) return -1;
            uint32_t take = bf - 1 < excess ? bf - 1 : excess;
            freqs[bi] = (uint16_t)(freqs[bi] - take);
            excess -= take;
        }
    }
    for (int i = 0; i < 256; i++)
        if ((counts[i] != 0) != (freqs[i] != 0)) return -1;
    return 0;
}

ORC_API size_t orc_rans_bound(size_t n)      /* lmz/native/lmzcore.c:949-954 */
{
    return HDR_BYTES + 2 * n + 4 * NLANES + 64;
}

/* One encoder step, rans_enc_put lmz/native/lmzcore.c:808-841: emit the low
 * 16 bits when the state would overflow the symbol's bound, then
 * x = (x / f) * 4096 + (x % f) + start, written the reference's way as
 * x + start + (x / f) * (4096 - f). */
static void enc_put(uint32_t *x, uint8_t **pp, uint32_t start, uint32_t f)
{
    uint32_t v = *x;
    uint64_t bound = ((uint64_t)(RANS_LOW >> PROB_BITS) << 16) * f;
    if (v >= bound) {
        uint8_t *p = *pp - 2;
        p[0] = (uint8_t)(v & 0xFF);
        p[1] = (uint8_t)((v >> 8) & 0xFF);
        *pp = p;
        v >>= 16;
    }
    *x = v + start + (v / f) * (PROB_SCALE - f);
}

/* Body walk shared by both stream layouts: rans_enc_body
 * lmz/native/lmzcore.c:958-979 (ragged tail first, then whole groups of eight
 * from lane 7 down to lane 0, then the eight states flushed lane 7 first so
 * lane 0's state ends up lowest in memory). Returns where the coded bytes begin. */
static uint8_t *enc_body(const uint8_t *src, size_t n, uint8_t *end, const uint16_t *freqs)
{
    uint32_t start[256], acc = 0;
    for (int s = 0; s < 256; s++) {
        start[s] = acc;
        acc += freqs[s];
    }
    uint32_t x[NLANES];
    for (int k = 0; k < NLANES; k++) x[k] = RANS_LOW;
    uint8_t *p = end;
    size_t i = n;
    while (i > 0) {
        i--;
        enc_put(&x[i & (NLANES - 1)], &p, start[src[i]], freqs[src[i]]);
    }
    for (int k = NLANES - 1; k >= 0; k--) {
        p -= 4;
        p[0] = (uint8_t)x[k];
        p[1] = (uint8_t)(x[k] >> 8);
        p[2] = (uint8_t)(x[k] >> 16);
        p[3] = (uint8_t)(x[k] >> 24);
    }
    return p;
}

/* rans_encode_impl, lmz/native/lmzcore.c:1318-1383 (portable path). `counts`
 * may be NULL to count here. Returns the stream length or -1. */
ORC_API long orc_rans_encode(const uint8_t *src, size_t n, uint8_t *dst, size_t cap,
                             const uint64_t *counts)
{
    if (n == 0 || cap < orc_rans_bound(n)) return -1;
    uint64_t own[256];
    if (!counts) {
        orc_hist(src, n, own);
        counts = own;
    } else {
        uint64_t total = 0;
        for (int i = 0; i < 256; i++) total += counts[i];
        if (total != n) {
            orc_hist(src, n, own);
            counts = own;
        }
    }
    uint16_t freqs[256];
    if (orc_rans_normalize(counts, freqs) != 0) return -1;
    uint8_t *end = dst + cap;
    uint8_t *p = enc_body(src, n, end, freqs);
    size_t coded = (size_t)(end - p);
    dst[0] = 'R';
    dst[1] = '1';
    dst[2] = dst[3] = 0;
    for (int s = 0; s < 256; s++) {
        dst[4 + 2 * s] = (uint8_t)(freqs[s] & 0xFF);
        dst[5 + 2 * s] = (uint8_t)(freqs[s] >> 8);
    }
    memmove(dst + HDR_BYTES, p, coded);
    return (long)(HDR_BYTES + coded);
}

/* lmzx_encode_shared, scratchpad/gpu/shared_enc.c:96-124: code against a
 * caller-supplied table; the stream is [8 states][coded bytes]. -2 when the
 * table does not sum to 4096, -3 when it cannot represent a symbol of `src`. */
ORC_API long orc_rans_encode_shared(const uint8_t *src, size_t n, const uint16_t *freqs,
                                    uint8_t *dst, size_t cap)
{
    uint32_t sum = 0;
    for (int s = 0; s < 256; s++) sum += freqs[s];
    if (sum != PROB_SCALE) return -2;
    for (size_t i = 0; i < n; i++)
        if (!freqs[src[i]]) return -3;
    if (cap < 2 * n + 4 * NLANES) return -1;
    uint8_t *end = dst + cap;
    uint8_t *p = enc_body(src, n, end, freqs);
    size_t coded = (size_t)(end - p);
    memmove(dst, p, coded);
    return (long)coded;
}
