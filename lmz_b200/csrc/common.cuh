// Shared definitions for the sm_100a lmz decode library: format constants,
// job descriptors handed over by the host, status codes, and the thin PTX
// wrappers (mbarrier + CTA-local bulk async copy) the kernels stage their
// compressed input with.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace lmz {

// ---- stream format (reference: lmz/native/lmzcore.c:755-767) ---------------
constexpr uint32_t PROB_BITS = 12;
constexpr uint32_t PROB_SCALE = 1u << PROB_BITS;
constexpr uint32_t RANS_LOW = 1u << 16;
constexpr uint32_t NLANES = 8;        // interleaved states per stream
constexpr uint32_t HDR_BYTES = 516;   // 'R','1',0,0 + 256 x u16 frequencies
constexpr uint32_t STATE_BYTES = 32;  // 8 x u32 initial states

// ---- kernel geometry --------------------------------------------------------
constexpr uint32_t TILE = 128;        // symbols one 8-lane group retires per tile (16 steps)
constexpr uint32_t SLOT = 256;        // bytes per bulk copy
constexpr uint32_t NSLOT = 4;         // slots in one group's input ring
constexpr uint32_t RING = SLOT * NSLOT;
constexpr uint32_t PAD_BYTES = 576;   // readable slack owed after the last stream
constexpr uint32_t WAIT_LIMIT = 1u << 22;   // bounded mbarrier polls before giving up

// ---- per-stream status words -------------------------------------------------
constexpr uint32_t ST_OK = 0;
constexpr uint32_t ST_BAD_HEADER = 1;   // magic, frequency sum or minimum length
constexpr uint32_t ST_OVERRUN = 2;      // a refill was needed past the stream's end
constexpr uint32_t ST_TIMEOUT = 3;      // an input copy never landed (bounded wait ran out)
constexpr uint32_t ST_BAD_SHAPE = 4;    // lengths in a payload disagree with the record
constexpr uint32_t ST_BAD_CRC = 5;      // decoded chunk does not match the record's crc32
constexpr uint32_t ST_SLACK = 0x100;    // soft: final states != 2^16 or cursor != length

// One rANS stream to decode.  Written by the host planner (numpy structured
// array with the same layout) or by a device planning kernel.
struct StreamJob {
    uint64_t src_off;   // stream start, bytes from the source base
    uint64_t dst_off;   // first output byte, bytes from the destination base
    uint32_t src_len;   // stream length in bytes
    uint32_t n;         // symbols to produce
    uint32_t flags;     // reserved
    uint32_t aux;       // reserved
};
static_assert(sizeof(StreamJob) == 32, "StreamJob layout is shared with the host");

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Bytes of dynamic shared memory this launch was given.
__device__ __forceinline__ uint32_t dynamic_smem_bytes()
{
    uint32_t v;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(v));
    return v;
}

// Loads and stores by 32-bit shared-space address (no generic-pointer arithmetic).
__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8_1(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1+1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_u8(uint32_t a, uint32_t v)
{
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 lds_u128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_u16(uint32_t a, uint32_t v)
{
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_u32(uint32_t a, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ uint2 lds_u64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count)
                 : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: false when the phase did not complete within WAIT_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// CTA-local 1-D bulk copy global -> shared, completion counted on `bar`.
// Source, destination and size are all multiples of 16 bytes.  No multicast:
// the destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

}  // namespace lmz
