// C-ABI shared library: sm_100a decode of lmz rANS byte-plane streams.
//
// The first nine exports are the boundary the reference's Python binds
// (lmz/gpu/lmzgpu.cu:341-527, ctypes signatures at lmz/gpu/__init__.py:130-148)
// with the same names, argument meaning, return codes and error behaviour; the
// rest are additive entry points for whole-archive decode.  Declarations and
// the per-function contract live in include/lmz_b200.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/lmz_b200.h"
#include "rans_kernel.cuh"
#include "chunk_kernels.cuh"
#include "cond_kernels.cuh"
#include "fused_kernel.cuh"
#include "encode_kernel.cuh"
#include "save_kernels.cuh"

using namespace lmz;

#define API extern "C" __attribute__((visibility("default")))

// Why the last call on this thread failed (lmz_gpu_last_error).
static thread_local char g_err[256];

// Record a reason and hand back the code to return.
static int report(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

static int fail_msg(int rc, const char *what) { return report(rc, "%s", what); }

static int fail_cuda(const char *what, cudaError_t e)
{
    return report(LMZ_GPU_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

// A CUDA call inside a function that returns a code: leave with ECUDA when it fails.
#define CK(what, x)                                                                    \
    if (cudaError_t status_of_call = (x); status_of_call != cudaSuccess)               \
        return fail_cuda(what, status_of_call)

static int device_ready()
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) {
        cudaGetLastError();
        return fail_msg(LMZ_GPU_ENODEV, "no CUDA device");
    }
    return LMZ_GPU_OK;
}

// Kernels ask for more dynamic shared memory than the default 48 KiB; the
// opt-in is per device and is made once.
template <class K>
static int opt_in_smem(K kernel, uint32_t bytes, bool *done /* [64] by device */)
{
    int dev = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return LMZ_GPU_OK;
    CK("cudaFuncSetAttribute",
       cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return LMZ_GPU_OK;
}

constexpr int WARPS_NARROW = 4;    // 2 CTAs/SM: 32 streams resident
constexpr int WARPS_WIDE = 8;
// Batches at least this large are occupancy-bound and take the compact tables;
// smaller ones are latency-bound per stream and keep the shorter narrow lookup.
constexpr unsigned COMPACT_MIN_JOBS = 148 * 32 * 2;

template <int MODE, int WARPS>
static int launch_rans_mode(const RansArgs &a, cudaStream_t cs)
{
    static bool done[64];
    constexpr uint32_t shm = rans_smem_bytes<MODE>(WARPS);
    int rc = opt_in_smem(k_rans<MODE, WARPS>, shm, done);
    if (rc) return rc;
    unsigned blocks = (a.njobs + WARPS * 4 - 1) / (WARPS * 4);
    k_rans<MODE, WARPS><<<blocks, WARPS * 32, shm, cs>>>(a);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_rans", le);
    return LMZ_GPU_OK;
}

// k_stream takes all the shared memory one CTA may have and lays its tables out from
// both ends, counting on the window starting F_SMEM_BASE bytes in (what the
// driver reserves per CTA on this architecture).
static int stream_smem_ok()
{
    static int state[64];                       // 0 unknown, 1 good, -1 bad
    int dev = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail_msg(LMZ_GPU_EUNSUPPORTED, "device index out of range");
    if (state[dev] == 0) {
        int reserved = 0, optin = 0;
        CK("cudaDeviceGetAttribute", cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev));
        CK("cudaDeviceGetAttribute", cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        state[dev] = (reserved == (int)F_SMEM_BASE && optin >= (int)F_SMEM_DYN) ? 1 : -1;
    }
    if (state[dev] < 0)
        return fail_msg(LMZ_GPU_EUNSUPPORTED, "this GPU's shared memory per CTA is not the 1 KiB + 227 KiB k_stream is laid out for");
    return LMZ_GPU_OK;
}

// CFN = 128 is for streams the caller knows to have at most F_SMALL_LIVE live symbols;
// CFN = 0 is the per-stream wide table (12 streams per SM), CFN = -1 one wide table per CTA.
static int sm_count(int *out);

template <int SINK, bool CRC, int CFN, int WARPS_ = 0>
static int launch_stream(const StreamArgs &a0, cudaStream_t cs)
{
    if (a0.njobs == 0) return LMZ_GPU_OK;
    StreamArgs a = a0;
    constexpr int WARPS = WARPS_ ? WARPS_ : stream_warps(CFN, CRC, SINK);
    static bool done[64];
    int rc = stream_smem_ok();
    if (rc) return rc;
    // the shared-table instance needs little shared memory and runs two CTAs per SM
    constexpr bool PAIRED = CFN < 0 && SINK == SINK_BYTES;      // two CTAs per SM
    constexpr uint32_t shm = PAIRED ? 2u * F_WIDE_BYTES + WARPS * 4 * stream_group_bytes(CFN) : F_SMEM_DYN;
    rc = opt_in_smem(k_stream<SINK, CRC, WARPS, CFN>, shm, done);
    if (rc) return rc;
    constexpr bool DIRECT = stream_direct(CFN, WARPS);
    constexpr unsigned groups = DIRECT ? F_DIRECT_GROUPS : stream_groups(CFN, WARPS);
    unsigned per = groups;
    if (a.per_cta) {
        per = a.per_cta;          // the caller's job list is laid out for this many streams per CTA
    } else {
        // as many waves of CTAs as full CTAs would need, the streams spread evenly over them
        // (when the device holds the count, as if every job of the launch were of this class)
        int sms = 0;
        rc = sm_count(&sms);
        if (rc) return rc;
        const unsigned slots = (unsigned)sms * (PAIRED ? 2u : 1u);
        const unsigned waves = (a.njobs + slots * groups - 1) / (slots * groups);
        per = (a.njobs + waves * slots - 1) / (waves * slots);
        if (!DIRECT) per = (per + 3u) & ~3u;
        if (per > groups) per = groups;
    }
    a.per_cta = per;
    unsigned blocks = (a.njobs + per - 1) / per;
    k_stream<SINK, CRC, WARPS, CFN><<<blocks, WARPS * 32, shm, cs>>>(a);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_stream", le);
    return LMZ_GPU_OK;
}

// `force_mode` < 0 picks by batch size.
static std::atomic<int> g_force_table_mode{-1};


static StreamArgs as_stream_args(const RansArgs &a)
{
    StreamArgs sa{};
    sa.src = a.src; sa.sjobs = a.jobs; sa.offs = a.offs; sa.plane = a.plane;
    sa.njobs = a.njobs; sa.dst = a.dst; sa.status = a.status; sa.any_bad = a.any_bad;
    sa.shared_hdr = a.shared_hdr;
    return sa;
}

// A large batch whose tables the host cannot see: sort the streams by alphabet size on the
// device and give the small ones to the denser 128-entry instance.  The index list lives in
// stream-ordered memory for the duration of the two launches.  Returns 1 when that memory
// is not to be had (the caller then runs everything on the 256-entry instance).
// A memory pool of this library's own per device, which keeps what is freed into it: the
// default pool hands memory back to the driver at every synchronisation, and getting it
// again costs more than the index list's kernels.
static cudaMemPool_t scratch_pool()
{
    static cudaMemPool_t pools[64];
    static bool tried[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried[dev]) {
        tried[dev] = true;
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) == cudaSuccess) {
            uint64_t keep = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            pools[dev] = pool;
        } else {
            cudaGetLastError();
        }
    }
    return pools[dev];
}

static int launch_compact_sorted(const RansArgs &a, cudaStream_t cs)
{
    uint32_t *buf = nullptr;
    const size_t bytes = ((size_t)a.njobs + 2) * sizeof(uint32_t);
    cudaMemPool_t pool = scratch_pool();
    if (!pool || cudaMallocFromPoolAsync((void **)&buf, bytes, pool, cs) != cudaSuccess) {
        cudaGetLastError();
        return 1;
    }
    uint32_t *counts = buf, *order = buf + 2;
    StreamArgs sa = as_stream_args(a);
    int rc = LMZ_GPU_OK;
    do {
        if (cudaMemsetAsync(counts, 0, 8, cs) != cudaSuccess) { rc = fail_msg(LMZ_GPU_ECUDA, "cudaMemsetAsync failed"); break; }
        k_classify<<<(a.njobs + 7) / 8, 256, 0, cs>>>(sa, F_SMALL_LIVE, order, counts);
        cudaError_t le = cudaGetLastError();
        if (le != cudaSuccess) { rc = fail_cuda("launch k_classify", le); break; }
        sa.order = order;
        sa.count = counts;
        sa.order_from_back = 0;
        rc = launch_stream<SINK_BYTES, false, F_SMALL_CFN>(sa, cs);
        if (rc) break;
        sa.count = counts + 1;
        sa.order_from_back = 1;
        rc = launch_stream<SINK_BYTES, false, 256>(sa, cs);
    } while (0);
    cudaFreeAsync(buf, cs);
    return rc;
}

// A launch that gives every stream an SM slot at once with 12 streams per SM is bound by
// the length of the per-symbol dependent chain alone, and a wide table per stream shortens
// it by one shared-memory round trip.  (13 such tables fit an SM too, but then not the long
// tiles that pay for the instance: above 12 per SM the narrow tables are faster.)
static int launch_rans(const RansArgs &a, cudaStream_t cs, bool may_alloc = true)
{
    if (a.njobs == 0) return LMZ_GPU_OK;
    int sms = 0;
    int rc = sm_count(&sms);
    if (rc) return rc;
    if (a.shared_hdr) {
        // one table for the whole launch: the k_stream instance (128 streams per SM, leaner
        // steps) once every SM is full, the plain kernel (shorter chain on a lone warp) below
        const int forced = g_force_table_mode.load(std::memory_order_relaxed);
        const bool plain = forced == T_NARROW || (forced < 0 && a.njobs < (unsigned)sms * 128u);
        return plain ? launch_rans_mode<T_WIDE, WARPS_WIDE>(a, cs)
                     : launch_stream<SINK_BYTES, false, -1>(as_stream_args(a), cs);
    }
    const int forced = g_force_table_mode.load(std::memory_order_relaxed);
    int mode = forced;
    if (mode < 0)
        mode = a.njobs <= (unsigned)sms * F_WIDE_GROUPS ? T_WIDE1
             : a.njobs <= (unsigned)sms * F_DIRECT_GROUPS ? T_WIDE13
             : a.njobs >= COMPACT_MIN_JOBS ? T_COMPACT : T_NARROW;
    if (mode == T_WIDE1) return launch_stream<SINK_BYTES, false, 0>(as_stream_args(a), cs);
    if (mode == T_WIDE13) return launch_stream<SINK_BYTES, false, 0, 4>(as_stream_args(a), cs);
    if (mode == T_COMPACT) {
        if (may_alloc && forced < 0) {
            int rc = launch_compact_sorted(a, cs);
            if (rc != 1) return rc;
        }
        return launch_stream<SINK_BYTES, false, 256>(as_stream_args(a), cs);
    }
    return launch_rans_mode<T_NARROW, WARPS_NARROW>(a, cs);
}

// ------------------------------------------------------- the reference's nine

API int lmz_gpu_abi_version(void) { return 1; }
API const char *lmz_gpu_last_error(void) { return g_err; }
API int lmz_gpu_grain(void) { return 1; }
API int lmz_gpu_header_bytes(void) { return (int)HDR_BYTES; }
API int lmz_gpu_pad_bytes(void) { return (int)PAD_BYTES; }

API int lmz_gpu_device_name(char *buf, int cap)
{
    if (!buf || cap <= 0) return fail_msg(LMZ_GPU_EUNSUPPORTED, "no room for the device name");
    if (int rc = device_ready()) return rc;
    int dev = 0, cc_major = 0, cc_minor = 0, sms = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    cudaDeviceProp prop;
    CK("cudaGetDeviceProperties", cudaGetDeviceProperties(&prop, dev));
    cc_major = prop.major; cc_minor = prop.minor; sms = prop.multiProcessorCount;
    snprintf(buf, (size_t)cap, "%s sm_%d%d %d SMs", prop.name, cc_major, cc_minor, sms);
    return LMZ_GPU_OK;
}

// What is wrong with the stream at `p` of `len` bytes as far as its first 516 bytes can
// tell (NULL = nothing): the checks lmz_rans_decode makes before it touches a state
// (lmz/native/lmzcore.c:1413-1427).
static const char *header_defect(const uint8_t *p, uint64_t len)
{
    if (len < HDR_BYTES + STATE_BYTES) return "a stream is shorter than its own header";
    if (p[0] != 'R' || p[1] != '1') return "a stream does not start with the rANS magic";
    uint32_t total = 0;
    for (const uint8_t *f = p + 4; f < p + HDR_BYTES; f += 2) total += f[0] | ((uint32_t)f[1] << 8);
    return total == PROB_SCALE ? nullptr : "a stream's frequencies do not sum to 4096";
}

API int lmz_gpu_validate(const void *streams_v, const void *off_v, unsigned nstr)
{
    const uint8_t *base = static_cast<const uint8_t *>(streams_v);
    const uint64_t *pairs = static_cast<const uint64_t *>(off_v);
    for (const uint64_t *e = pairs; e != pairs + 2 * (size_t)nstr; e += 2)
        if (const char *defect = header_defect(base + e[0], e[1])) return fail_msg(LMZ_GPU_EBADSTREAM, defect);
    return LMZ_GPU_OK;
}

API int lmz_gpu_decode_batch_dev(const void *d_hdr, const void *d_streams, const void *d_off,
                                 unsigned nstr, unsigned plane, void *d_out, void *cuda_stream,
                                 unsigned tpb)
{
    (void)tpb;  // block shape is fixed by the shared-memory layout
    if (nstr == 0) return LMZ_GPU_OK;
    if (plane == 0) return fail_msg(LMZ_GPU_EUNSUPPORTED, "plane is zero");
    int rc = device_ready();
    if (rc) return rc;
    RansArgs a{};
    a.src = (const uint8_t *)d_streams;
    a.offs = (const uint64_t *)d_off;
    a.plane = plane;
    a.njobs = nstr;
    a.dst = (uint8_t *)d_out;
    a.shared_hdr = (const uint8_t *)d_hdr;
    return launch_rans(a, (cudaStream_t)cuda_stream);
}

namespace {
// Device memory that lives as long as one host-form call.
struct Transient {
    void *p = nullptr;
    ~Transient() { if (p) cudaFree(p); }
    cudaError_t take(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1); }
    template <class T> T *as() const { return static_cast<T *>(p); }
};
}  // namespace

API int lmz_gpu_decode_batch(const void *hdr, const void *streams, size_t nbytes, const void *off,
                             unsigned nstr, unsigned plane, void *out)
{
    if (nstr == 0) return LMZ_GPU_OK;
    if (plane == 0) return fail_msg(LMZ_GPU_EUNSUPPORTED, "plane is zero");
    if (int rc = device_ready()) return rc;
    // every (offset, length) pair must lie inside the buffer, and a length must fit the
    // 32 bits the kernels carry it in
    const uint64_t *pairs = static_cast<const uint64_t *>(off);
    for (unsigned i = 0; i < nstr; i++) {
        const uint64_t at = pairs[2 * i], len = pairs[2 * i + 1];
        if (at > nbytes || len > nbytes - at) return fail_msg(LMZ_GPU_EBADSTREAM, "a stream lies outside the buffer");
        if (len >> 32) return fail_msg(LMZ_GPU_EUNSUPPORTED, "a stream is 4 GiB or longer");
    }
    if (!hdr)
        if (int rc = lmz_gpu_validate(streams, off, nstr)) return rc;

    const size_t out_bytes = (size_t)nstr * plane, table_bytes = (size_t)nstr * 16;
    Transient coded, table, plain, verdict, shared;
    CK("cudaMalloc(streams)", coded.take(nbytes + PAD_BYTES));
    CK("cudaMalloc(offsets)", table.take(table_bytes));
    CK("cudaMalloc(out)", plain.take(out_bytes));
    CK("cudaMalloc(verdict)", verdict.take(sizeof(uint32_t)));
    CK("copy streams in", cudaMemcpy(coded.p, streams, nbytes, cudaMemcpyHostToDevice));
    CK("clear the slack", cudaMemset(coded.as<uint8_t>() + nbytes, 0, PAD_BYTES));
    CK("copy offsets in", cudaMemcpy(table.p, off, table_bytes, cudaMemcpyHostToDevice));
    CK("clear the verdict", cudaMemset(verdict.p, 0, sizeof(uint32_t)));
    if (hdr) {
        CK("cudaMalloc(table)", shared.take(HDR_BYTES));
        CK("copy table in", cudaMemcpy(shared.p, hdr, HDR_BYTES, cudaMemcpyHostToDevice));
    }
    RansArgs a{};
    a.src = coded.as<uint8_t>();
    a.offs = table.as<uint64_t>();
    a.plane = plane;
    a.njobs = nstr;
    a.dst = plain.as<uint8_t>();
    a.shared_hdr = shared.as<uint8_t>();
    a.any_bad = verdict.as<uint32_t>();
    if (int rc = launch_rans(a, 0)) return rc;
    CK("cudaDeviceSynchronize", cudaDeviceSynchronize());
    uint32_t any_bad = 0;
    CK("copy the verdict out", cudaMemcpy(&any_bad, verdict.p, sizeof any_bad, cudaMemcpyDeviceToHost));
    if (any_bad) return fail_msg(LMZ_GPU_EBADSTREAM, "a stream is malformed or truncated");
    CK("copy plaintext out", cudaMemcpy(out, plain.p, out_bytes, cudaMemcpyDeviceToHost));
    return LMZ_GPU_OK;
}

// ------------------------------------------------------------------- additive

API int lmz_gpu_set_table_mode(int mode)
{
    if (mode != -1 && mode != T_NARROW && mode != T_COMPACT && mode != T_WIDE1 && mode != T_WIDE13)
        return fail_msg(LMZ_GPU_EUNSUPPORTED,
                        "table mode must be -1 (auto), 0 (narrow), 2 (compact), 3 (wide per stream) or 4 (wide, 13 per SM)");
    g_force_table_mode.store(mode, std::memory_order_relaxed);
    return LMZ_GPU_OK;
}

// ---- batch encode (no counterpart in the reference's GPU library) -------------------

constexpr unsigned ENCODE_MAX_PLANE = 1u << 29;      // slot sizes stay below 2^31

API int lmz_gpu_encode_slot_bytes(unsigned plane)
{
    return plane == 0 || plane > ENCODE_MAX_PLANE ? 0 : (int)encode_slot_bytes(plane);
}

API int lmz_gpu_encode_batch_dev(const void *d_planes, unsigned nstr, unsigned plane, void *d_slots,
                                 void *d_lengths, void *cuda_stream)
{
    int rc = device_ready();
    if (rc) return rc;
    if (nstr == 0) return LMZ_GPU_OK;
    if (!d_planes || !d_slots || !d_lengths) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    if (plane == 0 || plane > ENCODE_MAX_PLANE) return fail_msg(LMZ_GPU_EUNSUPPORTED, "plane must be 1 .. 2^29 bytes");
    if ((uintptr_t)d_slots & 511u) return fail_msg(LMZ_GPU_EUNSUPPORTED, "the slot buffer must be 512-byte aligned");
    constexpr int WARPS = 4;      // 43 KiB of shared memory a CTA: five CTAs (80 streams) per SM
    static bool done[64];
    constexpr uint32_t shm = encode_smem_bytes(WARPS);
    rc = opt_in_smem(k_encode<WARPS>, shm, done);
    if (rc) return rc;
    EncodeArgs a{};
    a.src = (const uint8_t *)d_planes;
    a.plane = plane;
    a.nstr = nstr;
    a.slots = (uint8_t *)d_slots;
    a.slot_bytes = encode_slot_bytes(plane);
    a.lengths = (uint32_t *)d_lengths;
    k_encode<WARPS><<<(nstr + WARPS * 4 - 1) / (WARPS * 4), WARPS * 32, shm, (cudaStream_t)cuda_stream>>>(a);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_encode", le);
    return LMZ_GPU_OK;
}

API int lmz_gpu_pack_streams_dev(const void *d_slots, unsigned plane, const void *d_offsets, unsigned nstr,
                                 void *d_out, void *cuda_stream)
{
    int rc = device_ready();
    if (rc) return rc;
    if (nstr == 0) return LMZ_GPU_OK;
    if (!d_slots || !d_offsets || !d_out) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    if (plane == 0 || plane > ENCODE_MAX_PLANE) return fail_msg(LMZ_GPU_EUNSUPPORTED, "plane must be 1 .. 2^29 bytes");
    k_pack_streams<<<nstr, 128, 0, (cudaStream_t)cuda_stream>>>((const uint8_t *)d_slots, encode_slot_bytes(plane),
                                                              (const uint64_t *)d_offsets, nstr, (uint8_t *)d_out);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_pack_streams", le);
    return LMZ_GPU_OK;
}

// ---- chunk framing for the save path (no counterpart in the reference's GPU library) --------

static int framing_args(const void *d_src, uint64_t nbytes, unsigned chunk)
{
    if (!d_src) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    if (chunk < 2 || (chunk & 1u) || (nbytes & 1u))
        return fail_msg(LMZ_GPU_EUNSUPPORTED, "chunk size and byte count must be even (whole BF16 elements)");
    if (nbytes > (uint64_t)chunk * 0x7fffffffu) return fail_msg(LMZ_GPU_EUNSUPPORTED, "too many chunks for one call");
    return LMZ_GPU_OK;
}

API int lmz_gpu_split_bf16_dev(const void *d_src, uint64_t nbytes, unsigned chunk, void *d_planes, void *cuda_stream)
{
    int rc = device_ready();
    if (rc) return rc;
    if (nbytes == 0) return LMZ_GPU_OK;
    rc = framing_args(d_src, nbytes, chunk);
    if (rc) return rc;
    if (!d_planes) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    const unsigned nchunks = (unsigned)((nbytes + chunk - 1) / chunk);
    k_split_bf16<<<nchunks, 256, 0, (cudaStream_t)cuda_stream>>>((const uint8_t *)d_src, nbytes, chunk, (uint8_t *)d_planes);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_split_bf16", le);
    return LMZ_GPU_OK;
}

API int lmz_gpu_frame_bf16_dev(const void *d_src, uint64_t nbytes, unsigned chunk, const void *d_lengths,
                               void *d_meta, const void *d_planes, const void *d_slots, const void *d_offsets,
                               void *d_out, void *cuda_stream)
{
    int rc = device_ready();
    if (rc) return rc;
    if (nbytes == 0) return LMZ_GPU_OK;
    rc = framing_args(d_src, nbytes, chunk);
    if (rc) return rc;
    if (!d_lengths || !d_meta) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    const unsigned nchunks = (unsigned)((nbytes + chunk - 1) / chunk), nfull = (unsigned)(nbytes / chunk);
    cudaStream_t cs = (cudaStream_t)cuda_stream;
    if (!d_out) {
        k_frame_decide<<<(nchunks + 127) / 128, 128, 0, cs>>>(nbytes, chunk, nchunks, (const uint32_t *)d_lengths,
                                                             (FrameMeta *)d_meta);
    } else {
        if (!d_planes || !d_slots || !d_offsets) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
        const unsigned tail = (unsigned)(nbytes - (uint64_t)nfull * chunk);
        k_frame_pack<<<nchunks, 256, 0, cs>>>((const uint8_t *)d_src, nbytes, chunk, (const uint32_t *)d_lengths,
                                              (const FrameMeta *)d_meta, (const uint8_t *)d_planes,
                                              (const uint8_t *)d_slots, encode_slot_bytes(chunk / 2),
                                              tail ? encode_slot_bytes(tail / 2) : 0u, nfull,
                                              (const uint64_t *)d_offsets, (uint8_t *)d_out);
    }
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch chunk framing", le);
    return LMZ_GPU_OK;
}

API int lmz_gpu_crc32_chunks_dev(const void *d_src, uint64_t nbytes, unsigned chunk, const void *d_crc_tables,
                                 void *d_meta, void *cuda_stream)
{
    int rc = device_ready();
    if (rc) return rc;
    if (nbytes == 0) return LMZ_GPU_OK;
    if (!d_src || !d_crc_tables || !d_meta || chunk == 0) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    static bool done[64];
    constexpr uint32_t shm = 5u * (1024u << 4);       // four tables replicated 16x, and room to align them
    rc = opt_in_smem(k_crc32_chunks, shm, done);
    if (rc) return rc;
    const unsigned nchunks = (unsigned)((nbytes + chunk - 1) / chunk);
    k_crc32_chunks<<<nchunks, 256, shm, (cudaStream_t)cuda_stream>>>((const uint8_t *)d_src, nbytes, chunk,
                                                                     (const CrcTables *)d_crc_tables, (FrameMeta *)d_meta);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_crc32_chunks", le);
    return LMZ_GPU_OK;
}

API int lmz_gpu_set_device(int device)
{
    int rc = device_ready();
    if (rc) return rc;
    CK("cudaSetDevice", cudaSetDevice(device));
    return LMZ_GPU_OK;
}

API int lmz_gpu_decode_streams_dev(const void *d_jobs, unsigned njobs, const void *d_src,
                                   void *d_dst, const void *d_shared_hdr, void *d_status,
                                   void *d_any_bad, void *cuda_stream)
{
    if (njobs == 0) return LMZ_GPU_OK;
    int rc = device_ready();
    if (rc) return rc;
    RansArgs a{};
    a.src = (const uint8_t *)d_src;
    a.jobs = (const StreamJob *)d_jobs;
    a.njobs = njobs;
    a.dst = (uint8_t *)d_dst;
    a.shared_hdr = (const uint8_t *)d_shared_hdr;
    a.status = (uint32_t *)d_status;
    a.any_bad = (uint32_t *)d_any_bad;
    return launch_rans(a, (cudaStream_t)cuda_stream);
}

#include "chunk_abi.inl"

// ------------------------------------------------- checked decode, no allocation

// Some hosts cannot let a plug-in allocate device memory: an inference server or
// training job whose own pool has already claimed all of HBM (cudaMalloc then fails
// or fragments the pool), or a loader that runs where the embedding framework
// forbids driver allocations.  lmz_gpu_decode_batch_dev serves them but cannot say
// whether a stream was truncated, because its per-stream verdicts need memory the
// reference's signature has no argument for.  This entry point keeps those verdicts
// in a fixed device array that is part of the library image instead.
//
// The array costs LMZ_GPU_NOALLOC_MAX_STREAMS * 4 + 256 bytes on every GPU that
// loads the library, until the process exits.  Every call on a device shares it:
// calls that overlap on the GPU (different CUDA streams, different host threads)
// race on the verdicts and must be serialised by the caller.
static __device__ __align__(256) uint32_t g_noalloc_verdicts[64 + LMZ_GPU_NOALLOC_MAX_STREAMS];

// In host code the array's name only stands for the symbol; the address a kernel
// can use comes from cudaGetSymbolAddress, per device, with that device current.
static int noalloc_scratch(uint32_t **out)
{
    static uint32_t *ptr_of[64];
    static std::mutex mu;
    int dev = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail_msg(LMZ_GPU_EUNSUPPORTED, "device index above 63");
    std::lock_guard<std::mutex> lock(mu);
    if (!ptr_of[dev]) {
        void *p = nullptr;
        CK("cudaGetSymbolAddress(verdicts)", cudaGetSymbolAddress(&p, g_noalloc_verdicts));
        ptr_of[dev] = static_cast<uint32_t *>(p);
    }
    *out = ptr_of[dev];
    return LMZ_GPU_OK;
}

API int lmz_gpu_decode_batch_dev_noalloc(const void *d_hdr, const void *d_streams,
                                         const void *d_off, unsigned nstr, unsigned plane,
                                         void *d_out, void *cuda_stream, uint32_t *h_status)
{
    if (nstr == 0) return LMZ_GPU_OK;
    if (plane == 0) return fail_msg(LMZ_GPU_EUNSUPPORTED, "plane is zero");
    if (nstr > LMZ_GPU_NOALLOC_MAX_STREAMS) {
        snprintf(g_err, sizeof g_err,
                 "lmz_gpu_decode_batch_dev_noalloc takes at most %u streams per call, got %u; "
                 "split the batch", (unsigned)LMZ_GPU_NOALLOC_MAX_STREAMS, nstr);
        return LMZ_GPU_EUNSUPPORTED;
    }
    int rc = device_ready();
    if (rc) return rc;
    uint32_t *scratch = nullptr;
    rc = noalloc_scratch(&scratch);          // first call on a device resolves the symbol
    if (rc) return rc;
    cudaStream_t cs = (cudaStream_t)cuda_stream;
    // the summary word keeps the previous call's value: it must start at zero
    CK("cudaMemsetAsync(verdict summary)", cudaMemsetAsync(scratch, 0, 256, cs));
    RansArgs a{};
    a.src = (const uint8_t *)d_streams;
    a.offs = (const uint64_t *)d_off;
    a.plane = plane;
    a.njobs = nstr;
    a.dst = (uint8_t *)d_out;
    a.shared_hdr = (const uint8_t *)d_hdr;
    a.status = scratch + 64;                 // every job writes its own word
    a.any_bad = scratch;
    rc = launch_rans(a, cs, /*may_alloc=*/false);
    if (rc) return rc;
    uint32_t bad = 0;
    CK("cudaMemcpyAsync(verdict summary)",
       cudaMemcpyAsync(&bad, scratch, sizeof bad, cudaMemcpyDeviceToHost, cs));
    if (h_status)
        CK("cudaMemcpyAsync(verdicts)", cudaMemcpyAsync(h_status, scratch + 64, (size_t)nstr * 4,
                                                        cudaMemcpyDeviceToHost, cs));
    CK("cudaStreamSynchronize", cudaStreamSynchronize(cs));
    if (bad) return fail_msg(LMZ_GPU_EBADSTREAM, "a stream is malformed or truncated");
    return LMZ_GPU_OK;
}
