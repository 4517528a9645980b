// Additive C-ABI entry points for whole-archive decode (included by lmz_b200.cu).

#include "cond_kernels.cuh"
#include "cond_finish.cuh"

static_assert(sizeof(lmz_stream_job) == sizeof(StreamJob), "public and device StreamJob differ");

API int lmz_gpu_struct_sizes(unsigned *out5)
{
    out5[0] = (unsigned)sizeof(StreamJob);
    out5[1] = (unsigned)sizeof(ChunkJob);
    out5[2] = (unsigned)sizeof(CondJob);
    out5[3] = (unsigned)sizeof(CondState);
    out5[4] = (unsigned)sizeof(FusedJob);
    return LMZ_GPU_OK;
}

API int lmz_gpu_piece_bytes(void) { return (int)PIECE_BYTES; }
API int lmz_gpu_shared_group(void) { return F_SHARED_SINK_WARPS * 4; }
API int lmz_gpu_delta_job_bytes(void) { return (int)sizeof(DeltaJob); }

API int lmz_gpu_crc_tables(void *host_dst, size_t cap)
{
    if (cap < sizeof(CrcTables)) return (int)sizeof(CrcTables);
    static CrcTables tabs;
    static std::once_flag once;
    std::call_once(once, [] { crc_build_tables(tabs); });
    memcpy(host_dst, &tabs, sizeof tabs);
    return (int)sizeof(CrcTables);
}

// Plain pieces: 4 sub-blocks (1024 threads) share one set of CRC tables.
static int launch_finish(const FinishArgs &fa, int sms, cudaStream_t cs)
{
    if (fa.piece_begin >= fa.piece_end) return LMZ_GPU_OK;
    constexpr int SUBS = 4;
    static bool done[64];
    constexpr uint32_t shm = finish_smem(SUBS);
    int rc = opt_in_smem(k_finish<SUBS>, shm, done);
    if (rc) return rc;
    unsigned n = (fa.piece_end - fa.piece_begin + SUBS - 1) / SUBS;
    unsigned grid = n < (unsigned)sms ? n : (unsigned)sms;
    k_finish<SUBS><<<grid, FINISH_THREADS * SUBS, shm, cs>>>(fa);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_finish", le);
    return LMZ_GPU_OK;
}

static int launch_cond_finish(const FinishArgs &fa, int sms, cudaStream_t cs)
{
    if (fa.piece_begin >= fa.piece_end) return LMZ_GPU_OK;
    static bool done[64];
    constexpr uint32_t shm = cond_finish_smem();
    int rc = stream_smem_ok();                   // the kernel's layout counts on the same shared window as k_stream's
    if (rc) return rc;
    rc = opt_in_smem(k_cond_finish, shm, done);
    if (rc) return rc;
    // one CTA per SM, four pieces in flight in each
    unsigned n = (fa.piece_end - fa.piece_begin + CF_SUBS - 1) / CF_SUBS;
    unsigned grid = n < (unsigned)sms ? n : (unsigned)sms;
    k_cond_finish<<<grid, CF_THREADS, shm, cs>>>(fa);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_cond_finish", le);
    return LMZ_GPU_OK;
}

static int sm_count(int *out)
{
    static int cached[64];
    int dev = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && cached[dev]) { *out = cached[dev]; return LMZ_GPU_OK; }
    int n = 0;
    CK("cudaDeviceGetAttribute", cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev >= 0 && dev < 64) cached[dev] = n;
    *out = n;
    return LMZ_GPU_OK;
}

// A second stream per device, so the fused kernel (most of the work) overlaps the
// few latency-bound streams and pieces that cannot be fused.  Created on first use.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex busy;     // held by the host thread that is between its fork and its join
};

// From fork to join one host thread owns the device's side stream and its two events
// (another thread's record would move them under it); whichever way the call ends, the
// caller's stream is made to wait for what was put on the side stream.
struct SideScope {
    SideStream *side = nullptr;
    cudaStream_t main = nullptr;
    bool forked = false;
    std::unique_lock<std::mutex> owner;
    cudaError_t fork(SideStream *s, cudaStream_t cs)
    {
        side = s; main = cs;
        owner = std::unique_lock<std::mutex>(s->busy);
        cudaError_t e = cudaEventRecord(s->fork, cs);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s->stream, s->fork, 0);
        forked = e == cudaSuccess;
        return e;
    }
    cudaError_t join()
    {
        if (!forked) return cudaSuccess;
        forked = false;
        cudaError_t e = cudaEventRecord(side->join, side->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(main, side->join, 0);
        return e;
    }
    ~SideScope() { join(); }
};

// `which`: 0 = the fused kernel's stream, 1 = the conditioned chunks' counting stream.
static int side_stream(SideStream **out, int which = 0)
{
    static SideStream per_dev[2][64];
    static std::mutex mu;
    int dev = 0;
    CK("cudaGetDevice", cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { *out = nullptr; return LMZ_GPU_OK; }
    std::lock_guard<std::mutex> lock(mu);
    SideStream &s = per_dev[which][dev];
    if (!s.stream) {
        CK("cudaStreamCreate", cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
        CK("cudaEventCreate", cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
        CK("cudaEventCreate", cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
    }
    *out = &s;
    return LMZ_GPU_OK;
}

API int lmz_host_alphabet_sizes(const void *base, const uint64_t *offs, size_t n, uint16_t *out)
{
    if (!base || !offs || !out) return fail_msg(LMZ_GPU_EUNSUPPORTED, "null argument");
    const uint8_t *b = (const uint8_t *)base;
    for (size_t i = 0; i < n; i++) {
        const uint8_t *h = b + offs[i] + 4;
        unsigned live = 0;
        for (unsigned s = 0; s < 256; s++) live += (h[2 * s] | h[2 * s + 1]) != 0;
        out[i] = (uint16_t)live;
    }
    return LMZ_GPU_OK;
}

// Chunks whose two BF16 planes are both coded, jobs [first, first + count) of the plan's list: alphabets
// counted on the device, then chunks whose first plane has a small one (the rule) to the instance with
// mixed table sizes (72 streams per SM), the others to the one with full-size tables for both planes (64).
static int launch_two_plane(const lmz_decode_plan *p, uint32_t first, uint32_t count, cudaStream_t cs)
{
    if (count == 0) return LMZ_GPU_OK;
    if (!p->d_delta_jobs || !p->d_delta_status || !p->d_delta_order)
        return fail_msg(LMZ_GPU_EUNSUPPORTED, "two-plane jobs without their arrays");
    StreamArgs da{};
    da.src = (const uint8_t *)p->d_payload;
    da.djobs = (const DeltaJob *)p->d_delta_jobs + first;
    da.njobs = 2 * count;
    da.dst = (uint8_t *)p->d_out;
    da.status = (uint32_t *)p->d_delta_status + 2 * (size_t)first;
    da.any_bad = (uint32_t *)p->d_any_bad;
    da.piece_crc = (uint32_t *)p->d_piece_crc;
    da.tabs = (const CrcTables *)p->d_crc_tables;
    // work space: `count` indices and two counters, at 2 * first + ... so the two passes never share it
    uint32_t *order = (uint32_t *)p->d_delta_order + (first ? first + 2 : 0);
    uint32_t *counts = order + count;
    CK("memset two-plane counts", cudaMemsetAsync(counts, 0, 8, cs));
    StreamArgs ca = da;
    ca.njobs = count;
    k_classify<<<(count + 7) / 8, 256, 0, cs>>>(ca, F_SMALL_LIVE, order, counts);
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return fail_cuda("launch k_classify", le);
    da.order = order;
    const bool crc = p->d_piece_crc != nullptr;
    int rc = LMZ_GPU_OK;
    for (int big = 0; big < 2 && !rc; big++) {
        da.count = counts + big;
        da.order_from_back = big;
        rc = big ? (crc ? launch_stream<SINK_DELTA, true, 256>(da, cs) : launch_stream<SINK_DELTA, false, 256>(da, cs))
                 : (crc ? launch_stream<SINK_DELTA, true, F_HYBRID_CFN>(da, cs) : launch_stream<SINK_DELTA, false, F_HYBRID_CFN>(da, cs));
    }
    return rc;
}

API int lmz_gpu_decode_chunks_dev(const lmz_decode_plan *p, void *cuda_stream)
{
    if (!p) return fail_msg(LMZ_GPU_EUNSUPPORTED, "no plan");
    int rc = device_ready();
    if (rc) return rc;
    cudaStream_t cs = (cudaStream_t)cuda_stream;
    int sms = 0;
    rc = sm_count(&sms);
    if (rc) return rc;

    // `phases` selects parts of the sequence (for timing one kernel alone); 0 runs it all.
    const uint32_t ph = p->phases ? p->phases : 0x1fu;

    if (p->d_any_bad && (ph & 1u)) CK("memset any_bad", cudaMemsetAsync(p->d_any_bad, 0, 4, cs));

    // 0. BF16 chunks with a coded exponent plane and a stored sign/mantissa plane, and
    //     4-byte-element chunks with a coded top plane and three stored planes:
    //     decode, merge, write and checksum in one kernel
    SideStream *side = nullptr;
    SideScope scope;
    if (p->n_fused_t % (F_SHARED_SINK_WARPS * 4u))
        return fail_msg(LMZ_GPU_EUNSUPPORTED, "n_fused_t is not a multiple of lmz_gpu_shared_group()");
    const bool other_work = p->n_stream_jobs || p->n_cond || p->piece_split[2] > p->piece_split[0] ||
                            p->piece_split[5] > p->piece_split[3];
    if (p->n_delta_plain > p->n_delta) return fail_msg(LMZ_GPU_EUNSUPPORTED, "n_delta_plain exceeds n_delta");
    if ((p->n_fused || p->n_fused_t) && (ph & 16u)) {
        cudaStream_t fs = cs;
        if (ph == 0x1fu && other_work) {        // whole decode: run the fused kernel beside the rest
            rc = side_stream(&side);
            if (rc) return rc;
            if (side) {
                CK("fork to the side stream", scope.fork(side, cs));
                fs = side->stream;
            }
        }
        StreamArgs sa{};
        sa.src = (const uint8_t *)p->d_payload;
        sa.jobs = (const FusedJob *)p->d_fused_jobs;
        sa.njobs = p->n_fused;
        sa.dst = (uint8_t *)p->d_out;
        sa.status = (uint32_t *)p->d_fused_status;
        sa.any_bad = (uint32_t *)p->d_any_bad;
        sa.piece_crc = (uint32_t *)p->d_piece_crc;
        sa.tabs = (const CrcTables *)p->d_crc_tables;
        // BF16 chunks, then chunks of 4-byte elements; in each, small alphabets first
        // (denser instance), then the rest
        if (p->n_fused_f32 > p->n_fused) return fail_msg(LMZ_GPU_EUNSUPPORTED, "n_fused_f32 exceeds n_fused");
        const uint32_t nbf = p->n_fused - p->n_fused_f32;
        const uint32_t nsmall = p->n_fused_small < nbf ? p->n_fused_small : nbf;
        const uint32_t nsmall4 = p->n_fused_f32_small < p->n_fused_f32 ? p->n_fused_f32_small : p->n_fused_f32;
        auto part = [&](uint32_t cnt) { sa.jobs += sa.njobs; sa.status += sa.njobs; sa.njobs = cnt; };
        if (p->d_fused_order) {
            // the host has not looked at the tables: count alphabets here, small ones to the
            // front of an index list, and give each class of each group its instance
            uint32_t *order = (uint32_t *)p->d_fused_order, *counts = order + p->n_fused;
            CK("memset fused counts", cudaMemsetAsync(counts, 0, 16, fs));
            const uint32_t group_n[2] = {nbf, p->n_fused_f32};
            for (int grp = 0; grp < 2; grp++) {
                sa.njobs = group_n[grp];
                sa.order = nullptr;
                sa.count = nullptr;
                if (sa.njobs) {
                    k_classify<<<(sa.njobs + 7) / 8, 256, 0, fs>>>(sa, F_SMALL_LIVE, order, counts);
                    cudaError_t le = cudaGetLastError();
                    if (le != cudaSuccess) return fail_cuda("launch k_classify", le);
                    sa.order = order;
                    for (int big = 0; big < 2 && !rc; big++) {
                        sa.count = counts + big;
                        sa.order_from_back = big;
                        const bool crc = p->d_piece_crc != nullptr;
                        if (grp == 0)
                            rc = big ? (crc ? launch_stream<SINK_BF16, true, 256>(sa, fs) : launch_stream<SINK_BF16, false, 256>(sa, fs))
                                     : (crc ? launch_stream<SINK_BF16, true, F_SMALL_CFN>(sa, fs) : launch_stream<SINK_BF16, false, F_SMALL_CFN>(sa, fs));
                        else
                            rc = big ? (crc ? launch_stream<SINK_F32, true, 256>(sa, fs) : launch_stream<SINK_F32, false, 256>(sa, fs))
                                     : (crc ? launch_stream<SINK_F32, true, F_SMALL_CFN>(sa, fs) : launch_stream<SINK_F32, false, F_SMALL_CFN>(sa, fs));
                    }
                    if (rc) return rc;
                }
                sa.jobs += group_n[grp];
                sa.status += group_n[grp];
                order += group_n[grp];
                counts += 2;
            }
            sa.njobs = 0;            // nothing is left for the host-sorted launches below
        } else {
        sa.njobs = nsmall;
        rc = p->d_piece_crc ? launch_stream<SINK_BF16, true, F_SMALL_CFN>(sa, fs)
                            : launch_stream<SINK_BF16, false, F_SMALL_CFN>(sa, fs);
        if (rc) return rc;
        part(nbf - nsmall);
        rc = p->d_piece_crc ? launch_stream<SINK_BF16, true, 256>(sa, fs)
                            : launch_stream<SINK_BF16, false, 256>(sa, fs);
        if (rc) return rc;
        part(nsmall4);
        rc = p->d_piece_crc ? launch_stream<SINK_F32, true, F_SMALL_CFN>(sa, fs)
                            : launch_stream<SINK_F32, false, F_SMALL_CFN>(sa, fs);
        if (rc) return rc;
        part(p->n_fused_f32 - nsmall4);
        rc = p->d_piece_crc ? launch_stream<SINK_F32, true, 256>(sa, fs)
                            : launch_stream<SINK_F32, false, 256>(sa, fs);
        if (rc) return rc;
        }
        if (p->n_fused_t) {
            // chunks of a shared-table archive: every CTA takes one table's next 80 of them
            StreamArgs ta{};
            ta.src = (const uint8_t *)p->d_payload;
            ta.jobs = (const FusedJob *)p->d_fused_jobs + p->n_fused;
            ta.njobs = p->n_fused_t;
            ta.dst = (uint8_t *)p->d_out;
            ta.status = (uint32_t *)p->d_fused_status + p->n_fused;
            ta.any_bad = (uint32_t *)p->d_any_bad;
            ta.piece_crc = (uint32_t *)p->d_piece_crc;
            ta.tabs = (const CrcTables *)p->d_crc_tables;
            ta.tables = (const uint8_t *)p->d_tables;
            ta.per_cta = F_SHARED_SINK_WARPS * 4;
            if (!ta.tables) return fail_msg(LMZ_GPU_EUNSUPPORTED, "shared-table chunks without d_tables");
            rc = p->d_piece_crc ? launch_stream<SINK_BF16, true, -1>(ta, fs)
                                : launch_stream<SINK_BF16, false, -1>(ta, fs);
            if (rc) return rc;
        }
    }

    // 1. plain chunks with both planes coded: the two-plane kernel without a base (few chunks are of this
    //    shape: a short launch, beside the fused kernel when that one has a stream of its own)
    if (p->n_delta_plain && (ph & 1u)) {
        rc = launch_two_plane(p, 0, p->n_delta_plain, cs);
        if (rc) return rc;
    }

    //    and every rANS stream whose length is known up front, into scratch
    if (p->n_stream_jobs && (ph & 1u)) {
        RansArgs a{};
        a.src = (const uint8_t *)p->d_payload;
        a.jobs = (const StreamJob *)p->d_stream_jobs;
        a.njobs = p->n_stream_jobs;
        a.dst = (uint8_t *)p->d_scratch;
        a.status = (uint32_t *)p->d_stream_status;
        a.any_bad = (uint32_t *)p->d_any_bad;
        rc = launch_rans(a, cs);
        if (rc) return rc;
    }

    // 2. exponent-conditioned chunks: histogram -> bucket map -> segment decodes -> ranks
    if (p->n_cond && !p->d_piece_lcnt) return fail_msg(LMZ_GPU_EUNSUPPORTED, "conditioned chunks without d_piece_lcnt");
    if (p->n_cond && (ph & 2u)) {
        CondArgs c{};
        c.chunks = (const ChunkJob *)p->d_chunks;
        c.piece_chunk = (const uint32_t *)p->d_piece_chunk;
        c.cond_pieces = (const uint32_t *)p->d_cond_pieces;
        c.ncond_pieces = p->n_cond_pieces;
        c.cond_jobs = (const CondJob *)p->d_cond_jobs;
        c.cond_state = (CondState *)p->d_cond_state;
        c.ncond = p->n_cond;
        c.hist = (uint32_t *)p->d_hist;
        c.piece_cnt = (uint32_t *)p->d_piece_cnt;
        c.piece_wcnt = (uint16_t *)p->d_piece_wcnt;
        c.piece_lcnt = (uint32_t *)p->d_piece_lcnt;
        c.seg_jobs = (StreamJob *)p->d_seg_jobs;
        c.payload = (const uint8_t *)p->d_payload;
        c.scratch = (const uint8_t *)p->d_scratch;
        CK("memset hist", cudaMemsetAsync(p->d_hist, 0, (size_t)p->n_cond * 1024, cs));
        k_cond_hist<<<p->n_cond_pieces, 256, 0, cs>>>(c);
        k_cond_plan<<<(p->n_cond + 63) / 64, 64, 0, cs>>>(c);
        RansArgs a{};
        a.src = (const uint8_t *)p->d_payload;
        a.jobs = (const StreamJob *)p->d_seg_jobs;
        a.njobs = p->n_seg_jobs;
        a.dst = (uint8_t *)p->d_scratch;
        a.status = (uint32_t *)p->d_seg_status;
        a.any_bad = (uint32_t *)p->d_any_bad;
        // the bucket populations need only the bucket map, the segment decodes only the sizes:
        // both follow k_cond_plan and are independent of each other, so the counting (a pass over
        // the exponent planes at memory speed) runs beside the segment decodes (a few long streams
        // per SM, bound by their length)
        SideStream *aux = nullptr;
        SideScope counting;
        rc = side_stream(&aux, 1);
        if (rc) return rc;
        cudaStream_t ks = cs;
        if (aux && p->n_seg_jobs) {
            CK("fork to the counting stream", counting.fork(aux, cs));
            ks = aux->stream;
        }
        k_cond_count<<<p->n_cond_pieces, 256, 0, ks>>>(c);
        k_cond_scan<<<(p->n_cond * 8 + 127) / 128, 128, 0, ks>>>(c.chunks, c.cond_jobs, c.ncond, c.piece_cnt);
        cudaError_t le = cudaGetLastError();
        if (le != cudaSuccess) return fail_cuda("launch cond kernels", le);
        rc = launch_rans(a, cs);
        if (rc) return rc;
        CK("join the counting stream", counting.join());
    }

    // 3. finish: pass 1 (plain chunks), then pass 2 (refs and deltas, which read pass 1's output)
    FinishArgs f{};
    f.chunks = (const ChunkJob *)p->d_chunks;
    f.piece_chunk = (const uint32_t *)p->d_piece_chunk;
    f.payload = (const uint8_t *)p->d_payload;
    f.scratch = (const uint8_t *)p->d_scratch;
    f.out = (uint8_t *)p->d_out;
    f.piece_crc = (uint32_t *)p->d_piece_crc;
    f.tabs = (const CrcTables *)p->d_crc_tables;
    f.cond_jobs = (const CondJob *)p->d_cond_jobs;
    f.cond_state = (const CondState *)p->d_cond_state;
    f.piece_cnt = (const uint32_t *)p->d_piece_cnt;
    f.piece_wcnt = (const uint16_t *)p->d_piece_wcnt;
    f.piece_lcnt = (const uint32_t *)p->d_piece_lcnt;
    // piece groups: 0 pass-1 conditioned, 1 pass-1 plain, 2 fused (done above),
    //               3 pass-2 conditioned, 4 pass-2 plain
    if (!(ph & 4u)) CK("join the side stream", scope.join());
    for (int part = 0; part < 5 && (ph & 4u); part++) {
        if (part == 2) {
            // pass 2 (and the verdicts) read what the fused kernel wrote
            CK("join the side stream", scope.join());
            // delta chunks with both planes coded, now that the chunks they are differences against are in place
            rc = launch_two_plane(p, p->n_delta_plain, p->n_delta - p->n_delta_plain, cs);
            if (rc) return rc;
            continue;
        }
        f.piece_begin = p->piece_split[part];
        f.piece_end = p->piece_split[part + 1];
        // the conditioned-piece list holds pass 1's pieces, then pass 2's
        f.lcnt_first = part == 3 ? p->piece_split[1] - p->piece_split[0] : 0u;
        rc = (part == 0 || part == 3) ? launch_cond_finish(f, sms, cs)
                                      : launch_finish(f, sms, cs);
        if (rc) return rc;
    }

    // 4. verdicts
    if (p->n_chunks && (ph & 8u)) {
        CheckArgs k{};
        k.chunks = (const ChunkJob *)p->d_chunks;
        k.nchunks = p->n_chunks;
        k.piece_crc = (const uint32_t *)p->d_piece_crc;
        k.tabs = (const CrcTables *)p->d_crc_tables;
        k.cond_state = (const CondState *)p->d_cond_state;
        k.chunk_status = (uint32_t *)p->d_chunk_status;
        k.chunk_crc = (uint32_t *)p->d_chunk_crc;
        k.any_bad = (uint32_t *)p->d_any_bad;
        k_crc_check<<<(p->n_chunks + 127) / 128, 128, 0, cs>>>(k);
        cudaError_t le = cudaGetLastError();
        if (le != cudaSuccess) return fail_cuda("launch k_crc_check", le);
    }
    return LMZ_GPU_OK;
}
