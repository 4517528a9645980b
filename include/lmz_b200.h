/*
 * lmz_b200 -- C ABI of the sm_100a decoder for lmz checkpoint archives.
 *
 * Plain C: pointers and sizes only.  "d_" arguments are device pointers on the
 * current CUDA device, everything else is host memory.  Every function returns
 * one of the codes below; on failure a sentence is available from
 * lmz_gpu_last_error() (thread-local).  Nothing here throws, aborts or falls
 * back to the CPU.
 *
 * Section 1 is the interface the reference's Python layer binds
 * (lmz/gpu/__init__.py:130-148) and is call-compatible with the reference
 * library (lmz/gpu/lmzgpu.cu).  Section 2 is additive.
 */
#ifndef LMZ_B200_H
#define LMZ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes: lmz/gpu/lmzgpu.cu:49-56. */
#define LMZ_GPU_OK 0
#define LMZ_GPU_ENODEV (-1)       /* no CUDA device */
#define LMZ_GPU_EUNSUPPORTED (-2) /* a shape this library does not take */
#define LMZ_GPU_EBADSTREAM (-3)   /* malformed stream, chunk or archive data */
#define LMZ_GPU_ECUDA (-4)        /* a CUDA call or launch failed */
#define LMZ_GPU_EMISMATCH (-5)    /* a decoded chunk failed its checksum */

/* ------------------------------------------------------------------ section 1 */

/* lmz/gpu/lmzgpu.cu:341 -- 1; a caller ignores a library that answers otherwise. */
int lmz_gpu_abi_version(void);

/* lmz/gpu/lmzgpu.cu:344 -- why the last call on this thread failed. */
const char *lmz_gpu_last_error(void);

/* lmz/gpu/lmzgpu.cu:349 -- `plane` must be a multiple of this.  Returns 1: any
 * plane >= 1 is decoded, including lengths that are not a multiple of 8. */
int lmz_gpu_grain(void);

/* lmz/gpu/lmzgpu.cu:350 -- 516, the per-stream frequency table. */
int lmz_gpu_header_bytes(void);

/* lmz/gpu/lmzgpu.cu:351 -- readable bytes the caller of the _dev entry points
 * owes after the last stream (fetched, never used). */
int lmz_gpu_pad_bytes(void);

/* lmz/gpu/lmzgpu.cu:353-363 -- "<name> sm_XY N SMs" of the current device. */
int lmz_gpu_device_name(char *buf, int cap);

/* lmz/gpu/lmzgpu.cu:371-384 -- host-side check of every stream's magic and
 * frequency sum (and, here, its minimum length).  `off` is 2*nstr uint64
 * (byte offset, byte length). */
int lmz_gpu_validate(const void *streams, const void *off, unsigned nstr);

/* lmz/gpu/lmzgpu.cu:412-467 -- decode nstr streams resident on the device to
 * `plane` bytes each, stream-major, into d_out.  d_hdr is a 516-byte table
 * shared by all streams (each stream then starts at its 8 states) or NULL.
 * d_streams must be 16-byte aligned with lmz_gpu_pad_bytes() of slack after
 * the last stream.  Asynchronous on cuda_stream (NULL = default); `tpb` is
 * accepted and ignored. */
int lmz_gpu_decode_batch_dev(const void *d_hdr, const void *d_streams, const void *d_off,
                             unsigned nstr, unsigned plane, void *d_out, void *cuda_stream,
                             unsigned tpb);

/* lmz/gpu/lmzgpu.cu:478-527 -- the same for host memory: allocate, copy in,
 * decode, synchronise, copy out, free.  A stream that is malformed or
 * truncated returns LMZ_GPU_EBADSTREAM (the reference detects the former on
 * the host and returns garbage for the latter). */
int lmz_gpu_decode_batch(const void *hdr, const void *streams, size_t nbytes, const void *off,
                         unsigned nstr, unsigned plane, void *out);

/* ------------------------------------------------------------------ section 2 */

/* No counterpart in the reference (which always uses device 0): make `device`
 * current for this thread.  All other calls act on the current device. */
int lmz_gpu_set_device(int device);

/* One stream to decode; mirrors struct lmz::StreamJob.  32 bytes. */
typedef struct lmz_stream_job {
    uint64_t src_off; /* stream start, bytes from d_src */
    uint64_t dst_off; /* first output byte, bytes from d_dst */
    uint32_t src_len; /* stream length */
    uint32_t n;       /* symbols to decode */
    uint32_t flags;   /* 0 */
    uint32_t aux;     /* 0 */
} lmz_stream_job;

/* Generalises lmz_gpu_decode_batch_dev (lmz/gpu/lmzgpu.cu:412-467) to streams
 * of unequal decoded length written to arbitrary offsets.  d_status (njobs
 * uint32, may be NULL) receives 0, or 1 bad header, 2 truncated, 3 input
 * timeout, 0x100 decoded but with trailing slack; *d_any_bad (uint32, may be
 * NULL, caller zeroes it) is set when any status is 1..3.  Asynchronous. */
int lmz_gpu_decode_streams_dev(const void *d_jobs, unsigned njobs, const void *d_src,
                               void *d_dst, const void *d_shared_hdr, void *d_status,
                               void *d_any_bad, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* LMZ_B200_H */
