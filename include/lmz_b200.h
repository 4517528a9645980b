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
 * accepted and ignored.  Unlike the reference's, a batch of 9472 streams or more
 * with per-stream tables takes (nstr + 2) * 4 bytes of stream-ordered memory from
 * a pool this library keeps per device, for an index list that sorts the streams
 * by alphabet size; lmz_gpu_decode_batch_dev_noalloc never does. */
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

/* No counterpart in the reference: choose the per-stream decode-table layout for
 * streams that carry their own table.  -1 = by batch size (default), 0 = narrow
 * (5 KiB per stream), 2 = compact (2 KiB, the most streams per SM), 3 = a wide
 * 16 KiB table per stream (one lookup per symbol; 12 streams per SM, for launches
 * small enough to be bound by per-symbol latency), 4 = the same with 13 streams per SM
 * and every symbol stored straight to its output byte.  A tuning and testing knob;
 * results are identical. */
int lmz_gpu_set_table_mode(int mode);

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

/* No counterpart in the reference.  lmz_gpu_decode_batch_dev with per-stream
 * verdicts, for callers that may not allocate device memory -- a server or trainer
 * whose own pool already owns all of HBM, or a loader running where its host
 * framework forbids driver allocations.  The verdicts live in a fixed device array
 * inside the library (LMZ_GPU_NOALLOC_MAX_STREAMS * 4 + 256 bytes on every GPU that
 * loads it, held until the process exits); nothing is allocated or freed here.
 *
 * Arguments as lmz_gpu_decode_batch_dev (no tpb).  h_status is host memory for nstr
 * uint32 verdicts (0 ok, 1 bad header, 2 truncated, 3 input timeout, 0x100 trailing
 * slack) or NULL.  The call is synchronous -- it waits for cuda_stream and copies the
 * verdicts to the host before it returns -- and returns LMZ_GPU_EBADSTREAM if
 * any stream failed, LMZ_GPU_EUNSUPPORTED if nstr exceeds the maximum (split the
 * batch).  The first call on each device looks up the array's device address; make
 * that call before starting any stream capture.  All calls on a device share the
 * array: calls that overlap on the GPU race on it, so issue them one at a time. */
#define LMZ_GPU_NOALLOC_MAX_STREAMS 65536u
int lmz_gpu_decode_batch_dev_noalloc(const void *d_hdr, const void *d_streams, const void *d_off,
                                     unsigned nstr, unsigned plane, void *d_out,
                                     void *cuda_stream, uint32_t *h_status);

/* ---- batch encode -----------------------------------------------------------
 * No counterpart in the reference's GPU library (its encoder is CPU code,
 * lmz/native/lmzcore.c:882-937 and :958-979, :1318-1383).  Stream i is byte-identical
 * to what that encoder writes for plane i with the plane's own histogram.
 *
 * d_planes: nstr planes of `plane` bytes back to back.  d_slots: nstr slots of
 * lmz_gpu_encode_slot_bytes(plane) bytes, 512-byte aligned; stream i is written so
 * that it ENDS at the end of slot i.  d_lengths: nstr uint32, the stream lengths
 * (0 = that plane could not be coded).  plane is 1 .. 2^29; lmz_gpu_encode_slot_bytes
 * returns 0 outside that range.  Asynchronous on cuda_stream. */
int lmz_gpu_encode_slot_bytes(unsigned plane);
int lmz_gpu_encode_batch_dev(const void *d_planes, unsigned nstr, unsigned plane, void *d_slots,
                             void *d_lengths, void *cuda_stream);
/* Copy the streams out of their slots into one buffer: d_offsets = 2*nstr uint64
 * (byte offset in d_out, length) - the layout lmz_gpu_decode_batch_dev reads. */
int lmz_gpu_pack_streams_dev(const void *d_slots, unsigned plane, const void *d_offsets, unsigned nstr,
                             void *d_out, void *cuda_stream);

/* ---- chunk framing for the save path ------------------------------------------
 * No counterpart in the reference's GPU library; the reference frames chunks on the CPU
 * (lmz/codec.py:914-1009 encode_chunk, for BF16: :939-1003).  Together with the batch
 * encoder these turn BF16 bytes in HBM into the chunk payloads the reference writes at
 * chunk sizes below 2 MiB.  d_src: nbytes of BF16 data cut into chunks of `chunk` bytes
 * (the last may be shorter); both even.
 *
 * lmz_gpu_split_bf16_dev: d_planes (nbytes) receives, chunk by chunk at the chunk's own
 * offset, its exponent plane and then its sign/mantissa plane (lmz/native/lmzcore.c:430-437):
 * the layout lmz_gpu_encode_batch_dev takes with nstr = 2 * chunks, plane = chunk / 2.
 *
 * lmz_gpu_frame_bf16_dev, first with d_out = NULL: d_lengths (2 uint32 per chunk, the coded
 * length of each plane as the encoder reported it) -> d_meta (4 uint32 per chunk: payload
 * length, codec id, flags, crc32) with the first three filled in: a coded plane is kept where
 * it saves max(1024, n >> 8) bytes (lmz/codec.py:385-398), the chunk is CODEC_BF16 if a plane
 * is kept and the payload is shorter than the chunk, else stored (:997-1003).  Then with
 * d_offsets (uint64 per chunk: where its payload starts in d_out, from the lengths above),
 * d_planes and d_slots (the encoder's slots: full chunks first, then the short last chunk's
 * two): the payload bytes.
 *
 * lmz_gpu_crc32_chunks_dev: crc32 of every chunk's plaintext into d_meta (lmz/codec.py:931);
 * d_crc_tables as for the decode (lmz_gpu_crc_tables). */
int lmz_gpu_split_bf16_dev(const void *d_src, uint64_t nbytes, unsigned chunk, void *d_planes, void *cuda_stream);
int lmz_gpu_frame_bf16_dev(const void *d_src, uint64_t nbytes, unsigned chunk, const void *d_lengths,
                           void *d_meta, const void *d_planes, const void *d_slots, const void *d_offsets,
                           void *d_out, void *cuda_stream);
int lmz_gpu_crc32_chunks_dev(const void *d_src, uint64_t nbytes, unsigned chunk, const void *d_crc_tables,
                             void *d_meta, void *cuda_stream);

/* ---- whole-archive decode ---------------------------------------------------
 * The reference has no GPU counterpart for anything below: its chunk framing,
 * plane merge, exponent conditioning, delta undo and checksum run on the CPU
 * (lmz/codec.py:1075-1230, lmz/api.py:832-886).  These entry points run that
 * work on the device from descriptors the host planner builds out of the
 * archive's 32-byte chunk records (lmz/format.py:53-56). */

/* sizeof of {stream job, chunk job, cond job, cond state, fused job}, so a host
 * planner can check its mirrored layouts. */
int lmz_gpu_struct_sizes(unsigned *out5);

/* Chunks of a shared-table archive that one thread block decodes against one table (80):
 * the unit a planner pads each table's run of jobs to. */
int lmz_gpu_shared_group(void);

/* Output bytes one thread block finishes at a time (65536); chunks are cut into
 * pieces of this size and checksummed piecewise. */
int lmz_gpu_piece_bytes(void);
/* sizeof the delta job of lmz_decode_plan.d_delta_jobs (48). */
int lmz_gpu_delta_job_bytes(void);

/* Fill host_dst with the CRC-32 tables the finish kernel reads (upload them once
 * per device).  Returns the size in bytes; if cap is too small nothing is written. */
int lmz_gpu_crc_tables(void *host_dst, size_t cap);

/* Host helper for planners: out[i] = number of symbols with a non-zero frequency
 * in the 516-byte table of the stream that starts at base + offs[i] (host
 * pointers; the caller has checked that offs[i] + 516 is inside the buffer).
 * Streams with at most 104 live symbols may be listed first in d_fused_jobs and
 * counted in n_fused_small. */
int lmz_host_alphabet_sizes(const void *base, const uint64_t *offs, size_t n, uint16_t *out);

/* Everything lmz_gpu_decode_chunks_dev needs.  All pointers are device pointers.
 * Layouts of the job arrays are those of csrc/common.cuh and csrc/chunk_kernels.cuh;
 * lmz_b200/plan.py builds them. */
typedef struct lmz_decode_plan {
    const void *d_payload;      /* archive payload bytes, 16-byte aligned, pad_bytes() of slack */
    void *d_scratch;            /* decoded planes and segments */
    void *d_out;                /* the concatenated output space, 64 bytes of slack */
    const void *d_stream_jobs;  /* rANS streams whose decoded size the host knows */
    void *d_seg_jobs;           /* 8 per conditioned chunk, sized on the device */
    void *d_stream_status;      /* uint32 per stream job */
    void *d_seg_status;         /* uint32 per segment job */
    const void *d_fused_jobs;   /* chunks decoded, merged and checksummed by one kernel: BF16 chunks
                                 * (coded exponent plane, stored mantissa plane), the first
                                 * n_fused_small of them with at most 104 live symbols; then the
                                 * n_fused_f32 chunks of 4-byte elements (coded top byte plane, three
                                 * stored planes), the first n_fused_f32_small of them small likewise */
    void *d_fused_status;       /* uint32 per fused job */
    const void *d_delta_jobs;   /* BF16 chunks with both planes coded (csrc/fused_kernel.cuh, DeltaJob): decoded, merged
                                 * and checksummed by one kernel -- the first n_delta_plain of them plain chunks
                                 * (base_off all ones), in the first pass; the others delta chunks, XOR-ed with their
                                 * base once the chunks they are differences against have been written */
    void *d_delta_status;       /* uint32 per stream: two per job */
    void *d_delta_order;        /* n_delta + 4 uint32 of work space (the jobs sorted by alphabet size on the device) */
    const void *d_chunks;       /* chunk jobs, ordered: pass 1 cond, pass 1 plain, fused, pass 2 cond, pass 2 plain */
    const void *d_piece_chunk;  /* uint32 per piece: its chunk */
    const void *d_cond_jobs;
    void *d_cond_state;
    const void *d_cond_pieces;  /* uint32 piece ids of conditioned chunks */
    void *d_hist;               /* n_cond x 256 uint32 */
    void *d_piece_cnt;          /* n_pieces x 16 uint32 */
    void *d_piece_wcnt;         /* n_pieces x 64 uint16 */
    void *d_piece_lcnt;         /* n_cond_pieces x 2048 uint32 (8 KiB per conditioned piece) */
    void *d_piece_crc;          /* n_pieces uint32, or NULL to skip checksums */
    const void *d_crc_tables;
    void *d_chunk_status;       /* uint32 per chunk: 0 ok, 4 bad shape, 5 bad crc */
    void *d_chunk_crc;          /* computed crc32 per chunk, or NULL */
    void *d_any_bad;            /* uint32: bit 0 a stream failed, bit 1 a chunk failed */
    const void *d_tables;       /* shared-table chunks: the archive's 516-byte tables, 528 bytes apart */
    void *d_fused_order;        /* NULL, or n_fused + 4 uint32 of work space: the library then counts
                                 * every fused stream's alphabet on the device and sorts the jobs
                                 * itself (n_fused_small and n_fused_f32_small are ignored, the jobs may
                                 * come in any order within the BF16 and the 4-byte-element group) */
    uint32_t n_stream_jobs, n_seg_jobs, n_chunks, n_pieces, n_cond, n_cond_pieces, n_fused;
    uint32_t n_fused_small;     /* leading fused jobs whose streams have small alphabets (see
                                 * lmz_host_alphabet_sizes); they take the denser kernel instance */
    uint32_t n_fused_f32;       /* trailing fused jobs that are 4-byte-element chunks (counted in n_fused) */
    uint32_t n_fused_f32_small; /* the first of those, with small alphabets */
    uint32_t n_fused_t;         /* shared-table BF16 chunks: further jobs after the n_fused in d_fused_jobs (and
                                 * d_fused_status), `flags` = table number in d_tables, listed table by table
                                 * and each table's run padded with empty jobs (n = 0) to a multiple of
                                 * lmz_gpu_shared_group() */
    uint32_t n_delta;           /* jobs in d_delta_jobs */
    uint32_t n_delta_plain;     /* the first of them, which have no base */
    uint32_t piece_split[6];    /* piece-id boundaries of the five chunk groups */
    uint32_t phases;            /* 0 = everything; else bit 0 stream decode, bit 1 conditioned-chunk
                                 * kernels, bit 2 finish, bit 3 verdicts, bit 4 fused chunks
                                 * (to time one phase alone) */
} lmz_decode_plan;

/* Decode every chunk of the plan into d_out: rANS streams, conditioned-chunk
 * bookkeeping, then the fused merge / delta-XOR / CRC pass that writes the
 * plaintext once.  Asynchronous on cuda_stream; the caller reads d_any_bad and
 * the status arrays after synchronising. */
int lmz_gpu_decode_chunks_dev(const lmz_decode_plan *plan, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* LMZ_B200_H */
