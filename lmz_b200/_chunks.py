"""ctypes view of the additive whole-archive entry points (include/lmz_b200.h, section 2)."""
from __future__ import annotations

import ctypes

_v, _u32 = ctypes.c_void_p, ctypes.c_uint32


class DecodePlan(ctypes.Structure):
    """Mirror of `lmz_decode_plan`."""
    _fields_ = [(n, _v) for n in (
        "d_payload", "d_scratch", "d_out", "d_stream_jobs", "d_seg_jobs", "d_stream_status",
        "d_seg_status", "d_fused_jobs", "d_fused_status", "d_delta_jobs", "d_delta_status", "d_delta_order", "d_chunks", "d_piece_chunk", "d_cond_jobs", "d_cond_state",
        "d_cond_pieces", "d_hist", "d_piece_cnt", "d_piece_wcnt", "d_piece_lcnt", "d_piece_crc", "d_crc_tables",
        "d_chunk_status", "d_chunk_crc", "d_any_bad", "d_tables", "d_fused_order")] + [(n, _u32) for n in (
            "n_stream_jobs", "n_seg_jobs", "n_chunks", "n_pieces", "n_cond", "n_cond_pieces",
            "n_fused", "n_fused_small", "n_fused_f32", "n_fused_f32_small", "n_fused_t", "n_delta", "n_delta_plain")] + [("piece_split", _u32 * 6), ("phases", _u32)]


def bind(lib) -> None:
    lib.lmz_gpu_struct_sizes.restype = ctypes.c_int
    lib.lmz_gpu_struct_sizes.argtypes = [ctypes.POINTER(ctypes.c_uint * 5)]
    lib.lmz_gpu_piece_bytes.restype = ctypes.c_int
    lib.lmz_gpu_shared_group.restype = ctypes.c_int
    lib.lmz_gpu_delta_job_bytes.restype = ctypes.c_int
    lib.lmz_gpu_crc_tables.restype = ctypes.c_int
    lib.lmz_gpu_crc_tables.argtypes = [_v, ctypes.c_size_t]
    lib.lmz_host_alphabet_sizes.restype = ctypes.c_int
    lib.lmz_host_alphabet_sizes.argtypes = [_v, _v, ctypes.c_size_t, _v]
    lib.lmz_gpu_decode_chunks_dev.restype = ctypes.c_int
    lib.lmz_gpu_decode_chunks_dev.argtypes = [ctypes.POINTER(DecodePlan), _v]
