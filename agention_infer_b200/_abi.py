"""ctypes binding of the C ABI declared in include/agention_b200.h.

Loading fails loudly when libagention_b200.so is missing or cannot be loaded:
there is no Python or CPU substitute for the CUDA library.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libagention_b200.so"

AGN_OK, AGN_EINVAL, AGN_EUNSUPPORTED_DTYPE, AGN_ECUDA, AGN_EOOB_ID, AGN_ENOMEM, AGN_ETIMEOUT = range(7)
AGN_EFORMAT, AGN_ENOTFOUND, AGN_EIO = 7, 8, 9
AGN_F32, AGN_F16, AGN_Q8_0, AGN_Q4_K, AGN_Q6_K, AGN_BF16 = 0, 1, 8, 12, 14, 30
AGN_KV_Q8_0_WORDS = 1008  # a KV-cache layout (the GPU path's 36-byte Q8_0 blocks), not a GgmlType
AGN_Q5_0, AGN_Q5_K, AGN_Q2_K = 6, 13, 10
AGN_ROPE_NEOX, AGN_ROPE_NORMAL = 0, 1

_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)


class TensorInfo(C.Structure):
    """agn_tensor_info"""
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_int32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4),
                ("byte_offset", C.c_uint64), ("file_offset", C.c_uint64), ("n_rows", C.c_uint64), ("row_len", C.c_uint64),
                ("row_bytes", C.c_uint64), ("n_bytes", C.c_uint64)]


_pti = C.POINTER(TensorInfo)

# name -> (restype, argtypes); must list every AGN_API symbol of the header
SIGNATURES = {
    "agn_ctx_create": (_i32, [_i32, _pp]),
    "agn_ctx_destroy": (_i32, [_vp]),
    "agn_backend_name": (C.c_char_p, []),
    "agn_last_error": (C.c_char_p, [_vp]),
    "agn_status_string": (C.c_char_p, [_i32]),
    "agn_ctx_set_stream": (_i32, [_vp, _vp]),
    "agn_ctx_get_stream": (_i32, [_vp, _pp]),
    "agn_ctx_launch_count": (C.c_uint64, [_vp]),
    "agn_ctx_last_kernel": (C.c_char_p, [_vp]),
    "agn_launch_noop": (_i32, [_vp]),
    "agn_graph_begin": (_i32, [_vp]),
    "agn_graph_end": (_i32, [_vp, _pp]),
    "agn_graph_launch": (_i32, [_vp, _vp]),
    "agn_graph_destroy": (_i32, [_vp, _vp]),
    "agn_ctx_set_option": (_i32, [_vp, C.c_char_p, _i64]),
    "agn_malloc": (_i32, [_vp, _sz, _pp]),
    "agn_free": (_i32, [_vp, _vp]),
    "agn_host_alloc": (_i32, [_vp, _sz, _pp]),
    "agn_host_free": (_i32, [_vp, _vp]),
    "agn_memcpy_h2d": (_i32, [_vp, _vp, _vp, _sz]),
    "agn_memcpy_d2h": (_i32, [_vp, _vp, _vp, _sz]),
    "agn_memset": (_i32, [_vp, _vp, C.c_int, _sz]),
    "agn_sync": (_i32, [_vp]),
    "agn_event_create": (_i32, [_vp, _pp]),
    "agn_event_record": (_i32, [_vp, _vp]),
    "agn_event_elapsed_ms": (_i32, [_vp, _vp, _vp, C.POINTER(C.c_float)]),
    "agn_event_destroy": (_i32, [_vp, _vp]),
    "agn_rms_norm_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_add_residual_rms_norm_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_rope_f32": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _i32, _f32, _f32, _i32]),
    "agn_rope_qk_f32": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _i32, _f32, _f32, _i32]),
    "agn_qk_norm_rope_f32": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _f32, _i32, _vp, _i32, _f32, _f32, _i32]),
    "agn_qk_norm_rope_qk_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _i32,
                                       _f32, _f32, _i32]),
    "agn_silu_mul_f32": (_i32, [_vp, _vp, _vp, _vp, _i64]),
    "agn_softmax_rows_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _i32]),
    "agn_softmax_rows_unnorm_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _i32]),
    "agn_get_rows_f32": (_i32, [_vp, _i32, _vp, _sz, _i64, _i64, _vp, _i64, _vp]),
    "agn_kv_write_f32": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _i32, _i64]),
    "agn_kv_read_f32": (_i32, [_vp, _i32, _vp, _vp, _i64, _i64, _vp, _vp]),
    "agn_kv_bytes_per_token": (_i64, [_i32, _i64]),
    "agn_router_top2_f32": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "agn_gather_rows_by_expert_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp, _vp]),
    "agn_silu_mul_f16": (_i32, [_vp, _vp, _vp, _vp, _i64]),
    "agn_softmax_rows_scaled_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _i32, _f32]),
    "agn_qk_norm_rope_kv_write_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _i32, _f32, _f32,
                                             _i32, _i32, _vp, _vp, _i64]),
    "agn_softmax_rows_scaled_f32_out16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _i32, _f32, _i32]),
    "agn_softmax_rows_valid_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _i32, _f32, _i32]),
    "agn_silu_mul_f32_out16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32]),
    "agn_rms_norm_f32_out16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32]),
    "agn_add_residual_rms_norm_f32_out16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32]),
    "agn_q8_k_blocks": (_i64, [_i64]),
    "agn_quantize_rows_q8_k_f32": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "agn_rms_norm_q8_k_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp]),
    "agn_add_residual_rms_norm_q8_k_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp]),
    "agn_silu_mul_q8_k_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "agn_rms_norm_f16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_add_residual_rms_norm_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_rope_qk_f16": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _i32, _f32, _f32, _i32]),
    "agn_qk_norm_rope_qk_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _i32, _f32,
                                       _f32, _i32]),
    "agn_get_rows_f16": (_i32, [_vp, _i32, _vp, _sz, _i64, _i64, _vp, _i64, _vp]),
    "agn_host_rms_norm_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_host_add_residual_rms_norm_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "agn_host_silu_mul_f32": (_i32, [_vp, _vp, _vp, _vp, _i64]),
    "agn_host_rope_qk_f32": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _i32, _f32, _f32, _i32]),
    "agn_host_qk_norm_rope_qk_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _i32, _vp, _i32,
                                            _f32, _f32, _i32]),
    "agn_host_softmax_rows_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _i32, _i32]),
    "agn_host_quantize_rows_q8_k_f32": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "agn_host_get_rows_f32": (_i32, [_vp, _i32, _vp, _sz, _i64, _i64, _vp, _i64, _vp]),
    "agn_gather_rows_by_expert_noalloc_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp, _vp, C.c_char_p,
                                                     _sz]),
    "agn_rope_freq_scale": (_i32, [C.c_char_p, _i32, _f32, _vp]),
    "agn_gguf_parse": (_i32, [_vp, _sz, _pp, C.c_char_p, _sz]),
    "agn_gguf_split_index": (_i32, [C.c_char_p, _vp, _vp]),
    "agn_gguf_open": (_i32, [C.c_char_p, _pp, C.c_char_p, _sz]),
    "agn_gguf_close": (_i32, [_vp]),
    "agn_gguf_version": (C.c_uint32, [_vp]),
    "agn_gguf_tensor_count": (C.c_uint64, [_vp]),
    "agn_gguf_metadata_count": (C.c_uint64, [_vp]),
    "agn_gguf_data_offset": (C.c_uint64, [_vp]),
    "agn_gguf_get_u64": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "agn_gguf_get_f32": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    "agn_gguf_get_string": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_char_p)]),
    "agn_gguf_get_array_i64": (_i32, [_vp, C.c_char_p, _vp, C.c_uint64, _vp]),
    "agn_gguf_get_array_info": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "agn_gguf_tensor_at": (_i32, [_vp, C.c_uint64, _pti]),
    "agn_gguf_find_tensor": (_i32, [_vp, C.c_char_p, _pti]),
    "agn_gguf_upload_tensor": (_i32, [_vp, _vp, C.c_char_p, _pp, _pti]),
    "agn_gguf_upload_tensors": (_i32, [_vp, _vp, C.POINTER(C.c_char_p), C.c_uint64, C.POINTER(C.c_void_p), _pti, _i32,
                                       C.POINTER(C.c_uint64)]),
    "agn_gguf_tensor_data": (_i32, [_vp, C.c_char_p, _pp, C.POINTER(C.c_uint64)]),
    "agn_gguf_release_pages": (_i32, [_vp, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64)]),
    "agn_type_size": (_sz, [_i32, _sz]),
}

_lib = None


def load() -> C.CDLL:
    """dlopen the CUDA library and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m agention_infer_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
