"""ctypes binding of libsapient_cuda.so (the C ABI declared in include/sapient_cuda.h).

There is no CPU fallback: if the library is missing or has no CUDA device to run on,
the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsapient_cuda.so")

# status codes of include/sapient_cuda.h
SP_OK, SP_ERR_SHAPE, SP_ERR_DTYPE, SP_ERR_OOM, SP_ERR_CUDA, SP_ERR_KV_FULL = 0, 1, 2, 3, 4, 5
SP_ERR_COMM, SP_ERR_ARG, SP_ERR_VOCAB, SP_ERR_STATE, SP_ERR_IO = 6, 7, 8, 9, 10
SP_TP_HANDLE_BYTES = 64  # sizeof(cudaIpcMemHandle_t)


class SapientCudaError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"[status {status}] {msg}")
        self.status = status


class SpModelDesc(C.Structure):
    _fields_ = [
        ("arch", C.c_int32), ("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("max_ctx", C.c_int32), ("rotary_dim", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
        ("max_batch", C.c_int32), ("max_tokens", C.c_int32), ("device", C.c_int32), ("tp_rank", C.c_int32),
        ("tp_size", C.c_int32), ("kv_pages", C.c_int64),
    ]


_vp, _i32, _i64, _sz, _f = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); must list every symbol include/sapient_cuda.h declares
SIGNATURES = {
    "sp_cuda_last_error": (C.c_char_p, []),
    "sp_cuda_device_count": (_i32, []),
    "sp_cuda_upload_weight": (_i32, [_i32, _i32, _i64, _i64, _vp, _sz, C.POINTER(_vp)]),
    "sp_cuda_free_weight": (None, [_vp]),
    "sp_cuda_dequant": (_i32, [_vp, _vp]),
    "sp_cuda_matmul_nt": (_i32, [_vp, _vp, _i64, _vp]),
    "sp_cuda_matmul_nt_dev": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "sp_cuda_check_kernels": (_i32, [_i32]),
    "sp_cuda_set_gemv_path": (_i32, [_i32]),
    "sp_cuda_set_activation_digits": (_i32, [_i32]),
    "sp_cuda_weight_info": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_sz)]),
    "sp_cuda_rms_norm": (_i32, [_i32, _vp, _vp, _i64, _i64, _f, _vp]),
    "sp_cuda_layer_norm": (_i32, [_i32, _vp, _vp, _vp, _i64, _i64, _f, _vp]),
    "sp_cuda_rope": (_i32, [_i32, _vp, _i64, _i64, _i64, _vp, _f, _i64, _vp]),
    "sp_cuda_attention": (_i32, [_i32, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "sp_cuda_attention_paged_static": (_i32, [_i32, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _i32,
                                              _i32, _i32, _vp]),
    "sp_cuda_engine_set_kv_rounding": (_i32, [_vp, _i32]),
    "sp_cuda_engine_tp_handle": (_i32, [_vp, _vp, C.c_size_t]),
    "sp_cuda_engine_tp_connect": (_i32, [_vp, _vp, _i32]),
    "sp_cuda_engine_vocab_local": (_i32, [_vp, _vp, _vp]),
    "sp_cuda_engine_tp_set_wait_ms": (_i32, [_vp, _i32]),
    "sp_cuda_nccl_unique_id": (_i32, [C.c_char_p, _vp, C.c_size_t]),
    "sp_cuda_engine_tp_nccl_init": (_i32, [_vp, C.c_char_p, _vp]),
    "sp_cuda_engine_tp_set_allreduce": (_i32, [_vp, _i32]),
    "sp_cuda_engine_tp_reset": (_i32, [_vp]),
    "sp_cuda_engine_tp_block": (_i32, [_vp, _vp]),
    "sp_cuda_engine_tp_connect_local": (_i32, [_vp, _vp, _i32]),
    "sp_cuda_tp_shard": (_i32, [C.c_char_p, _i32, _vp, _i32, _vp, C.c_size_t, _i32, _i32, _i64, _vp, C.c_size_t, _vp, _vp]),
    "sp_cuda_set_large_m_gemm": (_i32, [_i32]),
    "sp_cuda_silu": (_i32, [_i32, _vp, _i64, _vp]),
    "sp_cuda_gelu": (_i32, [_i32, _vp, _i64, _vp]),
    "sp_cuda_add": (_i32, [_i32, _vp, _vp, _i64, _vp]),
    "sp_cuda_mul": (_i32, [_i32, _vp, _vp, _i64, _vp]),
    "sp_cuda_embed": (_i32, [_vp, _vp, _i64, _vp]),
    "sp_cuda_argmax": (_i32, [_i32, _vp, _i64, _i64, _vp]),
    "sp_cuda_engine_create": (_i32, [C.POINTER(SpModelDesc), C.POINTER(_vp)]),
    "sp_cuda_engine_set_tensor": (_i32, [_vp, C.c_char_p, _i32, _vp, _i32, _vp, _sz]),
    "sp_cuda_engine_finalize": (_i32, [_vp]),
    "sp_cuda_engine_from_gguf": (_i32, [C.c_char_p, _i32, _i32, _i32, C.POINTER(_vp)]),
    "sp_cuda_engine_desc": (_i32, [_vp, C.POINTER(SpModelDesc)]),
    "sp_cuda_engine_destroy": (None, [_vp]),
    "sp_cuda_engine_set_stream": (_i32, [_vp, _vp]),
    "sp_cuda_forward_logits": (_i32, [_vp, _vp, _sz, _i32, _vp]),
    "sp_cuda_forward_all_logits": (_i32, [_vp, _vp, _sz, _vp]),
    "sp_cuda_forward_all_logits_cached": (_i32, [_vp, _vp, _sz, _vp]),
    "sp_cuda_forward_slot": (_i32, [_vp, _i32, _vp, _sz, _i32, _vp]),
    "sp_cuda_decode_batch": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp]),
    "sp_cuda_decode_greedy": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp]),
    "sp_cuda_spec_greedy": (_i32, [_vp, _vp, _vp, _sz, _i32, _sz, _vp, _i32, _vp, C.POINTER(_sz), _vp]),
    "sp_cuda_engine_synchronize": (_i32, [_vp]),
    "sp_cuda_engine_set_graphs": (_i32, [_vp, _i32]),
    "sp_cuda_engine_set_ring": (_i32, [_vp, _i32]),
    "sp_cuda_engine_set_many_row_gemv": (_i32, [_vp, _i32]),
    "sp_cuda_engine_set_large_m_gemm": (_i32, [_vp, _i32]),
    "sp_cuda_engine_set_profile": (_i32, [_vp, _i32]),
    "sp_cuda_engine_profile_read": (_i32, [_vp, _vp, _vp, _i32, _i32]),
    "sp_cuda_engine_time_families": (_i32, [_vp, C.c_uint32, _i32, _i32, C.POINTER(C.c_float)]),
    "sp_cuda_reset_cache": (_i32, [_vp, _i32]),
    "sp_cuda_truncate_cache": (_i32, [_vp, _i32, _sz, C.POINTER(_sz)]),
    "sp_cuda_seq_len": (_i32, [_vp, _i32, C.POINTER(_sz)]),
    "sp_cuda_backend_label": (_i32, [_vp, C.c_char_p, _sz]),
    "sp_cuda_engine_set_trace": (_i32, [_vp, _i32]),
    "sp_cuda_debug_layer_out": (_i32, [_vp, _i32, _vp, _sz, C.POINTER(_i32)]),
    "sp_cuda_launch_count": (C.c_uint64, []),
    "sp_cuda_engine_resident_bytes": (_i32, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "sp_cuda_engine_slot_page": (_i32, [_vp, _i32, _i32, C.POINTER(_i32)]),
    "sp_cuda_engine_adopt_prefix": (_i32, [_vp, _i32, _vp, _i32]),
    "sp_cuda_batcher_create": (_i32, [_vp, _i32, _i32, C.POINTER(_vp)]),
    "sp_cuda_batcher_create_selftest": (_i32, [_i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(_vp)]),
    "sp_cuda_batcher_destroy": (None, [_vp]),
    "sp_cuda_batcher_submit": (_i32, [_vp, C.POINTER(C.c_uint32), C.c_size_t, C.c_size_t, C.POINTER(C.c_uint32), _i32, C.POINTER(C.c_uint64)]),
    "sp_cuda_batcher_step": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_i32)]),
    "sp_cuda_batcher_poll": (_i32, [_vp, C.c_uint64, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_size_t), C.POINTER(_i32)]),
    "sp_cuda_batcher_cancel": (_i32, [_vp, C.c_uint64]),
    "sp_cuda_batcher_forget": (_i32, [_vp, C.c_uint64]),
    "sp_cuda_batcher_stats": (_i32, [_vp, C.POINTER(C.c_uint64), _i32]),
    "sp_cuda_engine_load_stats": (_i32, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
}

_lib = None


def lib():
    """Loads the library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m sapient_b200.build` (needs nvcc). "
                "This package has no CPU fallback."
            )
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != SP_OK:
        raise SapientCudaError(status, lib().sp_cuda_last_error().decode(errors="replace"))
