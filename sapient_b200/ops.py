"""Per-op interface of the CUDA backend on host (numpy) buffers, mirroring the
reference's `LlmBackend` trait (crates/sapient-models/src/forward/backend.rs:57-115)
and the resident-weight kernel API of its GPU context
(crates/sapient-backends/wgpu/src/quant.rs:94-480). Every call goes through the C ABI.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import SapientCudaError, check, lib

F32, F16, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 8, 12, 13, 14, 30


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class Weight:
    """A [n, k] matrix of raw ggml blocks resident on the device (upload_q8_0 / upload_q4_k / upload_q6_k)."""

    def __init__(self, dtype: int, n: int, k: int, blocks, device: int = 0):
        raw = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        h = C.c_void_p()
        check(lib().sp_cuda_upload_weight(device, dtype, n, k, _p(raw), raw.size, C.byref(h)))
        self.h, self.dtype, self.n, self.k, self.device, self.nbytes = h, dtype, n, k, device, raw.size

    def dequant(self) -> np.ndarray:
        """Tensor::to_f32_vec — bit-exact f32 values, shape [n, k]."""
        out = np.empty((self.n, self.k), np.float32)
        check(lib().sp_cuda_dequant(self.h, _p(out)))
        return out

    def matmul_nt(self, x) -> np.ndarray:
        """Y[m, n] = X[m, k] · Wᵀ (kernels::matmul::matmul_nt) with host buffers."""
        x = _f32(x)
        if x.ndim != 2:
            raise SapientCudaError(_lib.SP_ERR_SHAPE, "matmul_nt expects 2-D tensors")
        if x.shape[1] != self.k:
            raise SapientCudaError(_lib.SP_ERR_SHAPE, f"shape mismatch: expected [{x.shape[0]}, {x.shape[1]}] got [{self.n}, {self.k}]")
        y = np.empty((x.shape[0], self.n), np.float32)
        check(lib().sp_cuda_matmul_nt(self.h, _p(x), x.shape[0], _p(y)))
        return y

    def matmul_nt_dev(self, x_ptr: int, m: int, y_ptr: int, stream: int = 0) -> None:
        """Device-pointer variant (no copies, no synchronisation)."""
        check(lib().sp_cuda_matmul_nt_dev(self.h, C.c_void_p(x_ptr), m, C.c_void_p(y_ptr), C.c_void_p(stream)))

    def embed(self, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)
        out = np.empty((ids.size, self.k), np.float32)
        check(lib().sp_cuda_embed(self.h, _p(ids), ids.size, _p(out)))
        return out

    def free(self) -> None:
        if getattr(self, "h", None):
            lib().sp_cuda_free_weight(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def matmul_nt(x, blocks, dtype: int, n: int, device: int = 0) -> np.ndarray:
    x = _f32(x)
    if x.ndim != 2:
        raise SapientCudaError(_lib.SP_ERR_SHAPE, "matmul_nt expects 2-D tensors")
    w = Weight(dtype, n, x.shape[1], blocks, device)
    try:
        return w.matmul_nt(x)
    finally:
        w.free()


def rms_norm(x, w, eps: float, device: int = 0) -> np.ndarray:
    x = _f32(x)
    rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
    y = np.empty_like(x)
    wv = _f32(w) if w is not None else None
    check(lib().sp_cuda_rms_norm(device, _p(x), _p(wv) if wv is not None else None, rows, dim, eps, _p(y)))
    return y


def layer_norm(x, w, b, eps: float, device: int = 0) -> np.ndarray:
    x = _f32(x)
    rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
    y = np.empty_like(x)
    wv = _f32(w) if w is not None else None
    bv = _f32(b) if b is not None else None
    check(lib().sp_cuda_layer_norm(device, _p(x), _p(wv) if wv is not None else None, _p(bv) if bv is not None else None,
                                   rows, dim, eps, _p(y)))
    return y


def rope(x, positions, base: float, rotary_dim: int | None = None, device: int = 0) -> np.ndarray:
    """apply_rope_positions / apply_rope_partial on x [n_heads, seq, head_dim]."""
    x = _f32(x)
    H, S, D = x.shape
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    if pos.size != S:
        raise SapientCudaError(_lib.SP_ERR_SHAPE, "positions length must match seq_len")
    y = np.empty_like(x)
    check(lib().sp_cuda_rope(device, _p(x), H, S, D, _p(pos), base, D if rotary_dim is None else rotary_dim, _p(y)))
    return y


def gqa_attention(q, k, v, device: int = 0) -> np.ndarray:
    """Causal GQA attention: q [H, sq, hd], k/v [Hkv, sk, hd] -> [H, sq, hd]. K/V are held as fp16 on the device."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    H, sq, hd = q.shape
    Hkv, sk, _ = k.shape
    out = np.empty_like(q)
    check(lib().sp_cuda_attention(device, _p(q), _p(k), _p(v), H, Hkv, sq, sk, hd, _p(out)))
    return out


def _unary(fn, x, device):
    x = _f32(x)
    y = np.empty_like(x)
    check(fn(device, _p(x), x.size, _p(y)))
    return y


def silu(x, device: int = 0):
    return _unary(lib().sp_cuda_silu, x, device)


def gelu(x, device: int = 0):
    return _unary(lib().sp_cuda_gelu, x, device)


def add(a, b, device: int = 0):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    check(lib().sp_cuda_add(device, _p(a), _p(b), a.size, _p(y)))
    return y


def mul(a, b, device: int = 0):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    check(lib().sp_cuda_mul(device, _p(a), _p(b), a.size, _p(y)))
    return y


def argmax(logits, device: int = 0) -> np.ndarray:
    """Row-wise argmax; ties resolve to the last maximum (Sampler's greedy rule)."""
    x = _f32(logits)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.empty(x2.shape[0], np.uint32)
    check(lib().sp_cuda_argmax(device, _p(x2), x2.shape[0], x2.shape[1], _p(out)))
    return out


def set_gemv_path(path: int) -> None:
    """0: tensor-core GEMV on tile-repacked weights (default); 1: CUDA-core GEMV on raw blocks; 3: per-warp streaming
    variant; 4: bulk-copy ring GEMV for calls of 1-5 rows."""
    check(lib().sp_cuda_set_gemv_path(path))


LARGE_M_DEFAULT = 2


def set_large_m_gemm(on) -> None:
    """Op-level matmuls with m >= 17 and k % 256 == 0: 2 (default) the tcgen05 / TMEM dequant GEMM with exact-class (leading
    part + remainder) operands; 1 / True the same GEMM with operands rounded to fp16; 0 / False exact integer-digit passes
    on the mma.sync kernels."""
    check(lib().sp_cuda_set_large_m_gemm(int(on)))


def launch_count() -> int:
    return int(lib().sp_cuda_launch_count())
