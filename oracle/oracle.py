"""ctypes front-end of the CPU oracle (oracle/sapient_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the benchmark's
CPU-baseline leg. Nothing under sapient_b200/ may import this module.

Array conventions follow the reference's CPU kernels: activations are float32,
row-major; quantised weights are raw ggml blocks as uint8, row-major [N, K/blk].
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .build import OUT, build_oracle

# ggml type codes (crates/sapient-io/src/gguf.rs:88-129 of the reference).
F32, F16, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 8, 12, 13, 14, 30

_lib = None


class SoModelDesc(C.Structure):
    _fields_ = [
        ("arch", C.c_int32), ("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("max_ctx", C.c_int32), ("rotary_dim", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
        ("kv_mode", C.c_int32),
    ]


def lib():
    global _lib
    if _lib is None:
        path = OUT
        if not os.path.exists(path):
            path = build_oracle()
        L = C.CDLL(path)
        fp, u8p, i64, u32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.c_int64, C.POINTER(C.c_uint32), C.POINTER(C.c_int64)
        vp = C.c_void_p
        sig = {
            "so_dequant": (C.c_int, [C.c_int, vp, i64, vp]),
            "so_byte_count": (i64, [C.c_int, i64]),
            "so_quantize_q8_0": (None, [vp, i64, vp]),
            "so_set_q8_mode": (None, [C.c_int]),
            "so_set_kquant_order": (None, [C.c_int]),
            "so_set_rows_at_once": (None, [C.c_int]),
            "so_dot_row": (C.c_float, [C.c_int, vp, vp, i64]),
            "so_matmul_nt": (C.c_int, [C.c_int, vp, vp, i64, i64, i64, vp]),
            "so_rms_norm": (None, [vp, vp, i64, i64, C.c_float, vp]),
            "so_layer_norm": (None, [vp, vp, vp, i64, i64, C.c_float, vp]),
            "so_rope": (None, [vp, i64, i64, i64, vp, C.c_float, i64, vp]),
            "so_attention": (None, [vp, vp, vp, i64, i64, i64, i64, i64, vp, vp]),
            "so_causal_mask": (None, [i64, i64, vp]),
            "so_silu": (None, [vp, i64, vp]),
            "so_gelu": (None, [vp, i64, vp]),
            "so_add": (None, [vp, vp, i64, vp]),
            "so_mul": (None, [vp, vp, i64, vp]),
            "so_embed": (C.c_int, [C.c_int, vp, i64, i64, vp, i64, vp]),
            "so_argmax": (i64, [vp, i64]),
            "so_unpermute_qk_rows": (None, [vp, i64, i64, i64, vp]),
            "so_f32_to_f16": (C.c_uint16, [C.c_float]),
            "so_f16_to_f32": (C.c_float, [C.c_uint16]),
            "so_kv_create": (vp, [C.c_int, i64, i64, i64]),
            "so_kv_destroy": (None, [vp]),
            "so_kv_update": (i64, [vp, i64, vp, i64, vp]),
            "so_kv_raw_f32": (None, [vp, vp]),
            "so_engine_create": (vp, [C.POINTER(SoModelDesc)]),
            "so_engine_destroy": (None, [vp]),
            "so_engine_set_tensor": (C.c_int, [vp, C.c_char_p, C.c_int, vp, C.c_int, vp, i64]),
            "so_engine_error": (C.c_char_p, [vp]),
            "so_engine_reset_cache": (None, [vp]),
            "so_engine_truncate_cache": (i64, [vp, i64]),
            "so_engine_seq_len": (i64, [vp]),
            "so_engine_forward_logits": (C.c_int, [vp, vp, i64, C.c_int, vp]),
            "so_engine_forward_all_logits": (C.c_int, [vp, vp, i64, C.c_int, vp]),
            "so_engine_trace": (i64, [vp, C.c_int, vp]),
            "so_num_threads": (C.c_int, []),
            "so_set_num_threads": (None, [C.c_int]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        del fp, u8p, u32p, i64p
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def byte_count(dtype: int, numel: int) -> int:
    return int(lib().so_byte_count(dtype, numel))


def dequant(dtype: int, blocks, numel: int) -> np.ndarray:
    b = _u8(blocks).reshape(-1)
    assert b.size == byte_count(dtype, numel), (b.size, byte_count(dtype, numel))
    out = np.empty(numel, np.float32)
    st = lib().so_dequant(dtype, _p(b), numel, _p(out))
    if st != 0:
        raise ValueError(f"unsupported dtype {dtype}")
    return out


def quantize_q8_0(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    assert x.size % 32 == 0
    out = np.empty(x.size // 32 * 34, np.uint8)
    lib().so_quantize_q8_0(_p(x), x.size, _p(out))
    return out


def set_q8_mode(mode: int) -> None:
    """0: the AVX2+FMA Q8_0 row dot (x86_64 default); 1: the portable scalar order."""
    lib().so_set_q8_mode(mode)


def set_kquant_order(mode: int) -> None:
    """0: the reference's evaluation order of the Q4_K / Q6_K row dots (one running accumulator over the row);
    1: per-super-block partial sums added to the row total — a second valid order of the same products, used to
    measure how far two correct implementations drift apart behind a step-function cache quantiser."""
    lib().so_set_kquant_order(mode)


def set_rows_at_once(on: bool) -> None:
    """matmul_nt walks K-quant rows eight at a time (default, bit-identical, faster) or one at a time."""
    lib().so_set_rows_at_once(int(on))


def dot_row(dtype: int, row_blocks, x) -> float:
    r, xx = _u8(row_blocks).reshape(-1), _f32(x).reshape(-1)
    return float(lib().so_dot_row(dtype, _p(r), _p(xx), xx.size))


class OracleError(RuntimeError):
    pass


def matmul_nt(x, w_blocks, dtype: int, n: int) -> np.ndarray:
    """Y[M,N] = X[M,K] · Wᵀ with W given as raw blocks; errors mirror matmul.rs."""
    x = _f32(x)
    if x.ndim != 2:
        raise OracleError("matmul_nt expects 2-D tensors")
    m, k = x.shape
    w = _u8(w_blocks).reshape(-1)
    y = np.empty((m, n), np.float32)
    st = lib().so_matmul_nt(dtype, _p(x), _p(w), m, k, n, _p(y))
    if st == 1:
        raise OracleError("k must be a multiple of the block size")
    if st != 0:
        raise OracleError("unsupported dtype")
    return y


def rms_norm(x, w, eps: float) -> np.ndarray:
    x = _f32(x)
    rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
    y = np.empty_like(x)
    wv = _f32(w) if w is not None else None
    lib().so_rms_norm(_p(x), _p(wv) if wv is not None else None, rows, dim, eps, _p(y))
    return y


def layer_norm(x, w, b, eps: float) -> np.ndarray:
    x = _f32(x)
    rows, dim = int(np.prod(x.shape[:-1])), x.shape[-1]
    y = np.empty_like(x)
    wv = _f32(w) if w is not None else None
    bv = _f32(b) if b is not None else None
    lib().so_layer_norm(_p(x), _p(wv) if wv is not None else None, _p(bv) if bv is not None else None, rows, dim, eps, _p(y))
    return y


def rope(x, positions, base: float, rotary_dim: int | None = None) -> np.ndarray:
    """x: [n_heads, seq, head_dim]."""
    x = _f32(x)
    H, S, D = x.shape
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    assert pos.size == S
    out = np.empty_like(x)
    lib().so_rope(_p(x), H, S, D, _p(pos), base, rotary_dim or D, _p(out))
    return out


def attention(q, k, v, mask=None) -> np.ndarray:
    """q [H, sq, hd]; k, v [Hkv, sk, hd]; mask [sq, sk] additive or None (built-in causal)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    H, sq, hd = q.shape
    Hkv, sk, _ = k.shape
    out = np.empty_like(q)
    mk = _f32(mask) if mask is not None else None
    lib().so_attention(_p(q), _p(k), _p(v), H, Hkv, sq, sk, hd, _p(mk) if mk is not None else None, _p(out))
    return out


def causal_mask(sq: int, sk: int) -> np.ndarray:
    out = np.empty((sq, sk), np.float32)
    lib().so_causal_mask(sq, sk, _p(out))
    return out


def _unary(fn, x):
    x = _f32(x)
    y = np.empty_like(x)
    fn(_p(x), x.size, _p(y))
    return y


def silu(x):
    return _unary(lib().so_silu, x)


def gelu(x):
    return _unary(lib().so_gelu, x)


def add(a, b):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    lib().so_add(_p(a), _p(b), a.size, _p(y))
    return y


def mul(a, b):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    lib().so_mul(_p(a), _p(b), a.size, _p(y))
    return y


def embed(dtype: int, table_bytes, vocab: int, hidden: int, ids) -> np.ndarray:
    t = _u8(table_bytes).reshape(-1)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.empty((ids.size, hidden), np.float32)
    st = lib().so_embed(dtype, _p(t), vocab, hidden, _p(ids), ids.size, _p(out))
    if st == 3:
        raise OracleError("token id out of vocab range")
    if st != 0:
        raise OracleError("unsupported embedding dtype")
    return out


def argmax(v) -> int:
    v = _f32(v).reshape(-1)
    return int(lib().so_argmax(_p(v), v.size))


def unpermute_qk_rows(raw_bytes, n_head: int, head_dim: int, row_bytes: int) -> np.ndarray:
    src = _u8(raw_bytes).reshape(-1)
    assert src.size == n_head * head_dim * row_bytes
    dst = np.empty_like(src)
    lib().so_unpermute_qk_rows(_p(src), n_head, head_dim, row_bytes, _p(dst))
    return dst


def f32_to_f16_bits(f: float) -> int:
    return int(lib().so_f32_to_f16(f))


def f16_bits_to_f32(h: int) -> float:
    return float(lib().so_f16_to_f32(h))


class KvCache:
    """update_kv_cache semantics (forward/common.rs:355-538). kind 0 f32, 1 Q8_0, 2 fp16-rounded."""

    def __init__(self, kind: int, n_kv: int, max_seq: int, hd: int):
        self.kind, self.n_kv, self.max_seq, self.hd = kind, n_kv, max_seq, hd
        self.h = lib().so_kv_create(kind, n_kv, max_seq, hd)

    def update(self, current_seq: int, new_k) -> np.ndarray:
        nk = _f32(new_k)
        new_seq = nk.shape[1]
        total = min(current_seq + new_seq, self.max_seq)
        out = np.empty((self.n_kv, total, self.hd), np.float32)
        t = lib().so_kv_update(self.h, current_seq, _p(nk), new_seq, _p(out))
        if t < 0:
            raise OracleError("new tokens exceed max cache size")
        return out

    def raw_f32(self) -> np.ndarray:
        out = np.empty((self.n_kv, self.max_seq, self.hd), np.float32)
        lib().so_kv_raw_f32(self.h, _p(out))
        return out

    def __del__(self):
        if getattr(self, "h", None):
            lib().so_kv_destroy(self.h)
            self.h = None


class OracleEngine:
    """Whole-model CPU forward mirroring LlamaForward / PhiForward of the reference.

    `weights` maps HF-style names (as produced by the reference's GGUF name map) to
    (ggml dtype code, dims [out, in] or [n], raw bytes).
    """

    def __init__(self, cfg: dict, weights: dict, kv_mode: int = 0):
        d = SoModelDesc()
        d.arch = 1 if cfg.get("arch") in ("phi2", "phi", 1) else 0
        d.n_layers, d.hidden, d.n_heads = cfg["n_layers"], cfg["hidden"], cfg["n_heads"]
        d.n_kv_heads, d.head_dim, d.ffn, d.vocab = cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"]
        d.max_ctx = cfg["max_ctx"]
        d.rotary_dim = cfg.get("rotary_dim") or cfg["head_dim"]
        d.norm_eps, d.rope_theta = cfg["norm_eps"], cfg["rope_theta"]
        d.kv_mode = kv_mode
        self.cfg = cfg
        self.h = lib().so_engine_create(C.byref(d))
        for name, (dtype, dims, raw) in weights.items():
            raw = _u8(raw).reshape(-1)
            dd = (C.c_int64 * len(dims))(*dims)
            st = lib().so_engine_set_tensor(self.h, name.encode(), dtype, dd, len(dims), _p(raw), raw.size)
            if st != 0:
                raise OracleError(self._err())

    def _err(self) -> str:
        return lib().so_engine_error(self.h).decode()

    def forward_logits(self, ids, use_cache: bool = True) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.size == 0:
            raise OracleError("empty input")
        out = np.empty(self.cfg["vocab"], np.float32)
        if lib().so_engine_forward_logits(self.h, _p(ids), ids.size, int(use_cache), _p(out)) != 0:
            raise OracleError(self._err())
        return out

    def forward_all_logits(self, ids) -> np.ndarray:
        return self._all(ids, 0)

    def forward_all_logits_cached(self, ids) -> np.ndarray:
        return self._all(ids, 1)

    def _all(self, ids, cached: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        if ids.size == 0:
            raise OracleError("empty input")
        out = np.empty((ids.size, self.cfg["vocab"]), np.float32)
        if lib().so_engine_forward_all_logits(self.h, _p(ids), ids.size, cached, _p(out)) != 0:
            raise OracleError(self._err())
        return out

    def reset_cache(self) -> None:
        lib().so_engine_reset_cache(self.h)

    def truncate_cache(self, n: int) -> int:
        return int(lib().so_engine_truncate_cache(self.h, n))

    @property
    def seq_len(self) -> int:
        return int(lib().so_engine_seq_len(self.h))

    def trace(self, layer: int) -> np.ndarray:
        """Hidden state after `layer` from the most recent forward, [seq, hidden]."""
        s = int(lib().so_engine_trace(self.h, layer, None))
        if s < 0:
            raise OracleError("no trace")
        buf = np.empty((s, self.cfg["hidden"]), np.float32)
        lib().so_engine_trace(self.h, layer, _p(buf))
        return buf

    def __del__(self):
        if getattr(self, "h", None):
            lib().so_engine_destroy(self.h)
            self.h = None


def num_threads() -> int:
    return int(lib().so_num_threads())


def set_num_threads(n: int) -> None:
    """Thread count of the oracle's parallel loops (the reference sizes its pool to all cores,
    crates/sapient-backends/cpu/src/pool.rs). Launchers that export OMP_NUM_THREADS=1 would otherwise pin it to one."""
    lib().so_set_num_threads(int(n))


def use_all_cores() -> int:
    """Sets the thread count to the cores this process may run on and returns it."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    set_num_threads(n)
    return num_threads()
