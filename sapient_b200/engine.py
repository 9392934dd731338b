"""`ForwardEngine` for the CUDA backend: the interface the reference's generation
pipeline drives (crates/sapient-models/src/forward/mod.rs:381-506), implemented by
the resident engine inside libsapient_cuda.so.

    eng = ForwardEngine.from_weights(cfg, weights)      # HF-named weight map
    eng = ForwardEngine.from_gguf("model.gguf")         # GGUF file
    logits = eng.forward_logits(ids, use_cache=True)    # last-position logits, f32 [vocab]

Batched extensions (no counterpart in the single-sequence reference engine):
`forward_slot`, `decode_batch`. Greedy speculative decoding lives in
sapient_b200/speculative.py.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import SapientCudaError, SpModelDesc, check, lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _ids(ids) -> np.ndarray:
    return np.ascontiguousarray(ids, dtype=np.uint32).reshape(-1)


class ForwardEngine:
    def __init__(self, handle, desc: SpModelDesc):
        self._h = handle
        self.desc = desc
        self.vocab = desc.vocab
        rows, first = C.c_int32(), C.c_int32()
        check(lib().sp_cuda_engine_vocab_local(handle, C.byref(rows), C.byref(first)))
        self.vocab_local, self.vocab_first = int(rows.value), int(first.value)  # this rank's slice of the logits
        self._tp_group = None

    # ── construction ────────────────────────────────────────────────────────
    @classmethod
    def from_weights(cls, cfg: dict, weights: dict, device: int = 0, max_batch: int = 1, max_tokens: int = 256,
                     kv_pages: int = 0, tp_rank: int = 0, tp_size: int = 1, fast_large_m: bool = False) -> "ForwardEngine":
        """cfg: arch ('llama'|'qwen2'|'phi2'), n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab,
        max_ctx, rotary_dim (optional), norm_eps, rope_theta. weights: name -> (ggml dtype, dims, uint8 bytes)
        with HF names and [out, in] dims, as the reference's GGUF name map yields. fast_large_m: steps of 17 rows and
        more on the tcgen05 GEMM with operands rounded to fp16 instead of the default exact-class mode (see
        set_large_m_gemm)."""
        d = SpModelDesc()
        d.arch = 1 if cfg["arch"] in ("phi2", "phi") else 0
        d.n_layers, d.hidden, d.n_heads, d.n_kv_heads = cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"]
        d.head_dim, d.ffn, d.vocab, d.max_ctx = cfg["head_dim"], cfg["ffn"], cfg["vocab"], cfg["max_ctx"]
        d.rotary_dim = cfg.get("rotary_dim") or cfg["head_dim"]
        d.norm_eps, d.rope_theta = cfg["norm_eps"], cfg["rope_theta"]
        d.max_batch, d.max_tokens, d.device, d.tp_rank, d.tp_size, d.kv_pages = max_batch, max_tokens, device, tp_rank, tp_size, kv_pages
        h = C.c_void_p()
        check(lib().sp_cuda_engine_create(C.byref(d), C.byref(h)))
        try:
            for name, (dtype, dims, raw) in weights.items():
                if hasattr(raw, "detach"):
                    raw = raw.detach().cpu().numpy()
                raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
                dd = (C.c_int64 * len(dims))(*dims)
                check(lib().sp_cuda_engine_set_tensor(h, name.encode(), dtype, dd, len(dims), _p(raw), raw.size))
            check(lib().sp_cuda_engine_finalize(h))
        except Exception:
            lib().sp_cuda_engine_destroy(h)
            raise
        eng = cls(h, d)
        if fast_large_m:
            eng.set_large_m_gemm(True)
        return eng

    @classmethod
    def from_gguf(cls, path: str, device: int = 0, max_ctx: int = 0, max_batch: int = 1) -> "ForwardEngine":
        h = C.c_void_p()
        check(lib().sp_cuda_engine_from_gguf(str(path).encode(), device, max_ctx, max_batch, C.byref(h)))
        d = SpModelDesc()
        check(lib().sp_cuda_engine_desc(h, C.byref(d)))
        return cls(h, d)

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().sp_cuda_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ── tensor parallelism (one process per GPU) ────────────────────────────
    def tp_handle(self) -> bytes:
        """CUDA IPC handle of this rank's communication block (after finalize)."""
        buf = (C.c_uint8 * _lib.SP_TP_HANDLE_BYTES)()
        check(lib().sp_cuda_engine_tp_handle(self._h, buf, _lib.SP_TP_HANDLE_BYTES))
        return bytes(buf)

    def tp_connect(self, handles=None, group=None) -> None:
        """Map every rank's communication block. Either pass the handles of all ranks in rank order, or a
        torch.distributed process group (default group when both are None) over which they are gathered; with a
        group, logit outputs are gathered to the full vocabulary as well."""
        if handles is None:
            import torch.distributed as dist

            handles = [None] * dist.get_world_size(group)
            dist.all_gather_object(handles, self.tp_handle(), group=group)
            self._tp_group = group if group is not None else dist.group.WORLD
        blob = b"".join(handles)
        if len(blob) != self.desc.tp_size * _lib.SP_TP_HANDLE_BYTES:
            raise SapientCudaError(_lib.SP_ERR_ARG, "tp_connect: one handle per rank expected")
        arr = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(lib().sp_cuda_engine_tp_connect(self._h, arr, self.desc.tp_size))

    def tp_set_wait_ms(self, ms: int) -> None:
        """Bound of the device-side waits on peers (default 5000 ms)."""
        check(lib().sp_cuda_engine_tp_set_wait_ms(self._h, int(ms)))

    def tp_reset(self) -> None:
        """Exchange counters, arrival marks and the sticky error flag back to their initial state. Every rank calls it,
        with a host barrier before and after."""
        check(lib().sp_cuda_engine_tp_reset(self._h))

    @staticmethod
    def nccl_library_path() -> str:
        """The NCCL shared object that torch ships (the copy torch.distributed's nccl backend loads), else the soname."""
        import os

        try:
            import nvidia.nccl as _n

            for base in list(getattr(_n, "__path__", [])):
                cand = os.path.join(base, "lib", "libnccl.so.2")
                if os.path.exists(cand):
                    return cand
        except ImportError:
            pass
        return "libnccl.so.2"

    def tp_nccl_init(self, group=None) -> None:
        """Sets up the library all-reduce arm (comparison with the fused peer push): rank 0 makes the NCCL id, the
        torch.distributed group carries it to the others, every rank joins. Collective over the group."""
        import torch.distributed as dist

        path = self.nccl_library_path().encode()
        box = [None]
        if dist.get_rank(group) == 0:
            buf = C.create_string_buffer(128)
            check(lib().sp_cuda_nccl_unique_id(path, buf, 128))
            box[0] = bytes(buf.raw)
        src = dist.get_global_rank(group, 0) if group is not None else 0
        dist.broadcast_object_list(box, src=src, group=group)
        check(lib().sp_cuda_engine_tp_nccl_init(self._h, path, box[0]))

    def tp_set_allreduce(self, nccl: bool) -> None:
        """False (default): sums of the column-split products by the push fused into the GEMV epilogue; True: through
        ncclAllReduce (after tp_nccl_init). Every rank the same."""
        check(lib().sp_cuda_engine_tp_set_allreduce(self._h, int(bool(nccl))))

    def tp_block(self) -> int:
        """Device address of this rank's communication block (for engines of one process)."""
        p = C.c_void_p()
        check(lib().sp_cuda_engine_tp_block(self._h, C.byref(p)))
        return int(p.value)

    def tp_connect_local(self, blocks) -> None:
        """Connect with the blocks (tp_block() of every rank, in rank order) of engines living in this process."""
        arr = (C.c_void_p * len(blocks))(*blocks)
        check(lib().sp_cuda_engine_tp_connect_local(self._h, arr, len(blocks)))

    def _gather(self, local: np.ndarray) -> np.ndarray:
        """Full-vocabulary logits from the ranks' slices (identity for a single-GPU engine or without a group)."""
        if self.desc.tp_size <= 1 or self._tp_group is None:
            return local
        import torch
        import torch.distributed as dist

        dev = f"cuda:{self.desc.device}" if dist.get_backend(self._tp_group) == "nccl" else "cpu"
        mine = torch.from_numpy(np.ascontiguousarray(local)).to(dev)
        parts = [torch.empty_like(mine) for _ in range(self.desc.tp_size)]
        dist.all_gather(parts, mine, group=self._tp_group)
        return torch.cat(parts, dim=-1).cpu().numpy()

    # ── the reference's ForwardEngine surface ───────────────────────────────
    def forward_logits(self, input_ids, use_cache: bool = True) -> np.ndarray:
        ids = _ids(input_ids)
        if ids.size == 0:
            raise SapientCudaError(_lib.SP_ERR_ARG, "empty input")
        out = np.empty(self.vocab_local, np.float32)
        check(lib().sp_cuda_forward_logits(self._h, _p(ids), ids.size, int(use_cache), _p(out)))
        return self._gather(out)

    def forward_all_logits(self, input_ids) -> np.ndarray:
        ids = _ids(input_ids)
        if ids.size == 0:
            raise SapientCudaError(_lib.SP_ERR_ARG, "empty input")
        out = np.empty((ids.size, self.vocab_local), np.float32)
        check(lib().sp_cuda_forward_all_logits(self._h, _p(ids), ids.size, _p(out)))
        return self._gather(out)

    def forward_all_logits_cached(self, input_ids) -> np.ndarray:
        ids = _ids(input_ids)
        if ids.size == 0:
            raise SapientCudaError(_lib.SP_ERR_ARG, "empty input")
        out = np.empty((ids.size, self.vocab_local), np.float32)
        check(lib().sp_cuda_forward_all_logits_cached(self._h, _p(ids), ids.size, _p(out)))
        return self._gather(out)

    def reset_cache(self, slot: int = -1) -> None:
        check(lib().sp_cuda_reset_cache(self._h, slot))

    def truncate_cache(self, n: int, slot: int = 0) -> int:
        kept = C.c_size_t()
        check(lib().sp_cuda_truncate_cache(self._h, slot, n, C.byref(kept)))
        return int(kept.value)

    def backend_label(self) -> str:
        buf = C.create_string_buffer(64)
        check(lib().sp_cuda_backend_label(self._h, buf, 64))
        return buf.value.decode()

    def is_hybrid(self) -> bool:
        return False

    def embed(self, input_ids):
        raise SapientCudaError(_lib.SP_ERR_ARG, "embed() is not supported by the CUDA engine")

    # ── batched extensions ──────────────────────────────────────────────────
    def seq_len(self, slot: int = 0) -> int:
        n = C.c_size_t()
        check(lib().sp_cuda_seq_len(self._h, slot, C.byref(n)))
        return int(n.value)

    def slot_page(self, slot: int, index: int) -> int:
        """Pool page that holds tokens [16 * index, 16 * index + 16) of `slot`."""
        pg = C.c_int32()
        check(lib().sp_cuda_engine_slot_page(self._h, slot, index, C.byref(pg)))
        return int(pg.value)

    def adopt_prefix(self, slot: int, pages) -> None:
        """Makes the EMPTY `slot` a reader of pool pages that already hold its first 16 * len(pages) tokens."""
        pg = np.ascontiguousarray(pages, dtype=np.int32).reshape(-1)
        check(lib().sp_cuda_engine_adopt_prefix(self._h, slot, _p(pg), pg.size))

    def forward_slot(self, slot: int, input_ids, all_positions: bool = False) -> np.ndarray:
        ids = _ids(input_ids)
        if ids.size == 0:
            raise SapientCudaError(_lib.SP_ERR_ARG, "empty input")
        out = np.empty((ids.size, self.vocab_local) if all_positions else (self.vocab_local,), np.float32)
        check(lib().sp_cuda_forward_slot(self._h, slot, _p(ids), ids.size, int(all_positions), _p(out)))
        return out

    def decode_batch(self, input_ids, slots, want_logits: bool = True, want_argmax: bool = False):
        """One token per sequence slot. Returns (logits [b, vocab] or None, argmax [b] or None)."""
        ids = _ids(input_ids)
        sl = np.ascontiguousarray(slots, dtype=np.int32).reshape(-1)
        assert ids.size == sl.size
        logits = np.empty((ids.size, self.vocab_local), np.float32) if want_logits else None
        am = np.empty(ids.size, np.uint32) if want_argmax else None
        check(lib().sp_cuda_decode_batch(self._h, _p(ids), _p(sl), ids.size, _p(logits) if want_logits else None,
                                         _p(am) if want_argmax else None))
        return logits, am

    def decode_greedy(self, first_ids, slots, steps: int, fetch: bool = True):
        """`steps` greedy decode steps kept on the device. Returns tokens [steps, b] (uint32), or None when
        fetch is False (then call synchronize() before touching the engine again)."""
        ids = _ids(first_ids)
        sl = np.ascontiguousarray(slots, dtype=np.int32).reshape(-1)
        assert ids.size == sl.size
        out = np.empty((steps, ids.size), np.uint32) if fetch else None
        check(lib().sp_cuda_decode_greedy(self._h, _p(ids), _p(sl), ids.size, steps, _p(out) if fetch else None))
        return out

    def set_kv_rounding(self, reference_q8_0: bool) -> None:
        """True (default): new K / V rows go through the reference's Q8_0 cache rounding before the fp16 store;
        False: plain fp16. Only while the cache is empty."""
        check(lib().sp_cuda_engine_set_kv_rounding(self._h, int(reference_q8_0)))

    def synchronize(self) -> None:
        check(lib().sp_cuda_engine_synchronize(self._h))

    def set_graphs(self, on: bool) -> None:
        check(lib().sp_cuda_engine_set_graphs(self._h, int(on)))

    def set_large_m_gemm(self, on) -> None:
        """Steps of 17 rows and more: 2 (default) the tcgen05 GEMM with exact-class operands (leading fp16 part + remainder
        of weights and activations); True / 1 the same GEMM with operands rounded to fp16 (2x faster; final logits of
        full-size models may leave the 2e-2 bar); False / 0 integer-digit GEMV passes of 10 rows."""
        check(lib().sp_cuda_engine_set_large_m_gemm(self._h, int(on)))

    def set_many_row_gemv(self, on: bool) -> None:
        """Steps of 11 rows and more as passes of up to 32 rows on the one-pass GEMV (exact integer products, weights read
        once per pass) instead of passes of 10 rows — for the steps that do not go to the tcgen05 GEMM (11-16 rows, or
        set_large_m_gemm(0))."""
        check(lib().sp_cuda_engine_set_many_row_gemv(self._h, int(on)))

    def set_ring(self, on: bool) -> None:
        """Steps of 1-5 rows on the persistent ring GEMV (opt-in: measured slower) or, the default, on the tile-row GEMV with
        separate producers."""
        check(lib().sp_cuda_engine_set_ring(self._h, int(on)))

    PROFILE_FAMILIES = ("gemv", "attention", "norm", "rope_kv", "elementwise", "embed", "argmax")

    def set_profile(self, on: bool) -> None:
        check(lib().sp_cuda_engine_set_profile(self._h, int(on)))

    def profile_read(self, reset: bool = True) -> dict:
        """{family: (device ms, launches)} accumulated over profiled forwards."""
        ms = np.zeros(8, np.float64)
        n = np.zeros(8, np.uint64)
        k = lib().sp_cuda_engine_profile_read(self._h, _p(ms), _p(n), 8, int(reset))
        return {self.PROFILE_FAMILIES[i]: (float(ms[i]), int(n[i])) for i in range(k)}

    def time_families(self, families, n_tokens: int = 1, reps: int = 20) -> float:
        """Device ms of one decode step restricted to the named kernel families (see PROFILE_FAMILIES; 'all' = whole
        step). The KV entries of the newest positions are undefined afterwards: truncate or reset before reuse."""
        if families == "all":
            mask = (1 << len(self.PROFILE_FAMILIES)) - 1
        else:
            mask = 0
            for f in ([families] if isinstance(families, str) else families):
                mask |= 1 << self.PROFILE_FAMILIES.index(f)
        ms = C.c_float()
        check(lib().sp_cuda_engine_time_families(self._h, mask, n_tokens, reps, C.byref(ms)))
        return float(ms.value)

    def set_stream(self, stream: int) -> None:
        check(lib().sp_cuda_engine_set_stream(self._h, C.c_void_p(stream)))

    def set_trace(self, on: bool) -> None:
        check(lib().sp_cuda_engine_set_trace(self._h, int(on)))

    def layer_out(self, layer: int) -> np.ndarray:
        buf = np.empty(self.desc.max_tokens * self.desc.hidden, np.float32)
        n = C.c_int32()
        check(lib().sp_cuda_debug_layer_out(self._h, layer, _p(buf), buf.size, C.byref(n)))
        return buf[: n.value * self.desc.hidden].reshape(n.value, self.desc.hidden).copy()

    def load_stats(self) -> tuple[float, int]:
        """(seconds spent moving weight bytes to the device, bytes moved)."""
        sec, nb = C.c_double(), C.c_uint64()
        check(lib().sp_cuda_engine_load_stats(self._h, C.byref(sec), C.byref(nb)))
        return float(sec.value), int(nb.value)

    def resident_bytes(self) -> tuple[int, int]:
        w, kv = C.c_uint64(), C.c_uint64()
        check(lib().sp_cuda_engine_resident_bytes(self._h, C.byref(w), C.byref(kv)))
        return int(w.value), int(kv.value)
