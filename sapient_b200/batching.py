"""Continuous batching over the paged KV cache (sp_cuda_batcher_*).

Host-side mirror of the scheduler inside the library: requests are queued with `submit`, every `step` admits what the
page pool can hold, prefills at most `prefill_chunk` prompt tokens and decodes one token of every running sequence.
The reference generates one sequence per engine (crates/sapient-generate/src/pipeline.rs:540-659) and re-uses a prompt
prefix only against the previous turn (pipeline.rs:818-830); batching is on its roadmap (docs/ROADMAP.md:312).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib


@dataclass
class BatcherStats:
    submitted: int
    finished: int
    steps: int
    prefill_tokens: int
    shared_tokens: int
    decode_tokens: int
    evicted_pages: int
    cached_pages: int
    free_pages: int


class ContinuousBatcher:
    def __init__(self, engine, prefill_chunk: int = 256, prefix_cache: bool = True):
        """engine: a finalised ForwardEngine with empty caches; its max_batch is the number of concurrent sequences. Close
        the batcher before the engine."""
        self._h = C.c_void_p()
        self._engine = engine  # keeps the engine alive
        check(lib().sp_cuda_batcher_create(engine._h, int(prefill_chunk), int(bool(prefix_cache)), C.byref(self._h)))

    @classmethod
    def selftest(cls, vocab: int, max_slots: int, max_ctx: int, n_pages: int, prefill_chunk: int = 64, prefix_cache: bool = True):
        """The scheduler over the library's host stand-in (no GPU, no model): for tests of the scheduling logic."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        self._engine = None
        check(lib().sp_cuda_batcher_create_selftest(vocab, max_slots, max_ctx, n_pages, int(prefill_chunk), int(bool(prefix_cache)),
                                                    C.byref(self._h)))
        return self

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().sp_cuda_batcher_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, prompt, max_new: int, eos=()) -> int:
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        e = np.ascontiguousarray(list(eos), dtype=np.uint32)
        rid = C.c_uint64()
        check(lib().sp_cuda_batcher_submit(self._h, p.ctypes.data_as(C.POINTER(C.c_uint32)), p.size, int(max_new),
                                           e.ctypes.data_as(C.POINTER(C.c_uint32)) if e.size else None, int(e.size), C.byref(rid)))
        return int(rid.value)

    def step(self) -> tuple[int, int]:
        """One scheduler iteration; returns (running, waiting) after it."""
        r, w = C.c_int32(), C.c_int32()
        check(lib().sp_cuda_batcher_step(self._h, C.byref(r), C.byref(w)))
        return int(r.value), int(w.value)

    def poll(self, rid: int) -> tuple[np.ndarray, bool]:
        n, fin = C.c_size_t(), C.c_int32()
        check(lib().sp_cuda_batcher_poll(self._h, rid, None, 0, C.byref(n), C.byref(fin)))
        out = np.zeros(max(int(n.value), 1), np.uint32)
        check(lib().sp_cuda_batcher_poll(self._h, rid, out.ctypes.data_as(C.POINTER(C.c_uint32)), out.size, C.byref(n), C.byref(fin)))
        return out[: int(n.value)], bool(fin.value)

    def cancel(self, rid: int) -> None:
        check(lib().sp_cuda_batcher_cancel(self._h, rid))

    def forget(self, rid: int) -> None:
        check(lib().sp_cuda_batcher_forget(self._h, rid))

    def stats(self) -> BatcherStats:
        v = (C.c_uint64 * 9)()
        check(lib().sp_cuda_batcher_stats(self._h, v, 9))
        return BatcherStats(*[int(x) for x in v])

    def run(self, max_steps: int = 1 << 30) -> int:
        """Steps until nothing is running or waiting; returns the number of iterations."""
        n = 0
        while n < max_steps:
            r, w = self.step()
            n += 1
            if r == 0 and w == 0:
                break
        return n
