"""Speculative decoding on top of two resident engines: a small draft model proposes k tokens one at a
time, the target model verifies all of them in ONE cache-appending forward pass (k rows through the
small-M tensor-core GEMV, one weight stream for the whole batch), rejected tokens are rolled back with
truncate_cache.

Mirrors crates/sapient-generate/src/speculative.rs:
  spec_prefill  :499-513   both models consume the prompt, next-token logits are kept
  spec_round    :523-631   draft, verify, rejection sampling, bonus token, cache reconciliation
  softmax / adjusted_dist / sample_from_probs :635-690

The engines only need forward_logits(ids, use_cache), forward_all_logits_cached(ids) and
truncate_cache(n), i.e. the reference's ForwardEngine surface; ForwardEngine from this package provides
them. The reference draws its uniform numbers from a clock-seeded generator (:692-708), so its runs are
not reproducible; here the caller passes `rand`, a callable returning floats in [0, 1), and `sample`, a
callable (logits, history) -> token id. The defaults are greedy sampling (last maximum wins, as
sampler.rs:161-168) and a seeded generator.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Sequence

import numpy as np


def greedy(logits: np.ndarray, history: Sequence[int] = ()) -> int:
    """argmax with the reference's tie rule: the last maximum wins (Iterator::max_by)."""
    lg = np.asarray(logits)
    return int(np.flatnonzero(lg == lg.max())[-1])


def softmax(logits: np.ndarray) -> np.ndarray:
    """f32 softmax as speculative.rs:635-643 (max-subtracted exp, divided by the sum when it is positive)."""
    lg = np.asarray(logits, dtype=np.float32)
    out = np.exp(lg - lg.max(), dtype=np.float32)
    s = np.float32(out.sum(dtype=np.float32))
    if s > 0:
        out = out / s
    return out.astype(np.float32)


def adjusted_dist(target: np.ndarray, draft: np.ndarray) -> np.ndarray:
    """max(0, target - draft) renormalised; if nothing is left, all mass on the target's best token
    (speculative.rs:647-672, the last maximum wins)."""
    adj = np.maximum(target.astype(np.float32) - draft.astype(np.float32), np.float32(0))
    s = np.float32(adj.sum(dtype=np.float32))
    if s > 1e-9:
        return (adj / s).astype(np.float32)
    adj = np.zeros_like(adj)
    adj[greedy(target)] = 1.0
    return adj


def sample_from_probs(probs: np.ndarray, r: float) -> int:
    """Inverse-CDF draw (speculative.rs:675-690): first index whose running sum exceeds r, else the last index."""
    cum = np.cumsum(probs.astype(np.float32), dtype=np.float32)
    idx = int(np.searchsorted(cum, np.float32(r), side="right"))
    return min(idx, len(probs) - 1)


@dataclass
class SpecState:
    all_tokens: List[int]
    target_next: np.ndarray  # target logits for the token at position committed_len
    draft_next: np.ndarray   # draft logits for the same position
    committed_len: int
    rounds: int = 0
    drafted: int = 0
    accepted_drafts: int = 0
    history: list = field(default_factory=list)  # (drafted, committed) per round


def spec_prefill(target, draft, prompt: Sequence[int]) -> SpecState:
    prompt = [int(t) for t in prompt]
    if not prompt:
        raise ValueError("spec_prefill: empty prompt")
    target_next = np.asarray(target.forward_logits(prompt, True), dtype=np.float32)
    draft_next = np.asarray(draft.forward_logits(prompt, True), dtype=np.float32)
    return SpecState(list(prompt), target_next, draft_next, len(prompt))


def spec_round(target, draft, state: SpecState, k: int, sample: Callable = greedy, rand: Callable[[], float] | None = None,
               eos_ids: Sequence[int] = ()):
    """One round; returns (committed tokens, hit_eos). After it both caches hold exactly the committed tokens."""
    if rand is None:
        raise ValueError("spec_round needs a uniform random source")
    l = state.committed_len
    # 1. draft up to k tokens, extending the draft cache
    drafts: List[int] = []
    dprobs: List[np.ndarray] = []
    dcur = state.draft_next
    for _ in range(k):
        probs = softmax(dcur)
        d = int(sample(dcur, state.all_tokens))
        drafts.append(d)
        dprobs.append(probs)
        if d in eos_ids:
            break
        dcur = np.asarray(draft.forward_logits([d], True), dtype=np.float32)
    m = len(drafts)
    if m == 0:
        return [], False
    # 2. the target scores all m drafts in one cache-appending pass: t_all[i] predicts the token after drafts[i]
    t_all = np.asarray(target.forward_all_logits_cached(drafts), dtype=np.float32).reshape(m, -1)
    # 3. rejection sampling
    accepted: List[int] = []
    rejected = False
    hit_eos = False
    n_draft_ok = 0
    for i in range(m):
        tprobs = softmax(state.target_next if i == 0 else t_all[i - 1])
        d = drafts[i]
        dp = max(float(dprobs[i][d]), 1e-9)
        tp = float(tprobs[d])
        if rand() < min(tp / dp, 1.0):
            accepted.append(d)
            n_draft_ok += 1
            if d in eos_ids:
                hit_eos = True
                rejected = True  # stop after EOS
                break
        else:
            corrected = sample_from_probs(adjusted_dist(tprobs, dprobs[i]), rand())
            accepted.append(corrected)
            rejected = True
            hit_eos = corrected in eos_ids
            break
    # 4. everything accepted: one bonus token from the last target logits
    if not rejected:
        bonus = int(sample(t_all[m - 1], state.all_tokens))
        accepted.append(bonus)
        hit_eos = bonus in eos_ids
    n_acc = len(accepted)
    # 5. reconcile the caches with the committed context
    if not hit_eos:
        if rejected:
            target.truncate_cache(l + n_acc - 1)
        state.target_next = np.asarray(target.forward_logits([accepted[-1]], True), dtype=np.float32)
        # The reference rewinds the draft to l and replays every committed token one by one (:612-618). The
        # draft cache already holds drafts[0 .. m-2]; the accepted ones among them stay, the rest of the
        # committed tokens go through in one call — same committed context, one forward instead of n_acc.
        keep = min(n_draft_ok, m - 1)
        draft.truncate_cache(l + keep)
        state.draft_next = np.asarray(draft.forward_logits(accepted[keep:], True), dtype=np.float32)
    state.all_tokens.extend(accepted)
    state.committed_len = l + n_acc
    state.rounds += 1
    state.drafted += m
    state.accepted_drafts += n_draft_ok
    state.history.append((m, n_acc))
    return accepted, hit_eos


def generate(target, draft, prompt: Sequence[int], max_new_tokens: int, k: int = 4, sample: Callable = greedy,
             rand: Callable[[], float] | None = None, eos_ids: Sequence[int] = (), seed: int = 0):
    """Prefill + rounds until max_new_tokens are committed or an EOS id appears. Returns (new tokens, state)."""
    if rand is None:
        rng = np.random.default_rng(seed)
        rand = lambda: float(rng.random(dtype=np.float32))  # noqa: E731
    state = spec_prefill(target, draft, prompt)
    out: List[int] = []
    while len(out) < max_new_tokens:
        committed, hit_eos = spec_round(target, draft, state, k, sample, rand, eos_ids)
        if not committed:
            break
        out.extend(committed)
        if hit_eos:
            break
    return out[:max_new_tokens], state


# ── greedy speculative decoding: k + 1 rows per verify pass ─────────────────────────────────────────────────────────
@dataclass
class GreedySpecStats:
    rounds: int = 0
    drafted: int = 0
    accepted_drafts: int = 0


def generate_greedy(target, draft, prompt: Sequence[int], max_new_tokens: int, k: int = 4, eos_ids: Sequence[int] = ()):
    """Greedy speculative decoding through the ForwardEngine surface (forward_logits / forward_all_logits_cached /
    truncate_cache), the host-side statement of the schedule sp_cuda_spec_greedy runs inside the library: the token
    committed last is fed to the target TOGETHER with the k drafts (one k + 1 row verify pass per round instead of the
    reference's k-row pass plus a single-token pass, speculative.rs:557,606), drafts are kept while they equal the
    target's arg-max, the target's pick after them is committed too. Works with any engine pair that offers those three calls,
    so the loop inside the library can be checked against it token for token. Returns (new tokens, GreedySpecStats)."""
    prompt = [int(t) for t in prompt]
    if not prompt:
        raise ValueError("generate_greedy: empty prompt")
    target.reset_cache()
    draft.reset_cache()
    st = GreedySpecStats()
    pending = greedy(target.forward_logits(prompt, True))
    draft.forward_logits(prompt, True)
    out: List[int] = [pending] if max_new_tokens > 0 else []
    stop = max_new_tokens == 0 or pending in eos_ids
    length = len(prompt)  # committed tokens held by both caches
    while not stop and len(out) < max_new_tokens:
        drafts: List[int] = []
        tok = pending
        for _ in range(k):
            tok = greedy(draft.forward_logits([tok], True))
            drafts.append(tok)
        logits = np.asarray(target.forward_all_logits_cached([pending] + drafts)).reshape(k + 1, -1)
        picks = [greedy(row) for row in logits]
        n = 0
        while n < k and drafts[n] == picks[n]:
            n += 1
        st.rounds += 1
        st.drafted += k
        st.accepted_drafts += n
        for t in drafts[:n] + [picks[n]]:
            if len(out) >= max_new_tokens or stop:
                break
            out.append(t)
            stop = t in eos_ids
        pending = picks[n]
        target.truncate_cache(length + 1 + n)
        if n < k:
            draft.truncate_cache(length + 1 + n)
        elif not stop and len(out) < max_new_tokens:
            draft.forward_logits([drafts[-1]], True)
        length += 1 + n
    return out, st


def generate_greedy_device(target, draft, prompt: Sequence[int], max_new_tokens: int, k: int = 4, eos_ids: Sequence[int] = ()):
    """The same schedule run by sp_cuda_spec_greedy (CUDA engines of this package only): the draft's greedy loop stays
    on the device and only token ids cross the host boundary. Returns (new tokens, GreedySpecStats)."""
    import ctypes as C

    from ._lib import check, lib

    ids = np.ascontiguousarray(prompt, dtype=np.uint32).reshape(-1)
    eos = np.ascontiguousarray(list(eos_ids), dtype=np.uint32).reshape(-1)
    out = np.zeros(max(max_new_tokens, 1), np.uint32)
    n_out = C.c_size_t()
    stats = np.zeros(3, np.uint64)
    check(lib().sp_cuda_spec_greedy(target._h, draft._h, ids.ctypes.data_as(C.c_void_p), ids.size, k, max_new_tokens,
                                    eos.ctypes.data_as(C.c_void_p) if eos.size else None, eos.size, out.ctypes.data_as(C.c_void_p),
                                    C.byref(n_out), stats.ctypes.data_as(C.c_void_p)))
    return [int(t) for t in out[: n_out.value]], GreedySpecStats(int(stats[0]), int(stats[1]), int(stats[2]))
