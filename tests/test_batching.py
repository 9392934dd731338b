"""Continuous batching scheduler (sp_cuda_batcher_*): the scheduling logic on the library's host stand-in (no GPU), then
the same properties on the CUDA engine.

Stand-in model: the next token after a sequence is FNV-1a-64 of its token ids modulo the vocabulary, computed from what
the page tables hold — a wrongly shared, recycled or overwritten page changes it. The property throughout: whatever
the arrival pattern, chunking, sharing and eviction, every request's tokens equal the generation of its prompt alone.
"""
import numpy as np
import pytest

from sapient_b200._lib import SapientCudaError
from sapient_b200.batching import ContinuousBatcher

VOCAB = 1000


def _next(tokens):
    h = 0xCBF29CE484222325
    for t in tokens:
        for b in range(4):
            h ^= (int(t) >> (8 * b)) & 0xFF
            h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h % VOCAB


def _alone(prompt, max_new, eos=()):
    seq, out = list(prompt), []
    while len(out) < max_new:
        t = _next(seq)
        out.append(t)
        if t in eos:
            break
        seq.append(t)
    return out


def _drain(b, ids, max_steps=100000):
    b.run(max_steps)
    res = {}
    for rid in ids:
        toks, fin = b.poll(rid)
        assert fin
        res[rid] = toks.tolist()
    return res


def test_requests_of_mixed_lengths_match_their_solo_generations():
    rng = np.random.default_rng(0)
    b = ContinuousBatcher.selftest(VOCAB, max_slots=4, max_ctx=256, n_pages=40, prefill_chunk=24, prefix_cache=False)
    want = {}
    for i in range(13):
        p = rng.integers(0, VOCAB, int(rng.integers(1, 90))).tolist()
        mn = int(rng.integers(1, 40))
        want[b.submit(p, mn)] = _alone(p, mn)
    got = _drain(b, want)
    assert got == want
    s = b.stats()
    assert s.finished == 13 and s.shared_tokens == 0 and s.cached_pages == 0
    assert s.free_pages == 40  # everything returned
    assert s.decode_tokens + 13 == sum(len(v) for v in want.values())  # the first token of each comes from the prefill
    b.close()


def test_arrivals_while_running_and_slots_are_refilled_at_once():
    rng = np.random.default_rng(1)
    b = ContinuousBatcher.selftest(VOCAB, max_slots=2, max_ctx=128, n_pages=16, prefill_chunk=16, prefix_cache=False)
    p0, p1, p2 = (rng.integers(0, VOCAB, n).tolist() for n in (5, 7, 9))
    a = b.submit(p0, 30)
    c = b.submit(p1, 4)
    assert b.step() == (2, 0)
    late = b.submit(p2, 4)  # arrives while both slots are busy
    running, waiting = b.step()
    assert (running, waiting) == (2, 1)
    # c finishes after 4 tokens; the very next iteration runs the late request in its slot while a still decodes
    seen_late_running = False
    for _ in range(40):
        running, waiting = b.step()
        if not b.poll(a)[1] and len(b.poll(late)[0]) > 0:
            seen_late_running = True
        if running == 0 and waiting == 0:
            break
    assert seen_late_running
    assert b.poll(a)[0].tolist() == _alone(p0, 30)
    assert b.poll(c)[0].tolist() == _alone(p1, 4)
    assert b.poll(late)[0].tolist() == _alone(p2, 4)
    b.close()


def test_shared_prompt_prefix_is_computed_once():
    rng = np.random.default_rng(2)
    system = rng.integers(0, VOCAB, 70).tolist()  # 4 whole pages + 6 tokens
    b = ContinuousBatcher.selftest(VOCAB, max_slots=3, max_ctx=256, n_pages=64, prefill_chunk=32, prefix_cache=True)
    first = b.submit(system + [1, 2, 3], 5)
    b.run()
    base = b.stats()
    assert base.prefill_tokens == 73 and base.shared_tokens == 0 and base.cached_pages >= 4
    want = {first: _alone(system + [1, 2, 3], 5)}
    ids = []
    for i in range(6):
        p = system + rng.integers(0, VOCAB, 1 + i).tolist()
        rid = b.submit(p, 6)
        want[rid] = _alone(p, 6)
        ids.append(rid)
    got = _drain(b, want)
    assert got == want
    s = b.stats()
    assert s.shared_tokens == 6 * 64  # four pages each
    assert s.prefill_tokens - base.prefill_tokens == sum(70 + 1 + i - 64 for i in range(6))
    b.close()


def test_a_prompt_that_is_entirely_indexed_still_computes_its_last_token():
    p = list(range(100, 132))  # exactly two pages
    b = ContinuousBatcher.selftest(VOCAB, max_slots=2, max_ctx=128, n_pages=32, prefill_chunk=64)
    a = b.submit(p, 20)
    b.run()
    c = b.submit(p, 20)
    b.run()
    assert b.poll(a)[0].tolist() == b.poll(c)[0].tolist() == _alone(p, 20)
    s = b.stats()
    assert s.shared_tokens == 16  # one page shared, the second recomputed: its last token's logits are needed
    b.close()


def test_concurrent_requests_share_a_prefix_that_is_still_being_decoded():
    rng = np.random.default_rng(3)
    system = rng.integers(0, VOCAB, 48).tolist()
    b = ContinuousBatcher.selftest(VOCAB, max_slots=4, max_ctx=256, n_pages=64, prefill_chunk=64)
    a = b.submit(system + [7], 50)
    b.step()  # prefilled, indexed, now decoding
    others = [b.submit(system + [8 + i], 10) for i in range(3)]
    b.run()
    assert b.stats().shared_tokens == 3 * 48
    assert b.poll(a)[0].tolist() == _alone(system + [7], 50)
    for i, rid in enumerate(others):
        assert b.poll(rid)[0].tolist() == _alone(system + [8 + i], 10)
    b.close()


def test_index_pages_are_evicted_when_the_pool_is_short_and_results_stay_right():
    rng = np.random.default_rng(4)
    b = ContinuousBatcher.selftest(VOCAB, max_slots=2, max_ctx=128, n_pages=12, prefill_chunk=64)
    want = {}
    for i in range(10):  # ten unrelated prompts of 3-4 pages each: the index fills the pool, later requests force eviction
        p = rng.integers(0, VOCAB, int(rng.integers(40, 60))).tolist()
        want[b.submit(p, 8)] = _alone(p, 8)
    got = _drain(b, want)
    assert got == want
    s = b.stats()
    assert s.evicted_pages > 0
    assert s.free_pages + s.cached_pages == 12
    b.close()


def test_admission_waits_for_pages_instead_of_failing_midway():
    rng = np.random.default_rng(5)
    # 8 pages = 128 tokens; each request needs 4 pages (40 + 24): only two fit at a time although 4 slots exist
    b = ContinuousBatcher.selftest(VOCAB, max_slots=4, max_ctx=128, n_pages=8, prefill_chunk=64, prefix_cache=False)
    want = {}
    for i in range(5):
        p = rng.integers(0, VOCAB, 40).tolist()
        want[b.submit(p, 24)] = _alone(p, 24)
    running, waiting = b.step()
    assert (running, waiting) == (2, 3)
    got = _drain(b, want)
    assert got == want
    b.close()


def test_eos_cancel_forget_and_errors():
    p = [5, 6, 7, 8]
    solo = _alone(p, 30)
    eos = solo[4]
    cut = solo.index(eos) + 1  # generation stops at the FIRST occurrence of the id
    b = ContinuousBatcher.selftest(VOCAB, max_slots=2, max_ctx=64, n_pages=8, prefill_chunk=8)
    a = b.submit(p, 30, eos=[eos])
    c = b.submit([1, 2, 3], 30)
    d = b.submit([9], 30)  # waits for a slot
    b.step()
    b.cancel(c)
    b.cancel(d)
    b.run()
    assert b.poll(a)[0].tolist() == solo[:cut]
    assert b.poll(c)[1] and b.poll(d)[1] and len(b.poll(d)[0]) == 0
    b.forget(d)
    with pytest.raises(SapientCudaError):
        b.poll(d)
    with pytest.raises(SapientCudaError):
        b.submit(list(range(60)), 10)  # 70 tokens in a 64-token window
    with pytest.raises(SapientCudaError):
        b.submit([], 4)
    assert b.stats().free_pages + b.stats().cached_pages == 8
    b.close()


# ── on the CUDA engine ──
@pytest.mark.gpu
@pytest.mark.parametrize("model", ["tiny_llama", "tiny_phi2"])
def test_engine_batcher_matches_solo_greedy_generation(model):
    from sapient_b200 import synth
    from sapient_b200.engine import ForwardEngine

    cfg, W = synth.build_model(synth.CONFIGS[model], seed=11, device="cuda", max_ctx=256)
    Wn = synth.weights_to_numpy(W)
    rng = np.random.default_rng(6)
    system = rng.integers(0, cfg["vocab"], 40).tolist()
    reqs = []
    for i in range(9):
        tail = rng.integers(0, cfg["vocab"], int(rng.integers(1, 30))).tolist()
        reqs.append(((system if i % 2 == 0 else []) + tail, int(rng.integers(4, 24))))
    solo_eng = ForwardEngine.from_weights(cfg, Wn, max_tokens=64)
    solo = []
    for p, mn in reqs:
        solo_eng.reset_cache()
        first = int(np.argmax(solo_eng.forward_logits(p, True)))  # unique maximum with random weights
        rest = solo_eng.decode_greedy([first], [0], mn - 1).reshape(-1).tolist() if mn > 1 else []
        solo.append([first] + rest)
    solo_eng.close()
    eng = ForwardEngine.from_weights(cfg, Wn, max_tokens=64, max_batch=4)
    b = ContinuousBatcher(eng, prefill_chunk=32, prefix_cache=True)
    ids = [b.submit(p, mn) for p, mn in reqs[:5]]
    b.step()
    b.step()
    ids += [b.submit(p, mn) for p, mn in reqs[5:]]  # arrive while the batch is running
    b.run()
    for rid, want in zip(ids, solo):
        got, fin = b.poll(rid)
        assert fin
        assert got.tolist() == want
    s = b.stats()
    assert s.finished == 9 and s.shared_tokens >= 32 * 3  # two whole pages of the common prompt, at least three times
    b.close()
    eng.close()


@pytest.mark.gpu
def test_copy_on_write_of_a_shared_partial_page():
    """Two slots that read the same pages, one of them truncated into the middle of a shared page and extended: the other
    slot's cache must be untouched and the extended one must equal a sequence computed from scratch."""
    from sapient_b200 import synth
    from sapient_b200.engine import ForwardEngine

    cfg, W = synth.build_model(synth.CONFIGS["tiny_llama"], seed=12, device="cuda", max_ctx=128)
    Wn = synth.weights_to_numpy(W)
    rng = np.random.default_rng(7)
    p = rng.integers(0, cfg["vocab"], 40).tolist()
    eng = ForwardEngine.from_weights(cfg, Wn, max_tokens=64, max_batch=3)
    eng.forward_slot(0, p, all_positions=False)
    eng.adopt_prefix(1, [eng.slot_page(0, 0), eng.slot_page(0, 1)])  # 32 shared tokens
    assert eng.seq_len(1) == 32
    eng.truncate_cache(24, slot=1)  # into the middle of shared page 1
    ext = rng.integers(0, cfg["vocab"], 10).tolist()
    got = eng.forward_slot(1, ext, all_positions=False)
    want = eng.forward_slot(2, p[:24] + ext, all_positions=False)
    np.testing.assert_allclose(got, want, atol=2e-3)
    # slot 0 still continues as if nothing happened
    nxt = eng.forward_slot(0, [3], all_positions=False)
    eng.reset_cache(2)
    ref = eng.forward_slot(2, p + [3], all_positions=False)
    np.testing.assert_allclose(nxt, ref, atol=2e-3)
    eng.close()


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_random_arrivals_cancellations_and_tight_pools_keep_every_invariant(seed):
    """Seeded stress of the scheduling logic on the host stand-in: requests with shared and unshared prefixes arrive at
    random iterations, some are cancelled while queued, prefilling or decoding, the pool is a fraction of what all of them
    would need at once. After every iteration the pool balances (free + index pages + pages of running slots = total);
    at the end every request that was not cancelled equals its solo generation and every page is free or indexed."""
    rng = np.random.default_rng(seed)
    n_pages, slots, ctx = int(rng.integers(10, 30)), int(rng.integers(1, 6)), 160
    b = ContinuousBatcher.selftest(VOCAB, max_slots=slots, max_ctx=ctx, n_pages=n_pages, prefill_chunk=int(rng.integers(4, 50)),
                                   prefix_cache=True)
    shared = [rng.integers(0, VOCAB, int(n)).tolist() for n in (33, 48, 17)]
    want, cancelled, pending = {}, set(), []
    for _ in range(60):
        base = shared[int(rng.integers(0, 3))] if rng.random() < 0.6 else []
        p = base + rng.integers(0, VOCAB, int(rng.integers(1, 40))).tolist()
        mn = int(rng.integers(1, 30))
        if (len(p) + mn + 15) // 16 > n_pages or len(p) + mn > ctx:
            continue
        pending.append((int(rng.integers(0, 120)), p, mn))
    pending.sort(key=lambda t: t[0])
    it, live = 0, []
    while pending or live:
        while pending and pending[0][0] <= it:
            _, p, mn = pending.pop(0)
            rid = b.submit(p, mn)
            want[rid] = _alone(p, mn)
            live.append(rid)
        if live and rng.random() < 0.08:
            victim = live[int(rng.integers(0, len(live)))]
            b.cancel(victim)
            cancelled.add(victim)
        b.step()
        s = b.stats()
        assert 0 <= s.free_pages <= n_pages and s.cached_pages <= n_pages
        live = [r for r in live if not b.poll(r)[1]]
        it += 1
        assert it < 20000, "scheduler stopped making progress"
    for rid, w in want.items():
        got, fin = b.poll(rid)
        assert fin
        if rid in cancelled:
            assert got.tolist() == w[: len(got)]  # whatever it had produced before the cancel is still right
        else:
            assert got.tolist() == w, rid
    s = b.stats()
    assert s.free_pages + s.cached_pages == n_pages
    b.close()
