"""Speculative decoding (sapient_b200/speculative.py): host logic on the CPU oracle engines, and the same
properties through the CUDA engines.

Properties (the reference has no stored token fixtures for this path):
  * draft == target and greedy sampling: every draft is accepted and the committed tokens are exactly the
    target's own greedy decode (parity = identical to target-only greedy);
  * any draft, any random stream: after every round both caches hold exactly the committed tokens, and the
    kept next-token logits equal a fresh forward over the committed tokens;
  * a random stream that always rejects commits one corrected token per round, drawn from max(0, p_t - p_d).
"""
import numpy as np
import pytest

from helpers import oracle_engine, tiny_model
from sapient_b200 import speculative as sp


def _prompt(cfg, n=12, seed=3):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).astype(np.uint32).tolist()


def _len(eng):
    return eng.seq_len() if callable(eng.seq_len) else eng.seq_len


def _greedy_decode(eng, prompt, n):
    out = []
    lg = eng.forward_logits(prompt, True)
    for _ in range(n):
        t = sp.greedy(lg)
        out.append(t)
        lg = eng.forward_logits([t], True)
    return out


def test_math_helpers():
    p = sp.softmax(np.array([1.0, 2.0, 3.0], np.float32))
    assert p.dtype == np.float32 and abs(float(p.sum()) - 1.0) < 1e-6 and p[2] > p[1] > p[0]
    # nothing left after subtracting the draft: all mass on the target's best token, last maximum wins
    t = np.array([0.25, 0.5, 0.25, 0.0], np.float32)
    assert np.array_equal(sp.adjusted_dist(t, t), np.array([0, 1, 0, 0], np.float32))
    tie = np.array([0.5, 0.5], np.float32)
    assert np.array_equal(sp.adjusted_dist(tie, tie), np.array([0, 1], np.float32))
    adj = sp.adjusted_dist(np.array([0.6, 0.4], np.float32), np.array([0.9, 0.1], np.float32))
    assert np.allclose(adj, [0.0, 1.0])
    probs = np.array([0.2, 0.3, 0.5], np.float32)
    assert sp.sample_from_probs(probs, 0.0) == 0 and sp.sample_from_probs(probs, 0.2) == 1
    assert sp.sample_from_probs(probs, 0.49) == 1 and sp.sample_from_probs(probs, 0.51) == 2
    assert sp.sample_from_probs(probs, 1.5) == 2
    assert sp.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 2


def _check_same_model_is_greedy(make_engine, cfg, W, new_tokens=14, k=4):
    prompt = _prompt(cfg)
    ref = _greedy_decode(make_engine(cfg, W), prompt, new_tokens)
    target, draft = make_engine(cfg, W), make_engine(cfg, W)
    out, st = sp.generate(target, draft, prompt, new_tokens, k=k, seed=1)
    assert out == ref
    # k drafts + 1 bonus per round, all drafts accepted
    assert st.accepted_drafts == st.drafted and all(c == d + 1 for d, c in st.history)
    assert _len(target) == st.committed_len == _len(draft)


def _check_cache_reconciliation(make_engine, cfg, Wt, Wd, rand, rounds=5, k=4, tol=2e-2):
    prompt = _prompt(cfg, 9, seed=5)
    target, draft = make_engine(cfg, Wt), make_engine(cfg, Wd)
    st = sp.spec_prefill(target, draft, prompt)
    for _ in range(rounds):
        committed, _ = sp.spec_round(target, draft, st, k, sp.greedy, rand)
        assert 1 <= len(committed) <= k + 1
        assert _len(target) == st.committed_len == _len(draft) == len(st.all_tokens)
    fresh_t, fresh_d = make_engine(cfg, Wt), make_engine(cfg, Wd)
    assert np.abs(fresh_t.forward_logits(st.all_tokens, True) - st.target_next).max() < tol
    assert np.abs(fresh_d.forward_logits(st.all_tokens, True) - st.draft_next).max() < tol
    return st


def test_same_model_equals_greedy_on_oracle(oracle):
    cfg, W = tiny_model("tiny_llama")
    _check_same_model_is_greedy(lambda c, w: oracle_engine(oracle, c, w), cfg, W)


def test_cache_reconciliation_on_oracle(oracle):
    cfg, Wt = tiny_model("tiny_llama", seed=7)
    _, Wd = tiny_model("tiny_llama", seed=8)
    rng = np.random.default_rng(0)
    st = _check_cache_reconciliation(lambda c, w: oracle_engine(oracle, c, w), cfg, Wt, Wd, lambda: float(rng.random()), tol=1e-4)
    assert st.rounds == 5 and st.drafted == 20


def test_always_reject_commits_one_corrected_token(oracle):
    cfg, Wt = tiny_model("tiny_llama", seed=7)
    _, Wd = tiny_model("tiny_llama", seed=8)
    target, draft = oracle_engine(oracle, cfg, Wt), oracle_engine(oracle, cfg, Wd)
    st = sp.spec_prefill(target, draft, _prompt(cfg))
    draws = iter([0.999999, 0.0] * 8)  # accept test fails (p_t/p_d < 1 for the draft's own argmax here), then inverse CDF at 0
    t_probs, d_probs = sp.softmax(st.target_next), sp.softmax(st.draft_next)
    d0 = sp.greedy(st.draft_next)
    assert t_probs[d0] / d_probs[d0] < 0.999999
    committed, hit = sp.spec_round(target, draft, st, 4, sp.greedy, lambda: next(draws))
    assert not hit and len(committed) == 1
    adj = sp.adjusted_dist(t_probs, d_probs)
    assert committed[0] == int(np.flatnonzero(adj > 0)[0])  # r = 0 picks the first token with mass left
    assert _len(target) == _len(draft) == st.committed_len


@pytest.mark.gpu
def test_same_model_equals_greedy_on_cuda():
    from sapient_b200.engine import ForwardEngine

    for name in ("tiny_llama", "tiny_phi2"):
        cfg, W = tiny_model(name)
        _check_same_model_is_greedy(lambda c, w: ForwardEngine.from_weights(c, w), cfg, W)


@pytest.mark.gpu
def test_cache_reconciliation_on_cuda():
    from sapient_b200.engine import ForwardEngine

    cfg, Wt = tiny_model("tiny_llama", seed=7)
    _, Wd = tiny_model("tiny_llama", seed=8)
    rng = np.random.default_rng(0)
    _check_cache_reconciliation(lambda c, w: ForwardEngine.from_weights(c, w), cfg, Wt, Wd, lambda: float(rng.random()))


@pytest.mark.gpu
def test_verify_pass_is_one_batched_forward():
    """The k drafts go through the target as one k-row decode step (one weight stream), not k steps."""
    from sapient_b200 import ops
    from sapient_b200.engine import ForwardEngine

    cfg, W = tiny_model("tiny_llama")
    eng = ForwardEngine.from_weights(cfg, W)
    eng.forward_logits(_prompt(cfg), True)
    eng.forward_all_logits_cached([1, 2, 3, 4])  # builds the 4-row graph
    eng.truncate_cache(12)
    n0 = ops.launch_count()
    eng.forward_all_logits_cached([1, 2, 3, 4])
    batched = ops.launch_count() - n0
    eng.truncate_cache(12)
    eng.forward_logits([1], True)
    eng.truncate_cache(12)
    n0 = ops.launch_count()
    eng.forward_logits([1], True)
    single = ops.launch_count() - n0
    assert batched == single  # same kernels per step whatever the row count


# ── greedy schedule with a k + 1 row verify pass (generate_greedy / sp_cuda_spec_greedy) ──
def test_greedy_schedule_equals_target_greedy_on_oracle(oracle):
    cfg, Wt = tiny_model("tiny_llama", seed=7)
    _, Wd = tiny_model("tiny_llama", seed=8)
    prompt = _prompt(cfg)
    ref = _greedy_decode(oracle_engine(oracle, cfg, Wt), prompt, 17)
    target, draft = oracle_engine(oracle, cfg, Wt), oracle_engine(oracle, cfg, Wd)
    out, st = sp.generate_greedy(target, draft, prompt, 17, k=4)
    assert out == ref
    assert st.drafted == 4 * st.rounds and 0 <= st.accepted_drafts <= st.drafted
    # draft == target: every draft is accepted, k + 1 tokens per round after the first token
    target, draft = oracle_engine(oracle, cfg, Wt), oracle_engine(oracle, cfg, Wt)
    out, st = sp.generate_greedy(target, draft, prompt, 16, k=4)
    assert out == ref[:16] and st.accepted_drafts == st.drafted == 4 * 3
    # an EOS id ends the stream right after it
    eos = ref[5]
    out, _ = sp.generate_greedy(oracle_engine(oracle, cfg, Wt), oracle_engine(oracle, cfg, Wd), prompt, 17, k=4, eos_ids=[eos])
    assert out == ref[: ref.index(eos) + 1]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny_llama", "tiny_llama_wide", "tiny_phi2_wide"])
def test_device_greedy_spec_equals_target_greedy(name):
    """sp_cuda_spec_greedy (draft loop on the device, k + 1 row verify, arg-max ids only) against the target's own
    greedy decoding and against the host-side statement of the same schedule."""
    from sapient_b200.engine import ForwardEngine

    cfg, Wt = tiny_model(name, seed=7, max_ctx=128)
    _, Wd = tiny_model(name, seed=8, max_ctx=128)
    prompt = _prompt(cfg, 10)
    n_new = 48
    ref = _greedy_decode(ForwardEngine.from_weights(cfg, Wt), prompt, n_new)
    for Wdraft, all_accepted in ((Wd, False), (Wt, True)):
        target, draft = ForwardEngine.from_weights(cfg, Wt), ForwardEngine.from_weights(cfg, Wdraft)
        out, st = sp.generate_greedy_device(target, draft, prompt, n_new, k=4)
        assert out == ref
        t2, d2 = ForwardEngine.from_weights(cfg, Wt), ForwardEngine.from_weights(cfg, Wdraft)
        out_h, st_h = sp.generate_greedy(t2, d2, prompt, n_new, k=4)
        assert out_h == ref and (st_h.rounds, st_h.drafted, st_h.accepted_drafts) == (st.rounds, st.drafted, st.accepted_drafts)
        if all_accepted:
            assert st.accepted_drafts == st.drafted and st.rounds == -(-(n_new - 1) // 5)
        for e in (target, draft, t2, d2):
            e.close()
    # generation stops after an EOS id; bad arguments are refused
    target, draft = ForwardEngine.from_weights(cfg, Wt), ForwardEngine.from_weights(cfg, Wd)
    out, _ = sp.generate_greedy_device(target, draft, prompt, n_new, k=4, eos_ids=[ref[7]])
    assert out == ref[: ref.index(ref[7]) + 1]
    from sapient_b200 import _lib

    with pytest.raises(_lib.SapientCudaError):
        sp.generate_greedy_device(target, draft, prompt, n_new, k=0)
    with pytest.raises(_lib.SapientCudaError):
        sp.generate_greedy_device(target, draft, [], n_new, k=4)
