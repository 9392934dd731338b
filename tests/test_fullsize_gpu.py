"""Full-size parity: the synthetic models of the benchmark configurations at their own prompt and decode lengths,
against the CPU oracle, teacher-forced with the oracle's greedy tokens.

    qwen05b  Qwen2.5-0.5B shape, 128-token prompt + 128 decode steps
    llama8b  Llama-3-8B shape,   128-token prompt + 100 decode steps
    phi2     Phi-2 shape,        128-token prompt +  64 decode steps
    qwen15b  Qwen2.5-1.5B shape, 256-token prompt + 100 decode steps (the speculative target)

Per model, two comparisons, both with the bars of the task written out and no per-model constants:

  * fp16 cache on both sides (the oracle's kv_mode 1; the engine with the Q8_0 pre-rounding off). Every rounding on
    the path is continuous, so this isolates the kernels. Bars: final logits within 2e-2 max-abs at every position
    checked; the engine's greedy pick equals the oracle's (exact arg-max) on >= 99 % of the decode steps.

  * the reference's own configuration: the oracle keeps the Q8_0 KV cache of forward/common.rs:449-538 (an f32 cache
    where head_dim is not a multiple of 32), the engine rounds new K / V rows the same way before its fp16 store. That
    quantiser is a step function: a difference of one unit in the last place of a K / V value can move an int8 level,
    i.e. 0.8 % of the block's maximum, and the layers above amplify it. How much of that is inherent is MEASURED
    here instead of assumed: the oracle is run a second time with nothing changed but the evaluation order of its
    row dots (per-super-block partial sums for the K-quants, the portable scalar order for Q8_0 — both orders exist in
    the reference for other targets), on the same tokens. The engine must stay as close to the reference as the
    reference stays to itself: its worst logit deviation is at most max(2e-2, 2 x the oracle-vs-oracle deviation) — the
    factor covers the scatter of a maximum over ~10^7 logits of two chaotic trajectories — and it agrees with the
    oracle's greedy pick at least as often as the reordered oracle does, or on 99 % of the steps.

The engines run in their default configuration: decode steps on exact integer products with three-digit activations,
prompts (steps of 17 rows and more) on the tcgen05 GEMM with exact-class operands (fp16 leading part + remainder of weights
and activations, ~1e-6 per product). The same GEMM with operands rounded once to fp16 (~3e-4 per product, twice as fast)
is measured by a further test on the same inputs: its prompt leaves the 2e-2 bar on the largest model (that is why it is
not the default); what is asserted for it is that the deviation stays of the order of the fp16
roundings it introduces — an O(1) fault (a misplaced tile) would be hundreds of times larger — and that greedy decoding
still follows the oracle.

Each run prints one line per comparison; with SAPIENT_PARITY_REPORT=<file> the numbers are appended there as JSON lines.
"""
import json
import os

import numpy as np
import pytest

from sapient_b200 import synth
from sapient_b200.engine import ForwardEngine

pytestmark = pytest.mark.gpu
LOGIT_BAR = 2e-2
AGREE = 0.99
SELF_FACTOR = 2.0

CASES = [("qwen05b", 128, 128), ("llama8b", 128, 100), ("phi2", 128, 64), ("qwen15b", 256, 100)]


def _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode, tokens=None):
    """Prompt logits + `steps` decode logits. tokens None: feeds its own greedy picks and returns them."""
    ref = oracle.OracleEngine(cfg, Wn, kv_mode=kv_mode)
    out = [ref.forward_logits(ids, True)]
    fed = []
    for s in range(steps):
        tok = int(oracle.argmax(out[-1])) if tokens is None else int(tokens[s])
        fed.append(tok)
        out.append(ref.forward_logits([tok], True))
    return np.stack(out), np.array(fed, np.uint32)


def _cuda_run(cfg, Wn, ids, tokens, reference_cache, fast_large_m=False, large_m_mode=None):
    eng = ForwardEngine.from_weights(cfg, Wn, max_tokens=256, fast_large_m=fast_large_m)
    if large_m_mode is not None:
        eng.set_large_m_gemm(large_m_mode)
    eng.set_kv_rounding(reference_cache)
    out = [eng.forward_logits(ids, True)]
    for tok in tokens:
        out.append(eng.forward_logits([int(tok)], True))
    eng.close()
    return np.stack(out)


def _picks(oracle, logits):
    return np.array([oracle.argmax(row) for row in logits])


def _compare(oracle, got, want):
    """(worst |dlogit|, rms dlogit, exact greedy agreements over the decode steps, median top-2 gap of `want`)."""
    d = got.astype(np.float64) - want.astype(np.float64)
    exact = int((_picks(oracle, got[:-1]) == _picks(oracle, want[:-1])).sum())  # row s chooses the token of step s
    top2 = np.partition(want[:-1], -2, axis=1)[:, -2:]
    return float(np.abs(d).max()), float(np.sqrt((d * d).mean())), exact, float(np.median(top2[:, 1] - top2[:, 0]))


def _report(rec):
    print(json.dumps(rec))
    path = os.environ.get("SAPIENT_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")


@pytest.mark.parametrize("name,prompt_len,steps", CASES)
def test_full_size_model_logits_and_greedy_agreement(oracle, name, prompt_len, steps):
    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=3000, device="cuda", max_ctx=512)
    Wn = synth.weights_to_numpy(W)
    del W
    torch.cuda.empty_cache()
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
    need = int(np.ceil(AGREE * steps))

    # ── kernels: continuous (fp16) cache rounding on both sides ──
    want, toks = _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode=1)
    got = _cuda_run(cfg, Wn, ids, toks, reference_cache=False)
    worst, rms, exact, gap = _compare(oracle, got, want)
    _report({"model": name, "prompt": prompt_len, "steps": steps, "cache": "fp16 both sides", "worst_dlogit": worst, "rms_dlogit": rms,
             "exact_top1": exact, "median_top2_gap": gap, "logit_std": float(want.std())})
    assert worst < LOGIT_BAR, worst
    assert exact >= need, (exact, steps)

    # ── the reference's configuration: Q8_0 cache in the oracle, the same rounding before the engine's fp16 store ──
    want, toks = _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode=0)
    try:
        oracle.set_kquant_order(1)
        oracle.set_q8_mode(1)
        other, _ = _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode=0, tokens=toks)
    finally:
        oracle.set_kquant_order(0)
        oracle.set_q8_mode(0)
    self_worst, self_rms, self_exact, _ = _compare(oracle, other, want)
    got = _cuda_run(cfg, Wn, ids, toks, reference_cache=True)
    worst, rms, exact, gap = _compare(oracle, got, want)
    _report({"model": name, "prompt": prompt_len, "steps": steps, "cache": "reference (Q8_0 where head_dim % 32 == 0)", "worst_dlogit": worst,
             "rms_dlogit": rms, "exact_top1": exact, "oracle_reordered_worst_dlogit": self_worst, "oracle_reordered_rms_dlogit": self_rms,
             "oracle_reordered_exact_top1": self_exact, "median_top2_gap": gap})
    assert worst <= max(LOGIT_BAR, SELF_FACTOR * self_worst), (worst, self_worst)
    assert exact >= min(need, self_exact), (exact, self_exact, steps)


@pytest.mark.parametrize("name,prompt_len,steps", [c for c in CASES if c[0] in ("qwen05b", "llama8b", "phi2")])
def test_exact_tensor_core_prompt_meets_the_same_bars(oracle, name, prompt_len, steps):
    """The prompt (128 rows) on the tcgen05 GEMM with exact-class operands (mode 2: leading fp16 part + remainder of weights
    and activations), decode steps unchanged: the bars of the default path, unloosened — 2e-2 on the final logits and
    exact greedy agreement on >= 99 % of the steps, with the continuous cache rounding on both sides."""
    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=3000, device="cuda", max_ctx=512)
    Wn = synth.weights_to_numpy(W)
    del W
    torch.cuda.empty_cache()
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
    steps = min(steps, 48)
    want, toks = _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode=1)
    got = _cuda_run(cfg, Wn, ids, toks, reference_cache=False, large_m_mode=2)
    worst, rms, exact, gap = _compare(oracle, got, want)
    _report({"model": name, "prompt": prompt_len, "steps": steps, "cache": "fp16 both sides", "path": "tcgen05 prompt, exact-class operands",
             "worst_dlogit": worst, "rms_dlogit": rms, "exact_top1": exact, "logit_std": float(want.std())})
    assert worst < LOGIT_BAR, worst
    assert exact >= int(np.ceil(AGREE * steps)), (exact, steps)


@pytest.mark.parametrize("name,prompt_len,steps", [c for c in CASES if c[0] in ("qwen05b", "llama8b")])
def test_fast_large_m_path_is_reported_and_sane(oracle, name, prompt_len, steps):
    """The tcgen05 GEMM with operands rounded to fp16 for the prompt (opt-in), decode steps unchanged: numbers for the record, and two
    sanity bounds — the logit deviation stays below 5 % of the logits' own spread (the fp16 roundings account for ~3 %
    on the 8B shape; a wrong tile would give ~100 %), and at least 95 % of the greedy picks equal the oracle's."""
    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=3000, device="cuda", max_ctx=512)
    Wn = synth.weights_to_numpy(W)
    del W
    torch.cuda.empty_cache()
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
    steps = min(steps, 32)
    want, toks = _oracle_run(oracle, cfg, Wn, ids, steps, kv_mode=1)
    got = _cuda_run(cfg, Wn, ids, toks, reference_cache=False, fast_large_m=True)
    worst, rms, exact, gap = _compare(oracle, got, want)
    _report({"model": name, "prompt": prompt_len, "steps": steps, "cache": "fp16 both sides", "path": "tcgen05 prompt (opt-in)",
             "worst_dlogit": worst, "rms_dlogit": rms, "exact_top1": exact, "logit_std": float(want.std())})
    assert worst < 0.05 * float(want.std()), (worst, float(want.std()))
    assert exact >= int(np.ceil(0.95 * steps)), (exact, steps)
