"""Full-size parity: the Qwen2.5-0.5B-shaped and the Llama-3-8B-shaped synthetic models (BASELINE configs) against the
CPU oracle, teacher-forced with the oracle's tokens.

Two comparisons per model:
  * kernels: both sides round new K / V rows to fp16 (continuous rounding). Bar: final logits within 2e-2 max-abs,
    greedy top-1 agreement >= 99 %.
  * reference configuration: the oracle keeps the reference's Q8_0 cache, the engine applies the same Q8_0 rounding
    before its fp16 store (its default). That rounding is a step function: a 1e-7 difference in a K / V value moves a
    whole int8 level (0.8 % of the block maximum), and 32 layers amplify such flips, so at the 8B shape the logits of
    two correct implementations differ by ~0.1 (the oracle itself moves by ~0.36 when its cache is switched from
    Q8_0 to fp16). The 2e-2 logit bar is therefore asserted on the kernels comparison and the greedy-agreement bar
    everywhere; the deviation under the reference cache is printed and bounded loosely (0.5B shape: 1.7e-2 while the
    48-token prompt went through the integer GEMV, 2.7e-2 now that steps of 17 rows and more use the tcgen05 GEMM
    with fp16 operands, whose 3e-4 relative error flips a few more int8 levels; 8B shape: ~0.12).
A CUDA pick counts as agreeing when it is the oracle's pick or the oracle's own logits rank it within 4e-2 of its
maximum (random-init models have near-flat logits; ties in the 2nd digit carry no information about the kernels)."""
import numpy as np
import pytest

from sapient_b200 import synth
from sapient_b200.engine import ForwardEngine

pytestmark = pytest.mark.gpu
LOGIT_BAR = 2e-2
MARGIN = 4e-2


def _run(oracle, cfg, Wn, ids, steps, reference_cache: bool):
    eng = ForwardEngine.from_weights(cfg, Wn, max_tokens=64)
    eng.set_kv_rounding(reference_cache)
    ref = oracle.OracleEngine(cfg, Wn, kv_mode=0 if reference_cache else 1)
    got, want = eng.forward_logits(ids, True), ref.forward_logits(ids, True)
    worst = float(np.abs(got - want).max())
    agree = exact = 0
    tok = int(oracle.argmax(want))
    for _ in range(steps):
        got, want = eng.forward_logits([tok], True), ref.forward_logits([tok], True)
        worst = max(worst, float(np.abs(got - want).max()))
        pick, ref_pick = int(oracle.argmax(got)), int(oracle.argmax(want))
        exact += int(pick == ref_pick)
        agree += int(pick == ref_pick or want.max() - want[pick] <= MARGIN)
        tok = ref_pick  # teacher forcing
    eng.close()
    return worst, exact, agree


@pytest.mark.parametrize("name,prompt_len,steps,ref_logit_bar", [("qwen05b", 48, 24, 0.05), ("llama8b", 16, 6, 0.25)])
def test_full_size_model_logits_and_greedy_agreement(oracle, name, prompt_len, steps, ref_logit_bar):
    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=3000, device="cuda", max_ctx=256)
    Wn = synth.weights_to_numpy(W)
    del W
    torch.cuda.empty_cache()
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
    need = int(np.ceil(0.99 * steps))
    worst, exact, agree = _run(oracle, cfg, Wn, ids, steps, reference_cache=False)
    print(f"{name} fp16 cache both sides: worst |dlogit| = {worst:.2e}, exact top-1 {exact}/{steps}, within-margin {agree}/{steps}")
    assert worst < LOGIT_BAR, worst
    assert agree >= need, (agree, steps)
    worst, exact, agree = _run(oracle, cfg, Wn, ids, steps, reference_cache=True)
    print(f"{name} reference Q8_0 cache: worst |dlogit| = {worst:.2e}, exact top-1 {exact}/{steps}, within-margin {agree}/{steps}")
    assert worst < ref_logit_bar, worst
    assert agree >= need, (agree, steps)
