"""Prefill attention on tensor cores (attention_prefill_kernel): engines that put a whole prompt through the tiled
kernel (one sequence, more than 16 tokens per step, launched directly) against engines that feed the same prompt in
chunks of 32 tokens through replayed step graphs (the per-token kernel, which reads positions from device memory),
and against the oracle."""
import numpy as np
import pytest

from helpers import oracle_engine, tiny_model
from sapient_b200.engine import ForwardEngine

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen", "tiny_llama_tp"])
@pytest.mark.parametrize("n_prompt", [33, 64, 100, 150])
def test_tiled_prefill_attention_matches_per_token_kernel_and_oracle(oracle, name, n_prompt):
    cfg, W = tiny_model(name, max_ctx=256)
    ids = np.random.default_rng(n_prompt).integers(0, cfg["vocab"], n_prompt).astype(np.uint32)
    big = ForwardEngine.from_weights(cfg, W, max_tokens=256, fast_large_m=True)     # whole prompt in one chunk: tiled kernel + tcgen05 GEMM
    small = ForwardEngine.from_weights(cfg, W, max_tokens=32)    # chunks of 32: per-token kernel
    big.set_graphs(False)  # direct launches: the tiled kernel takes the first position as an argument
    for e in (big, small):
        e.set_kv_rounding(False)  # continuous cache rounding: this test is about the kernels
    a = big.forward_all_logits(ids)
    b = small.forward_all_logits(ids)
    ref = oracle_engine(oracle, cfg, W, kv_mode=1).forward_all_logits(ids)
    assert np.abs(a - b).max() < 2e-3, np.abs(a - b).max()
    assert np.abs(a - ref).max() < 3e-3, np.abs(a - ref).max()
    # a second chunk on top of a non-empty cache (pos0 > 0), then a decode step reading what prefill wrote
    more = np.random.default_rng(1).integers(0, cfg["vocab"], 40).astype(np.uint32)
    a2 = big.forward_all_logits_cached(more)
    b2 = small.forward_all_logits_cached(more)
    assert np.abs(a2 - b2).max() < 2e-3
    assert np.abs(big.forward_logits([5], True) - small.forward_logits([5], True)).max() < 2e-3
    big.close()
    small.close()


def test_replayed_step_graphs_do_not_freeze_positions():
    """The same number of rows at two different cache positions: the second call replays the step graph captured by
    the first, so nothing in it may depend on the positions the first call had."""
    cfg, W = tiny_model("tiny_llama", max_ctx=256)
    rng = np.random.default_rng(9)
    first, second = (rng.integers(0, cfg["vocab"], 40).astype(np.uint32) for _ in range(2))
    graphs = ForwardEngine.from_weights(cfg, W, max_tokens=64, fast_large_m=True)
    direct = ForwardEngine.from_weights(cfg, W, max_tokens=64, fast_large_m=True)
    direct.set_graphs(False)
    for e in (graphs, direct):
        e.set_kv_rounding(False)
    assert np.abs(graphs.forward_all_logits(first) - direct.forward_all_logits(first)).max() < 2e-3
    assert np.abs(graphs.forward_all_logits_cached(second) - direct.forward_all_logits_cached(second)).max() < 2e-3
