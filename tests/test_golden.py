"""Committed golden vectors (tests/golden/golden_v1.npz and golden_v2.npz — the formats and the model family added later —
made by tests/golden/make_golden.py): the oracle must still reproduce them on CPU; the CUDA path must match them on a GPU."""
import os
import sys

import numpy as np
import pytest

from helpers import tiny_model
from sapient_b200 import synth

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
G = np.load(os.path.join(HERE, "golden", "golden_v1.npz"))
G2 = np.load(os.path.join(HERE, "golden", "golden_v2.npz"))
G = {**{k: G[k] for k in G.files}, **{k: G2[k] for k in G2.files}}
TYPES = [(synth.Q4_K, "q4_k"), (synth.Q6_K, "q6_k"), (synth.Q8_0, "q8_0"), (synth.Q4_0, "q4_0"), (synth.Q5_K, "q5_k")]
MODELS = ["tiny_llama", "tiny_qwen", "tiny_phi2", "tiny_phi3"]


@pytest.mark.parametrize("dtype,tag", TYPES)
def test_oracle_reproduces_golden_blocks(oracle, dtype, tag):
    raw, x = G[f"{tag}_blocks"], G[f"{tag}_x"]
    assert np.array_equal(synth.random_bit_blocks(dtype, raw.size // synth.BLOCK[dtype][1], seed=dtype), raw)
    assert np.array_equal(oracle.dequant(dtype, raw, 6 * 512).reshape(6, 512).view(np.uint32), G[f"{tag}_dequant"].view(np.uint32))
    assert np.array_equal(oracle.matmul_nt(x, raw, dtype, 6), G[f"{tag}_y"])


@pytest.mark.parametrize("name", MODELS)
def test_oracle_reproduces_golden_logits(oracle, name):
    from make_golden import weights_digest

    cfg, W = tiny_model(name)
    assert weights_digest(W).encode() == G[f"{name}_digest"].tobytes(), "synthetic weights changed: regenerate the fixture"
    e = oracle.OracleEngine(cfg, W, kv_mode=0)
    got = [e.forward_logits(G[f"{name}_ids"], True)]
    for t in G[f"{name}_tokens_ref"]:
        got.append(e.forward_logits([t], True))
    assert np.array_equal(np.stack(got), G[f"{name}_logits_ref"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tag", TYPES)
def test_cuda_matches_golden_blocks(dtype, tag):
    from sapient_b200 import ops

    w = ops.Weight(dtype, 6, 512, G[f"{tag}_blocks"])
    assert np.array_equal(w.dequant().view(np.uint32), G[f"{tag}_dequant"].view(np.uint32))
    y = w.matmul_nt(G[f"{tag}_x"])
    want = G[f"{tag}_y"]
    assert np.linalg.norm(y - want) / np.linalg.norm(want) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("name", MODELS)
def test_cuda_matches_golden_logits(name):
    from sapient_b200.engine import ForwardEngine

    cfg, W = tiny_model(name)
    eng = ForwardEngine.from_weights(cfg, W)
    for tag, bar in (("f16", 2e-3), ("ref", 2e-2)):
        eng.reset_cache()
        eng.set_kv_rounding(tag == "ref")  # "f16": the oracle run with an fp16-rounded cache; "ref": the reference's Q8_0 cache
        got = [eng.forward_logits(G[f"{name}_ids"], True)]
        for t in G[f"{name}_tokens_{tag}"]:
            got.append(eng.forward_logits([t], True))
        got = np.stack(got)
        want = G[f"{name}_logits_{tag}"]
        assert np.max(np.abs(got - want)) < bar
        assert [int(np.flatnonzero(r == r.max())[-1]) for r in got[:-1]] == G[f"{name}_tokens_{tag}"].tolist()
    eng.close()
