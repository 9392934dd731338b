"""Engine-level parity: the resident CUDA engine against the whole-model CPU oracle on
identical weights and token ids, following the reference's GPU-vs-CPU coherence ladder
(crates/sapient-models/tests/wgpu_coherence.rs:305-600, forward_test.rs:165-188).

Bars: final logits within 2e-2 max-abs of the reference CPU path (Q8_0 KV cache when
head_dim % 32 == 0); greedy top-1 agreement >= 99 % of teacher-forced steps. Against the
oracle run with an fp16-rounded cache (what the device stores) the match is much tighter."""
import numpy as np
import pytest

from helpers import oracle_engine, rel_l2, tiny_model
from sapient_b200 import _lib, synth
from sapient_b200.engine import ForwardEngine

pytestmark = pytest.mark.gpu
LOGIT_BAR = 2e-2
# Prefill-shaped and decode-shaped calls must agree. They are not bit-identical: batches of more than two rows
# carry two int8 digits per activation (2^-15 of the block maximum) instead of three (2^-23), which moves logits
# by ~1e-4. The reference's own chunked-vs-per-token gate is 5e-3 (wgpu_coherence.rs:556-600).
INVARIANCE_BAR = 1e-3
MODELS = ["tiny_llama", "tiny_qwen", "tiny_phi2", "tiny_phi2_wide", "tiny_llama_wide", "tiny_phi3"]


def prompt(cfg, n, seed=0):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).astype(np.uint32)


@pytest.mark.parametrize("name", MODELS)
@pytest.mark.parametrize("kv", ["reference-q8_0-rounding", "plain-fp16"])
def test_prefill_and_decode_logits_match_oracle(oracle, name, kv):
    """Default engine: K / V get the reference's Q8_0 cache rounding before the fp16 store, so it tracks the oracle in the
    reference's own configuration (Q8_0 cache) closely. Plain-fp16 engine: tracks the oracle with an fp16-rounded cache.
    Either way the final logits stay within the 2e-2 bar of the reference configuration."""
    cfg, W = tiny_model(name)
    eng = ForwardEngine.from_weights(cfg, W)
    q8 = kv == "reference-q8_0-rounding" and cfg["head_dim"] % 32 == 0
    if kv == "plain-fp16":
        eng.set_kv_rounding(False)
    close = oracle_engine(oracle, cfg, W, kv_mode=0 if q8 else 1)   # the oracle this engine should sit on
    ref = oracle_engine(oracle, cfg, W, kv_mode=0)
    ids = prompt(cfg, 12)
    got = eng.forward_logits(ids, True)
    wclose, wref = close.forward_logits(ids, True), ref.forward_logits(ids, True)
    # the Q8_0 rounding is a step function: a 1e-7 difference in a K / V value can move one int8 level (0.8 % of the
    # block maximum), so that mode gets a wider band than plain fp16
    near = 5e-3 if q8 else 2e-3
    assert np.max(np.abs(got - wclose)) < near, np.max(np.abs(got - wclose))
    assert np.max(np.abs(got - wref)) < LOGIT_BAR
    agree = 0
    steps = 24
    tok = int(oracle.argmax(wref))
    for _ in range(steps):
        got = eng.forward_logits([tok], True)
        wclose, wref = close.forward_logits([tok], True), ref.forward_logits([tok], True)
        assert np.max(np.abs(got - wclose)) < near
        assert np.max(np.abs(got - wref)) < LOGIT_BAR
        agree += int(oracle.argmax(got) == oracle.argmax(wref) or wref.max() - wref[int(oracle.argmax(got))] <= 4e-2)
        tok = int(oracle.argmax(wref))  # teacher forcing with the reference's token
    assert agree >= int(np.ceil(0.99 * steps))
    assert eng.seq_len() == 12 + steps == ref.seq_len
    eng.close()


@pytest.mark.parametrize("name", MODELS)
def test_per_layer_hidden_states(oracle, name):
    cfg, W = tiny_model(name)
    eng = ForwardEngine.from_weights(cfg, W)
    eng.set_trace(True)
    # per-layer bars are about the kernels: run both sides with the continuous fp16 cache rounding (the Q8_0 rounding is
    # a step function that turns 1e-7 differences into single-level jumps)
    eng.set_kv_rounding(False)
    ref = oracle_engine(oracle, cfg, W, kv_mode=1)
    ids = prompt(cfg, 9, seed=3)
    eng.forward_logits(ids, True)
    ref.forward_logits(ids, True)
    for l in range(cfg["n_layers"]):
        assert rel_l2(eng.layer_out(l), ref.trace(l)) < 1e-3
    eng.close()


@pytest.mark.parametrize("name", MODELS)
def test_cached_decode_equals_full_forward_and_chunking_is_invisible(oracle, name):
    cfg, W = tiny_model(name)
    ids = prompt(cfg, 21, seed=5)
    big = ForwardEngine.from_weights(cfg, W, max_tokens=64)
    small = ForwardEngine.from_weights(cfg, W, max_tokens=4)  # 21 tokens -> 6 internal chunks
    # path-invariance is a statement about the kernels: continuous fp16 cache rounding on both engines (the Q8_0
    # rounding turns 1e-7 differences between the M = 1 and M = 16 kernels into single-level jumps)
    big.set_kv_rounding(False)
    small.set_kv_rounding(False)
    full = big.forward_logits(ids, False)
    chunked = small.forward_logits(ids, False)
    assert np.max(np.abs(full - chunked)) < INVARIANCE_BAR
    big.reset_cache()
    for t in ids[:-1]:
        big.forward_logits([t], True)
    step = big.forward_logits([ids[-1]], True)
    assert np.max(np.abs(full - step)) < INVARIANCE_BAR  # forward_test.rs:165-188
    all_rows = small.forward_all_logits(ids)
    assert all_rows.shape == (21, cfg["vocab"])
    assert np.max(np.abs(all_rows[-1] - full)) < INVARIANCE_BAR
    ref = oracle_engine(oracle, cfg, W, kv_mode=1)
    assert np.max(np.abs(all_rows - ref.forward_all_logits_cached(ids))) < 2e-3
    big.close(); small.close()


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen", "tiny_llama_wide"])
def test_many_row_gemv_passes_give_the_same_logits(oracle, name):
    """Prompts of 11 rows and more as passes of up to 32 rows on the one-pass GEMV (opt-in for engines): the same integer
    products as passes of 10 rows on the tile-row kernel, only the order of the f32 additions over k differs. (Both are
    what steps of 17 rows and more fall back to with the tcgen05 GEMM switched off; here it is off.)"""
    cfg, W = tiny_model(name)
    ids = prompt(cfg, 45, seed=8)  # 32 + 13 rows
    eng = ForwardEngine.from_weights(cfg, W, max_tokens=64)
    eng.set_kv_rounding(False)
    eng.set_large_m_gemm(0)
    base = eng.forward_all_logits(ids)
    eng.set_many_row_gemv(True)
    rows = eng.forward_all_logits(ids)
    eng.set_many_row_gemv(False)
    assert np.max(np.abs(rows - base)) < INVARIANCE_BAR
    ref = oracle_engine(oracle, cfg, W, kv_mode=1)
    assert np.max(np.abs(rows - ref.forward_all_logits_cached(ids))) < 2e-3
    eng.close()


def test_use_cache_false_resets_then_appends(oracle):
    cfg, W = tiny_model("tiny_llama")
    eng = ForwardEngine.from_weights(cfg, W)
    a = prompt(cfg, 6, 1)
    eng.forward_logits(a, True)
    assert eng.seq_len() == 6
    l1 = eng.forward_logits(a[:3], False)
    assert eng.seq_len() == 3  # reset, then append (wgpu_engine.rs:639-641)
    eng.reset_cache()
    assert np.array_equal(l1, eng.forward_logits(a[:3], True))
    eng.close()


def test_truncate_cache_rollback_and_verify_matches_sequential(oracle):
    cfg, W = tiny_model("tiny_qwen")
    eng = ForwardEngine.from_weights(cfg, W)
    ids = prompt(cfg, 10, 2)
    eng.forward_logits(ids, True)
    drafts = prompt(cfg, 5, 3)
    ver = eng.forward_all_logits_cached(drafts)  # one M=5 forward over the cached prompt
    assert eng.seq_len() == 15
    assert eng.truncate_cache(12) == 12 and eng.seq_len() == 12
    assert eng.truncate_cache(100) == 12
    assert eng.truncate_cache(10) == 10
    seq = np.stack([eng.forward_logits([t], True) for t in drafts])
    assert np.max(np.abs(ver - seq)) < INVARIANCE_BAR  # verify logits == sequential decode logits with the same cache
    eng.reset_cache()
    assert eng.seq_len() == 0
    eng.close()


def test_batched_decode_equals_independent_sequences(oracle):
    cfg, W = tiny_model("tiny_llama")
    B = 5
    eng = ForwardEngine.from_weights(cfg, W, max_batch=B, max_tokens=16)
    solo = ForwardEngine.from_weights(cfg, W)
    prompts = [prompt(cfg, 3 + 2 * i, seed=10 + i) for i in range(B)]  # ragged prompt lengths
    want_last = []
    for i, p in enumerate(prompts):
        got = eng.forward_slot(i, p)
        solo.reset_cache()
        want = solo.forward_logits(p, True)
        assert np.max(np.abs(got - want)) < INVARIANCE_BAR
        want_last.append(want)
    toks = np.array([int(oracle.argmax(w)) for w in want_last], np.uint32)
    for step in range(4):
        logits, am = eng.decode_batch(toks, np.arange(B), want_logits=True, want_argmax=True)
        nxt = []
        for i in range(B):
            prompts[i] = np.append(prompts[i], toks[i])
            solo.reset_cache()
            w = solo.forward_logits(prompts[i], True)
            assert np.max(np.abs(logits[i] - w)) < INVARIANCE_BAR
            assert am[i] == oracle.argmax(logits[i])
            nxt.append(int(oracle.argmax(w)))
        toks = np.array(nxt, np.uint32)
    # a permuted slot order gives the same rows
    l2, _ = eng.decode_batch(toks[::-1].copy(), np.arange(B)[::-1].copy())
    eng.truncate_cache(eng.seq_len(0) - 1, 0)
    eng.close(); solo.close()


def test_errors(oracle):
    cfg, W = tiny_model("tiny_llama", max_ctx=16)
    eng = ForwardEngine.from_weights(cfg, W)
    with pytest.raises(_lib.SapientCudaError) as e:
        eng.forward_logits([], True)
    assert e.value.status == _lib.SP_ERR_ARG
    with pytest.raises(_lib.SapientCudaError) as e:
        eng.forward_logits([cfg["vocab"]], True)
    assert e.value.status == _lib.SP_ERR_VOCAB and eng.seq_len() == 0
    eng.forward_logits(prompt(cfg, 16), True)
    with pytest.raises(_lib.SapientCudaError) as e:
        eng.forward_logits([1], True)
    assert e.value.status == _lib.SP_ERR_KV_FULL and eng.seq_len() == 16
    assert eng.backend_label() == "cuda" and not eng.is_hybrid()
    eng.close()
    W2 = dict(W)
    del W2["model.layers.1.mlp.down_proj.weight"]
    with pytest.raises(_lib.SapientCudaError) as e:
        ForwardEngine.from_weights(cfg, W2)
    assert e.value.status == _lib.SP_ERR_STATE


@pytest.mark.parametrize("name", MODELS)
def test_gguf_file_loads_to_the_same_engine(oracle, name, tmp_path):
    """GGUF round trip: ggml dim order, llama q/k row permutation (qwen2 must NOT be un-permuted),
    Phi fused qkv split + fc1/fc2 renames."""
    import torch

    cfg, Wt = synth.build_model(synth.CONFIGS[name], seed=11, device="cpu", max_ctx=64)
    if cfg["arch"] == "phi2":  # the reference's GGUF name map drops output_norm.bias (gguf_weights.rs:360-383)
        Wt.pop("model.norm.bias")
    path = str(tmp_path / f"{name}.gguf")
    synth.write_gguf(path, cfg, Wt)
    a = ForwardEngine.from_gguf(path)
    b = ForwardEngine.from_weights(cfg, synth.weights_to_numpy(Wt))
    ids = prompt(cfg, 7, 4)
    assert np.array_equal(a.forward_logits(ids, True), b.forward_logits(ids, True))
    assert a.desc.rotary_dim == cfg["rotary_dim"] and a.desc.head_dim == cfg["head_dim"]
    a.close(); b.close()


def test_phi3_fused_gate_up_is_cut_at_upload(oracle):
    """PhiForward keeps Phi-3's `mlp.gate_up_proj` fused (forward/phi.rs:559-604: rows 0..ffn gate, the rest up); an engine
    handed that tensor must equal one handed the two halves."""
    cfg, W = tiny_model("tiny_phi3")
    fused = dict(W)
    for l in range(cfg["n_layers"]):
        p = f"model.layers.{l}.mlp."
        (dt, gd, g), (dt2, ud, u) = fused.pop(p + "gate_proj.weight"), fused.pop(p + "up_proj.weight")
        assert dt == dt2
        fused[p + "gate_up_proj.weight"] = (dt, [gd[0] + ud[0], gd[1]], np.concatenate([np.asarray(g).reshape(-1), np.asarray(u).reshape(-1)]))
    a = ForwardEngine.from_weights(cfg, fused)
    b = ForwardEngine.from_weights(cfg, W)
    ids = prompt(cfg, 9, 2)
    assert np.array_equal(a.forward_logits(ids, True), b.forward_logits(ids, True))
    ref = oracle_engine(oracle, cfg, W, kv_mode=0)
    assert np.max(np.abs(b.forward_logits(ids, False) - ref.forward_logits(ids, True))) < 2e-2
    a.close(); b.close()


@pytest.mark.parametrize("fast", [False, True], ids=["exact-class-operands", "fp16-rounded-operands"])
def test_batched_decode_of_twenty_sequences_goes_through_the_large_m_path(oracle, fast):
    """A 20-row decode step is one tcgen05 GEMM launch per matrix: by default with exact-class operands (rows agree with
    each sequence decoded alone to f32 rounding), with fast_large_m with operands rounded to fp16 (rows agree to that
    rounding). Attention runs unsplit either way."""
    cfg, W = tiny_model("tiny_llama")
    B = 20
    eng = ForwardEngine.from_weights(cfg, W, max_batch=B, max_tokens=32, fast_large_m=fast)
    solo = ForwardEngine.from_weights(cfg, W)
    for e in (eng, solo):
        e.set_kv_rounding(False)  # continuous cache rounding: this test is about the kernels
    prompts = [prompt(cfg, 2 + (i % 5), seed=40 + i) for i in range(B)]
    toks = []
    for i, p in enumerate(prompts):
        toks.append(int(oracle.argmax(eng.forward_slot(i, p))))
    toks = np.array(toks, np.uint32)
    for step in range(3):
        logits, am = eng.decode_batch(toks, np.arange(B), want_logits=True, want_argmax=True)
        nxt = []
        for i in range(B):
            prompts[i] = np.append(prompts[i], toks[i])
            solo.reset_cache()
            w = solo.forward_logits(prompts[i], True)
            assert np.max(np.abs(logits[i] - w)) < (5e-3 if fast else 2e-4), (step, i)
            assert am[i] == oracle.argmax(logits[i])
            nxt.append(int(oracle.argmax(w)))
        toks = np.array(nxt, np.uint32)
    eng.close(); solo.close()


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen", "tiny_llama_wide"])
def test_batched_decode_at_longer_context_takes_the_tensor_core_grouped_kernel(oracle, name):
    """32 sequences x ~130 cached keys: enough (token, key) pairs for the tensor-core grouped-query kernel (a block per
    KV head whose query heads form the rows of the mma tile, keys split by context). Its rows must equal each sequence
    decoded alone — a 1-row step at the same context takes the f32 kernel — to rounding, and sit on the oracle."""
    cfg, W = tiny_model(name, max_ctx=192)
    B = 32
    eng = ForwardEngine.from_weights(cfg, W, max_batch=B, max_tokens=64)
    solo = ForwardEngine.from_weights(cfg, W, max_tokens=64)
    for e in (eng, solo):
        e.set_kv_rounding(False)
    prompts = [prompt(cfg, 128 + (i % 7), seed=100 + i) for i in range(B)]
    toks = np.array([int(oracle.argmax(eng.forward_slot(i, p))) for i, p in enumerate(prompts)], np.uint32)
    for step in range(2):
        logits, am = eng.decode_batch(toks, np.arange(B), want_logits=True, want_argmax=True)
        nxt = []
        for i in range(B):
            prompts[i] = np.append(prompts[i], toks[i])
            if i % 8 == 0:  # every eighth sequence against the single-sequence engine and the oracle
                solo.reset_cache()
                w = solo.forward_logits(prompts[i], True)
                assert np.max(np.abs(logits[i] - w)) < 2e-4, (step, i)
                ref = oracle_engine(oracle, cfg, W, kv_mode=1).forward_logits(prompts[i], True)
                assert np.max(np.abs(logits[i] - ref)) < 3e-3, (step, i)
            assert am[i] == oracle.argmax(logits[i])
            nxt.append(int(am[i]))
        toks = np.array(nxt, np.uint32)
    eng.close(); solo.close()


@pytest.mark.parametrize("ftype", ["f16", "bf16"])
def test_float_linears_are_quantised_to_q8_0_at_load_like_the_reference(oracle, ftype):
    """forward/common.rs:39-86: 2-D F16 / BF16 weight matrices (not norms, biases, the embedding table or lm_head) are
    quantised to Q8_0 once at load with quantize_q8_0_block (kernels/quant.rs:223-235). An engine handed the float
    tensors must equal, bit for bit, an engine handed the Q8_0 blocks the oracle's quantiser makes of them."""
    import torch

    cfg, W = tiny_model("tiny_llama")
    g = torch.Generator().manual_seed(3)
    Wf, Wq = dict(W), dict(W)
    n_conv = 0
    for name, (dt, dims, raw) in W.items():
        if len(dims) != 2 or any(s in name for s in ("norm", "bias", "embed", "lm_head")):
            continue
        w = torch.randn(dims[0], dims[1], generator=g) * 0.02
        if ftype == "f16":
            h = w.to(torch.float16)
            Wf[name] = (synth.F16, dims, h.view(torch.uint8).reshape(-1).numpy())
        else:
            h = w.to(torch.bfloat16)
            Wf[name] = (synth.BF16, dims, h.view(torch.uint8).reshape(-1).numpy())
        Wq[name] = (synth.Q8_0, dims, oracle.quantize_q8_0(h.float().numpy().reshape(-1)))
        n_conv += 1
    assert n_conv == 7 * cfg["n_layers"]
    a, b = ForwardEngine.from_weights(cfg, Wf), ForwardEngine.from_weights(cfg, Wq)
    ids = prompt(cfg, 9, 6)
    assert np.array_equal(a.forward_logits(ids, True), b.forward_logits(ids, True))
    assert np.array_equal(a.forward_logits([3], True), b.forward_logits([3], True))
    assert a.resident_bytes()[0] == b.resident_bytes()[0]  # stored as Q8_0, not as floats
    ref = oracle_engine(oracle, cfg, Wq, kv_mode=0)
    ref.forward_logits(ids, True)
    assert np.abs(a.forward_logits([4], True) - ref.forward_logits([3, 4], True)).max() < LOGIT_BAR
    a.close(); b.close()
