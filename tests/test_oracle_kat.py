"""Pins the CPU oracle: the reference's own known-answer tests, restated, plus an
independent numpy decoder (the `gguf` package) on random-bit blocks."""
import numpy as np
import pytest

from sapient_b200 import synth

Q8_0, Q4_K, Q6_K = synth.Q8_0, synth.Q4_K, synth.Q6_K


def test_q6_k_canonical_block_dot_is_1920(oracle):
    # crates/sapient-backends/cpu/src/kernels/quant.rs:2714-2734 (wrong scale indexing gives 896)
    block = np.zeros(210, np.uint8)
    block[:128] = 0x11
    block[128:192] = 0xAA
    block[192:208] = np.arange(16, dtype=np.uint8)
    block[208:210] = np.array([1.0], np.float16).view(np.uint8)
    x = np.ones(256, np.float32)
    assert abs(oracle.dot_row(Q6_K, block, x) - 1920.0) < 1e-3
    w = oracle.dequant(Q6_K, block, 256)
    assert np.array_equal(w, np.repeat(np.arange(16, dtype=np.float32), 16))


@pytest.mark.parametrize("dtype,gname", [(Q4_K, "Q4_K"), (Q6_K, "Q6_K"), (Q8_0, "Q8_0")])
def test_dequant_bit_identical_to_numpy_gguf(oracle, dtype, gname):
    import gguf

    nblocks = 96
    raw = synth.random_bit_blocks(dtype, nblocks, seed=1234 + dtype)
    be, bb = synth.BLOCK[dtype]
    got = oracle.dequant(dtype, raw, nblocks * be)
    want = gguf.quants.dequantize(raw.reshape(nblocks, bb), getattr(gguf.GGMLQuantizationType, gname)).reshape(-1)
    assert got.view(np.uint32).tolist() == want.astype(np.float32).view(np.uint32).tolist()


def test_q5_k_high_bit_is_per_element(oracle):
    # crates/sapient-core/src/tensor.rs:796-824: qh[l] bit u1 adds 16 to element l only.
    block = np.zeros(176, np.uint8)
    block[0:2] = np.array([1.0], np.float16).view(np.uint8)
    block[4] = 1  # sc0 = 1
    block[16 + 5] = 1  # qh[5] bit0 → element 5 of sub-block 0
    w = oracle.dequant(13, block, 256)
    want = np.zeros(256, np.float32)
    want[5] = 16.0
    assert np.array_equal(w, want)


def test_half_conversions_match_numpy(oracle):
    for h in range(0, 65536, 7):
        f = oracle.f16_bits_to_f32(h)
        ref = np.array([h], np.uint16).view(np.float16).astype(np.float32)[0]
        assert (np.isnan(f) and np.isnan(ref)) or f == ref
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 1e3, 7e4)])
    vals = np.concatenate([vals, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 5.96e-8, 2.98e-8, 2.9802322e-8], np.float32)])
    with np.errstate(over="ignore"):
        ref = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16_bits(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, ref)


def test_f32_linear_kat(oracle):
    # kernels/matmul.rs:1439-1451
    y = oracle.matmul_nt(np.array([[1, 2]], np.float32), np.array([[1, 2], [3, 4], [5, 6]], np.float32).view(np.uint8), 0, 3)
    assert y.tolist() == [[5.0, 11.0, 17.0]]


def test_norm_kats(oracle):
    # kernels/layernorm.rs:113-149
    y = oracle.layer_norm(np.array([[1, 2], [3, 4]], np.float32), None, None, 1e-5)
    assert np.allclose(y, [[-1, 1], [-1, 1]], atol=1e-4)
    y = oracle.rms_norm(np.array([[3, 4]], np.float32), np.ones(2, np.float32), 0.0)
    assert np.allclose(y, np.array([3, 4], np.float32) / np.sqrt(np.float32(12.5)), atol=1e-5)


def test_rope_kats(oracle):
    # kernels/rope.rs:167-205
    x = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 4)
    assert np.allclose(oracle.rope(x, [0], 10000.0), x, atol=1e-6)
    data = np.arange(1, 9, dtype=np.float32).reshape(1, 1, 8)
    o = oracle.rope(data, [3], 10000.0, 4)
    assert np.allclose(o[0, 0, 4:], data[0, 0, 4:], atol=1e-6)
    assert np.any(np.abs(o[0, 0, :4] - data[0, 0, :4]) > 1e-6)
    d2 = (np.arange(16, dtype=np.float32) * 0.1).reshape(1, 2, 8)
    assert np.array_equal(oracle.rope(d2, [2, 5], 10000.0), oracle.rope(d2, [2, 5], 10000.0, 8))
    # closed form for one pair: head_dim 2, theta = pos
    o = oracle.rope(np.array([1.0, 0.0], np.float32).reshape(1, 1, 2), [2], 10000.0)
    assert np.allclose(o.reshape(-1), [np.cos(2.0), np.sin(2.0)], atol=1e-6)


def test_attention_kats(oracle):
    # kernels/attention.rs:331-415
    m = oracle.causal_mask(3, 3)
    assert np.isneginf(m[0, 1]) and m[1, 0] == 0.0
    seq, dim = 4, 8
    v = np.repeat(np.arange(1, seq + 1, dtype=np.float32)[:, None], dim, 1).reshape(1, seq, dim)
    ones = np.ones((1, seq, dim), np.float32)
    out = oracle.attention(ones, ones, v, np.zeros((seq, seq), np.float32))
    assert np.allclose(out, 2.5, atol=1e-4)
    # leading -inf mask positions must not NaN the online softmax
    seq_k, hd = 8, 4
    kv = (np.arange(seq_k * hd) % 7).astype(np.float32) * 0.1
    kv = kv.reshape(1, seq_k, hd)
    mask = np.full((1, seq_k), -np.inf, np.float32)
    mask[0, -3:] = 0.0
    out = oracle.attention(np.ones((1, 1, hd), np.float32), kv, kv, mask).reshape(-1)
    assert np.all(np.isfinite(out))
    s = kv[0, -3:].sum(1) / np.sqrt(hd)
    p = np.exp(s - s.max())
    p /= p.sum()
    assert np.allclose(out, p @ kv[0, -3:], atol=1e-5)
    # built-in causal rule == explicit causal mask (what gqa_attention passes)
    rng = np.random.default_rng(3)
    q = rng.standard_normal((4, 3, 16)).astype(np.float32)
    k = rng.standard_normal((2, 7, 16)).astype(np.float32)
    vv = rng.standard_normal((2, 7, 16)).astype(np.float32)
    assert np.array_equal(oracle.attention(q, k, vv), oracle.attention(q, k, vv, oracle.causal_mask(3, 7)))
    # fully masked row: l == 0 → output 0 * (1/EPSILON) = 0
    out = oracle.attention(q[:, :1], k, vv, np.full((1, 7), -np.inf, np.float32))
    assert np.all(out == 0.0)


def test_kv_append_layout_kat(oracle):
    # crates/sapient-models/tests/inference_test.rs:9-62
    c = oracle.KvCache(0, 2, 4, 2)
    v1 = c.update(0, np.array([1, 1, 2, 2], np.float32).reshape(2, 1, 2))
    assert v1.shape == (2, 1, 2)
    v2 = c.update(1, np.array([3, 3, 4, 4, 5, 5, 6, 6], np.float32).reshape(2, 2, 2))
    assert v2.shape == (2, 3, 2)
    raw = c.raw_f32().reshape(2, 8)
    assert raw[0].tolist() == [1, 1, 3, 3, 4, 4, 0, 0]
    assert raw[1].tolist() == [2, 2, 5, 5, 6, 6, 0, 0]


def test_kv_sliding_window_and_q8_roundtrip(oracle):
    c = oracle.KvCache(0, 1, 3, 2)
    for i in range(5):
        view = c.update(min(i, 3), np.full((1, 1, 2), float(i), np.float32))
    assert view[0, :, 0].tolist() == [2.0, 3.0, 4.0]
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 3, 64)).astype(np.float32)
    c8 = oracle.KvCache(1, 2, 8, 64)
    got = c8.update(0, x)
    want = oracle.dequant(Q8_0, oracle.quantize_q8_0(x), x.size).reshape(x.shape)
    assert np.array_equal(got, want)
    assert np.max(np.abs(got - x)) < np.abs(x).max() / 127.0


def test_unpermute_inverts_llama_cpp_permutation(oracle):
    # crates/sapient-models/src/gguf_weights.rs:478-496
    n_head, head_dim, hidden = 3, 4, 5
    hf = np.array([[r * 100 + c for c in range(hidden)] for r in range(n_head * head_dim)], np.float32)
    raw = hf.view(np.uint8).reshape(-1)
    g = synth.permute_qk_rows_for_gguf(raw, n_head, head_dim, hidden * 4)
    assert not np.array_equal(g, raw)
    back = oracle.unpermute_qk_rows(g, n_head, head_dim, hidden * 4)
    assert np.array_equal(back, raw)


def test_elementwise_kats(oracle):
    assert oracle.gelu(np.zeros(1, np.float32))[0] == 0.0
    assert oracle.silu(np.zeros(1, np.float32))[0] == 0.0
    x = np.array([1.5, -2.0], np.float32)
    assert np.allclose(oracle.silu(x), x / (1 + np.exp(-x)), rtol=1e-6)
    assert np.allclose(oracle.gelu(x), 0.5 * x * (1 + np.tanh(0.79788456 * (x + 0.044715 * x ** 3))), rtol=1e-5, atol=1e-6)
    assert oracle.mul(np.array([1, 2, 3], np.float32), np.full(3, 2.0, np.float32)).tolist() == [2, 4, 6]


def test_argmax_last_max_wins(oracle):
    # crates/sapient-generate/src/sampler.rs:161-168 (Iterator::max_by keeps the last maximum)
    assert oracle.argmax(np.array([1, 5, 3, 5, 2], np.float32)) == 3
    assert oracle.argmax(np.array([7, 7, 7], np.float32)) == 2
    assert oracle.argmax(np.array([-1], np.float32)) == 0


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_matmul_nt_vs_dequantised_matmul(oracle, dtype):
    # kernels/matmul.rs:1272-1437: quantised path vs f32 matmul over the SAME decoded bytes
    rng = np.random.default_rng(dtype)
    for m, k, n in [(1, 512, 48), (3, 256, 17), (5, 1024, 8)]:
        raw = synth.random_bit_blocks(dtype, n * k // synth.BLOCK[dtype][0], seed=dtype * 7 + m)
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = oracle.dequant(dtype, raw, n * k).reshape(n, k)
        y = oracle.matmul_nt(x, raw, dtype, n)
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 1e-5
    oracle.set_q8_mode(1)
    try:
        raw = synth.random_bit_blocks(Q8_0, 8 * 8, seed=1)
        x = rng.standard_normal((2, 256)).astype(np.float32)
        y1 = oracle.matmul_nt(x, raw, Q8_0, 8)
    finally:
        oracle.set_q8_mode(0)
    y0 = oracle.matmul_nt(x, raw, Q8_0, 8)
    assert np.allclose(y0, y1, rtol=1e-4, atol=1e-6)


def test_matmul_nt_errors(oracle):
    # kernels/matmul.rs:863-865,1112-1114,576-580
    x = np.zeros((1, 128), np.float32)
    for dt in (Q4_K, Q6_K):
        with pytest.raises(oracle.OracleError):
            oracle.matmul_nt(x, np.zeros(144, np.uint8), dt, 1)
    with pytest.raises(oracle.OracleError):
        oracle.matmul_nt(np.zeros((1, 48), np.float32), np.zeros(68, np.uint8), Q8_0, 1)
    with pytest.raises(oracle.OracleError):
        oracle.embed(Q8_0, np.zeros(34 * 4, np.uint8), 4, 32, [4])


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_synth_quantisers_roundtrip(oracle, dtype):
    import torch

    g = torch.Generator().manual_seed(dtype)
    w = torch.randn(6, 512, generator=g) * 0.02
    raw = synth.quantize(dtype, w).numpy()
    assert raw.size == synth.byte_count(dtype, w.numel())
    back = oracle.dequant(dtype, raw, w.numel()).reshape(6, 512)
    err = np.abs(back - w.numpy()).max()
    tol = {Q4_K: 0.02 * 6 / 15, Q6_K: 0.02 * 6 / 31, Q8_0: 0.02 * 6 / 127}[dtype]
    assert err < tol, err


@pytest.mark.parametrize("dtype,block_bytes", [(12, 144), (14, 210)])
def test_rows_at_once_matmul_is_bit_identical_to_the_row_by_row_loop(oracle, dtype, block_bytes):
    """The tests run the oracle's K-quant matmul eight rows at a time (one row per SIMD lane, each lane the scalar
    operation sequence of kernels/quant.rs:625-652 / 2573-2613); the timing runs keep the reference's one-row loop.
    Both must give the same bits, also for row counts that leave a remainder."""
    rng = np.random.default_rng(5)
    n, k = 67, 1024
    w = rng.integers(0, 256, n * k // 256 * block_bytes, dtype=np.uint8).reshape(-1, block_bytes)
    d = np.frombuffer(np.float16(rng.uniform(1e-3, 1e-2, len(w))).tobytes(), np.uint8).reshape(-1, 2)
    if dtype == 12:
        w[:, 0:2] = d
        w[:, 2:4] = d[::-1]
    else:
        w[:, 208:210] = d
    x = rng.standard_normal((3, k)).astype(np.float32)
    try:
        oracle.set_rows_at_once(False)
        want = oracle.matmul_nt(x, w, dtype, n)
        oracle.set_rows_at_once(True)
        got = oracle.matmul_nt(x, w, dtype, n)
    finally:
        oracle.set_rows_at_once(True)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the second evaluation order differs in rounding only
    try:
        oracle.set_kquant_order(1)
        alt = oracle.matmul_nt(x, w, dtype, n)
    finally:
        oracle.set_kquant_order(0)
    assert not np.array_equal(alt.view(np.uint32), want.view(np.uint32))
    assert np.abs(alt - want).max() <= 1e-5 * np.abs(want).max()
