"""Per-op parity of the CUDA kernels against the CPU oracle, through the C ABI.

Bars (from the backend's contract): dequantised weights bit-exact; every other op
within 1e-3 relative L2 of the reference CPU path (most land near 1e-6)."""
import numpy as np
import pytest

from helpers import f16_round, rel_l2
from sapient_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
Q8_0, Q4_K, Q6_K = synth.Q8_0, synth.Q4_K, synth.Q6_K
REL_L2_BAR = 1e-3


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_dequant_bit_exact_random_bits(oracle, dtype):
    be, _ = synth.BLOCK[dtype]
    n, k = 37, 4 * 256
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=100 + dtype)
    w = ops.Weight(dtype, n, k, raw)
    got = w.dequant()
    want = oracle.dequant(dtype, raw, n * k).reshape(n, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_dequant_bit_exact_quantised_gaussian(oracle, dtype):
    import torch

    g = torch.Generator().manual_seed(dtype)
    wf = torch.randn(64, 1024, generator=g) * 0.02
    raw = synth.quantize(dtype, wf).numpy().reshape(-1)
    got = ops.Weight(dtype, 64, 1024, raw).dequant()
    want = oracle.dequant(dtype, raw, 64 * 1024).reshape(64, 1024)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q6_k_canonical_block(oracle):
    block = np.zeros(210, np.uint8)
    block[:128] = 0x11
    block[128:192] = 0xAA
    block[192:208] = np.arange(16, dtype=np.uint8)
    block[208:210] = np.array([1.0], np.float16).view(np.uint8)
    y = ops.matmul_nt(np.ones((1, 256), np.float32), block, Q6_K, 1)
    assert abs(float(y[0, 0]) - 1920.0) < 1e-3


# reference GPU-vs-CPU shapes (wgpu/tests/resident.rs:71-101,641-775) plus ragged row counts and every M bucket
MATMUL_CASES = [(1, 1536, 512), (3, 256, 48), (17, 256, 48), (1, 256, 1), (2, 512, 9), (4, 1024, 33), (5, 768, 7),
                (8, 2048, 64), (9, 512, 16), (32, 1024, 40),
                # 11 rows and more: the one-pass many-row kernel (K split over CTAs, ragged last row group, two passes)
                (11, 512, 16), (24, 4096, 300), (20, 2048, 2064), (47, 2048, 200), (64, 1024, 129), (32, 14336, 512),
                # more tiles than the GPU has SMs: every CTA of the persistent ring GEMV shares its first and last tile row
                (1, 4096, 2400), (2, 14336, 1024), (4, 4096, 1000), (3, 1536, 2728)]


# 0: the default tensor-core kernels; 4: the bulk-copy ring GEMV for 1-5 rows (tile-row kernel above)
@pytest.fixture(params=[0, 4, 1, 3], ids=["tensor-core-default", "tensor-core-ring", "cuda-core", "tensor-core-stream"])
def gemv_path(request):
    ops.set_gemv_path(request.param)
    yield request.param
    ops.set_gemv_path(0)


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
@pytest.mark.parametrize("m,k,n", MATMUL_CASES)
def test_matmul_nt_random_bits(oracle, gemv_path, dtype, m, k, n):
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m * 1000 + k + n)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=k + n + dtype)
    x = rng.standard_normal((m, k)).astype(np.float32)
    got = ops.matmul_nt(x, raw, dtype, n)
    want = oracle.matmul_nt(x, raw, dtype, n)
    assert got.shape == (m, n)
    err = rel_l2(got, want)
    assert err < REL_L2_BAR, err
    # cuda-core: f32 accumulation in a different order. tensor-core: exact integer products, activations held to 2^-23
    # (three digits) of each 256-column block's maximum up to 16 rows; from 17 rows on the tcgen05 GEMM with exact-class
    # operands (leading fp16 part + remainder).
    assert err < 2e-5, err


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
@pytest.mark.parametrize("m,k,n", [c for c in MATMUL_CASES if c[0] >= 11])
def test_matmul_nt_many_rows_on_the_integer_kernels(oracle, dtype, m, k, n):
    """Mode 0: 11 rows and more on the one-pass mma.sync kernel (passes of up to 32 rows) instead of the tcgen05 GEMM."""
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m * 1000 + k + n)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=k + n + dtype)
    x = rng.standard_normal((m, k)).astype(np.float32)
    try:
        ops.set_large_m_gemm(0)
        got = ops.matmul_nt(x, raw, dtype, n)
    finally:
        ops.set_large_m_gemm(ops.LARGE_M_DEFAULT)
    assert rel_l2(got, oracle.matmul_nt(x, raw, dtype, n)) < 2e-5


@pytest.mark.parametrize("dtype,m,k,n", [(Q4_K, 32, 4096, 1024), (Q6_K, 20, 2048, 640), (Q8_0, 64, 4096, 300)])
def test_many_row_pass_is_reproducible_and_equals_the_small_passes(oracle, dtype, m, k, n):
    """The one-pass kernel for 11-32 rows splits K over several CTAs on small matrices; partial rows are added in split
    order by the last CTA to arrive, so repeated calls give identical bits. Against the passes of 10 rows (gemv path 2,
    the same integer products in another k order) the difference is f32 rounding only."""
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m + k + n)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=k + n + dtype)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = ops.Weight(dtype, n, k, raw)
    try:
        ops.set_large_m_gemm(0)  # the mma.sync kernels (17 rows and more go to the tcgen05 GEMM by default)
        runs = [w.matmul_nt(x) for _ in range(5)]
        ops.set_gemv_path(2)
        small = w.matmul_nt(x)
    finally:
        ops.set_gemv_path(0)
        ops.set_large_m_gemm(ops.LARGE_M_DEFAULT)
        w.free()
    for r in runs[1:]:
        assert np.array_equal(r.view(np.uint32), runs[0].view(np.uint32))
    assert rel_l2(runs[0], small) < 2e-6
    assert rel_l2(runs[0], oracle.matmul_nt(x, raw, dtype, n)) < 2e-5


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_matmul_nt_activation_outliers_and_zeros(oracle, dtype):
    """Digit conversion edge cases: a huge outlier in one block, all-zero blocks, denormal-scale rows."""
    be, _ = synth.BLOCK[dtype]
    k, n = 1024, 24
    rng = np.random.default_rng(77)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=dtype)
    x = rng.standard_normal((4, k)).astype(np.float32)
    x[0, 5] = 3.0e4
    x[1, 256:512] = 0.0
    x[2] *= 1e-30
    x[3, :] = 0.0
    for rows in (x[:1], x[1:3], x):
        got = ops.matmul_nt(rows, raw, dtype, n)
        want = oracle.matmul_nt(rows, raw, dtype, n)
        assert np.all(np.isfinite(got))
        assert rel_l2(got, want) < REL_L2_BAR
    assert np.all(ops.matmul_nt(x[3:], raw, dtype, n) == 0.0)


def test_matmul_nt_q8_0_small_k_like_hidden_896(oracle):
    rng = np.random.default_rng(9)
    k, n = 896, 130
    raw = synth.random_bit_blocks(Q8_0, n * k // 32, seed=5)
    for m in (1, 2, 7):
        x = rng.standard_normal((m, k)).astype(np.float32)
        assert rel_l2(ops.matmul_nt(x, raw, Q8_0, n), oracle.matmul_nt(x, raw, Q8_0, n)) < 2e-5


def test_matmul_errors_mirror_reference():
    with pytest.raises(_lib.SapientCudaError) as e:
        ops.matmul_nt(np.zeros((1, 128), np.float32), np.zeros(72, np.uint8), Q4_K, 1)
    assert e.value.status == _lib.SP_ERR_SHAPE
    with pytest.raises(_lib.SapientCudaError):
        ops.matmul_nt(np.zeros((1, 48), np.float32), np.zeros(51, np.uint8), Q8_0, 1)
    w = ops.Weight(Q8_0, 4, 64, synth.random_bit_blocks(Q8_0, 8, 1))
    with pytest.raises(_lib.SapientCudaError) as e:
        w.matmul_nt(np.zeros((1, 32), np.float32))
    assert e.value.status == _lib.SP_ERR_SHAPE
    with pytest.raises(_lib.SapientCudaError):
        w.matmul_nt(np.zeros(64, np.float32))
    assert w.matmul_nt(np.zeros((0, 64), np.float32)).shape == (0, 4)


def test_norms(oracle):
    rng = np.random.default_rng(1)
    for rows, dim in [(1, 896), (5, 2560), (3, 4096), (2, 100)]:
        x = rng.standard_normal((rows, dim)).astype(np.float32) * 3
        w = (1 + 0.05 * rng.standard_normal(dim)).astype(np.float32)
        b = (0.02 * rng.standard_normal(dim)).astype(np.float32)
        assert rel_l2(ops.rms_norm(x, w, 1e-6), oracle.rms_norm(x, w, 1e-6)) < 1e-6
        assert rel_l2(ops.layer_norm(x, w, b, 1e-5), oracle.layer_norm(x, w, b, 1e-5)) < 1e-5
        assert rel_l2(ops.layer_norm(x, w, None, 1e-5), oracle.layer_norm(x, w, None, 1e-5)) < 1e-5
    y = ops.rms_norm(np.array([[3, 4]], np.float32), np.ones(2, np.float32), 0.0)
    assert np.allclose(y, np.array([3, 4], np.float32) / np.sqrt(np.float32(12.5)), atol=1e-6)
    y = ops.layer_norm(np.array([[1, 2], [3, 4]], np.float32), None, None, 1e-5)
    assert np.allclose(y, [[-1, 1], [-1, 1]], atol=1e-4)


def test_rope(oracle):
    rng = np.random.default_rng(2)
    # (heads, seq, head_dim, rotary_dim): full, Phi-2 partial 32/80, 64/64 (wgpu/tests/resident.rs:152-187)
    for H, S, D, R, base in [(3, 5, 64, 64, 1e6), (4, 3, 80, 32, 1e4), (2, 7, 128, 128, 5e5)]:
        x = rng.standard_normal((H, S, D)).astype(np.float32)
        pos = np.arange(11, 11 + S)
        got = ops.rope(x, pos, base, R)
        want = oracle.rope(x, pos, base, R)
        assert np.max(np.abs(got - want)) < 1e-6
        assert np.array_equal(got[:, :, R:], x[:, :, R:])
    x = np.array([1, 2, 3, 4], np.float32).reshape(1, 1, 4)
    assert np.allclose(ops.rope(x, [0], 10000.0), x, atol=1e-7)
    far = rng.standard_normal((1, 1, 128)).astype(np.float32)
    assert np.max(np.abs(ops.rope(far, [4095], 5e5) - oracle.rope(far, [4095], 5e5))) < 1e-6
    with pytest.raises(_lib.SapientCudaError):
        ops.rope(x, [0], 1e4, 3)
    with pytest.raises(_lib.SapientCudaError):
        ops.rope(x, [0], 1e4, 6)


# (H, Hkv, sq, sk, hd) from wgpu/tests/resident.rs:238-277 plus longer contexts spanning several KV pages
# the last four have enough (token, key) pairs for the tensor-core grouped-query kernel: groups of 4, 7, 6 and 8 heads,
# split and unsplit (sq > 4), last pages ragged
ATT_CASES = [(14, 2, 1, 23, 64), (4, 4, 6, 6, 80), (8, 2, 5, 9, 128), (32, 8, 1, 300, 128), (2, 1, 17, 50, 32),
             (32, 8, 1, 5003, 128), (14, 2, 3, 2001, 64), (12, 2, 6, 1100, 128), (16, 2, 2, 2500, 32)]


@pytest.mark.parametrize("H,Hkv,sq,sk,hd", ATT_CASES)
def test_attention(oracle, H, Hkv, sq, sk, hd):
    rng = np.random.default_rng(H + sk)
    q = rng.standard_normal((H, sq, hd)).astype(np.float32)
    k = f16_round(rng.standard_normal((Hkv, sk, hd)))  # the device cache is fp16: give both sides the same values
    v = f16_round(rng.standard_normal((Hkv, sk, hd)))
    got = ops.gqa_attention(q, k, v)
    want = oracle.attention(q, k, v, oracle.causal_mask(sq, sk))
    assert rel_l2(got, want) < 1e-5, rel_l2(got, want)
    # un-rounded K/V: only the fp16 storage error remains, still inside the per-op bar
    k2 = rng.standard_normal((Hkv, sk, hd)).astype(np.float32)
    v2 = rng.standard_normal((Hkv, sk, hd)).astype(np.float32)
    assert rel_l2(ops.gqa_attention(q, k2, v2), oracle.attention(q, k2, v2)) < REL_L2_BAR


def test_attention_uniform_scores_average_v():
    seq, dim = 4, 8
    v = np.repeat(np.arange(1, seq + 1, dtype=np.float32)[:, None], dim, 1).reshape(1, seq, dim)
    ones = np.ones((1, seq, dim), np.float32)
    out = ops.gqa_attention(ones[:, -1:], ones, v)
    assert np.allclose(out, 2.5, atol=1e-4)


def test_elementwise(oracle):
    rng = np.random.default_rng(4)
    a = (rng.standard_normal(5000) * 4).astype(np.float32)
    b = rng.standard_normal(5000).astype(np.float32)
    assert rel_l2(ops.silu(a), oracle.silu(a)) < 1e-6
    assert rel_l2(ops.gelu(a), oracle.gelu(a)) < 1e-6
    assert np.array_equal(ops.add(a, b), oracle.add(a, b))
    assert np.array_equal(ops.mul(a, b), oracle.mul(a, b))
    assert ops.gelu(np.zeros(1, np.float32))[0] == 0.0
    assert ops.silu(np.zeros(1, np.float32))[0] == 0.0


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
def test_embed_bit_exact_and_vocab_error(oracle, dtype):
    be, _ = synth.BLOCK[dtype]
    vocab, hidden = 50, 512
    raw = synth.random_bit_blocks(dtype, vocab * hidden // be, seed=3)
    ids = [0, 49, 7, 7, 31]
    w = ops.Weight(dtype, vocab, hidden, raw)
    got = w.embed(ids)
    want = oracle.embed(dtype, raw, vocab, hidden, ids)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    with pytest.raises(_lib.SapientCudaError) as e:
        w.embed([50])
    assert e.value.status == _lib.SP_ERR_VOCAB
    assert w.embed([]).shape == (0, hidden)


def test_argmax_last_maximum_wins(oracle):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((5, 151936)).astype(np.float32)
    x[1, 100] = x[1, 140000] = 50.0
    x[2, :] = 1.0
    x[3, 0] = 99.0
    got = ops.argmax(x)
    want = [oracle.argmax(r) for r in x]
    assert got.tolist() == want
    assert got[1] == 140000 and got[2] == 151935 and got[3] == 0
    assert ops.argmax(np.array([[1, 5, 3, 5, 2]], np.float32)).tolist() == [3]


def test_kernels_were_launched():
    before = ops.launch_count()
    ops.silu(np.ones(8, np.float32))
    assert ops.launch_count() == before + 1


# ── the other block formats the reference's loader keeps packed: Q4_0 and Q5_K ──
Q4_0, Q5_K = synth.Q4_0, synth.Q5_K


@pytest.mark.parametrize("dtype", [Q4_0, Q5_K])
def test_q4_0_and_q5_k_dequant_bit_exact_and_matmul(oracle, dtype):
    """Q4_0 (tensor.rs:362-377) and Q5_K with its per-element fifth bit (tensor.rs:421-467; the reference's own
    regression test for that bit: tensor.rs:796-824): dequantised values bit for bit on random-bit blocks, matmul_nt
    (kernels/quant.rs:104-114,1626-1665 row dots) within the operator bar. These formats run on the CUDA-core GEMV."""
    be, _ = synth.BLOCK[dtype]
    n, k = 37, 4 * 256
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=200 + dtype)
    w = ops.Weight(dtype, n, k, raw)
    got = w.dequant()
    want = oracle.dequant(dtype, raw, n * k).reshape(n, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    rng = np.random.default_rng(dtype)
    for m in (1, 3, 9, 20):
        x = rng.standard_normal((m, k)).astype(np.float32)
        assert rel_l2(w.matmul_nt(x), oracle.matmul_nt(x, raw, dtype, n)) < 2e-5
    # one row gathered from a Q5_K / Q4_0 embedding table
    assert np.array_equal(w.embed([5, 0, 36]).view(np.uint32), want[[5, 0, 36]].view(np.uint32))
    w.free()
    with pytest.raises(_lib.SapientCudaError):
        ops.Weight(dtype, 1, 48 if dtype == Q4_0 else 128, raw[:27 if dtype == Q4_0 else 88])


def test_q5_k_fifth_bit_is_per_element(oracle):
    """The reference's regression case (tensor.rs:796-824): d = 1, dmin = 0, every sub-block scale 1; qh[5] bit 0 sets
    element 5, qh[0] bit 2 (the first plane of the second 64-group) sets element 64, ql[3] = 2 gives element 3 the value 2;
    everything else is 0."""
    block = np.zeros(176, np.uint8)
    block[0:2] = np.array([1.0], np.float16).view(np.uint8)
    block[4:8] = 1    # 6-bit scales of sub-blocks 0..3
    block[12:16] = 1  # low nibbles: scales of sub-blocks 4..7
    block[16 + 5] = 0b00000001
    block[16 + 0] = 0b00000100
    block[48 + 3] = 0x02
    got = ops.Weight(Q5_K, 1, 256, block).dequant().reshape(-1)
    assert np.array_equal(got, oracle.dequant(Q5_K, block, 256))
    assert got[3] == 2.0 and got[5] == 16.0 and got[64] == 16.0 and np.count_nonzero(got) == 3
