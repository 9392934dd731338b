"""Large-M dequant GEMM on tcgen05 / TMEM (gemm_tc5.cu) through sp_cuda_matmul_nt, against the CPU oracle and
against the exact integer-product passes (mode 0 of sp_cuda_set_large_m_gemm); mode 1 = operands rounded to fp16,
mode 2 (the default) = exact-class operands.

Bar: 1e-3 relative L2 per op. The kernel rounds the (exactly dequantised) weights and the activations to fp16 and
accumulates in fp32, so it lands near 2e-4."""
import numpy as np
import pytest

from helpers import rel_l2
from sapient_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu
Q8_0, Q4_K, Q6_K = synth.Q8_0, synth.Q4_K, synth.Q6_K


def _large_m(on) -> None:
    _lib.check(_lib.lib().sp_cuda_set_large_m_gemm(int(on)))


@pytest.fixture(autouse=True)
def _opt_in():
    """Most tests here are about the fp16-operand mode (1); the process default (2, exact-class operands) is put back
    afterwards."""
    _large_m(1)
    yield
    _large_m(2)


# (m, k, n): m not a multiple of 16 / over 256 (two CTA columns), n not a multiple of 128 / 16, several K chunks
CASES = [(17, 256, 48), (32, 512, 144), (40, 256, 128), (64, 256, 128), (80, 512, 200), (100, 1024, 130), (300, 768, 72), (512, 512, 384)]


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
@pytest.mark.parametrize("m,k,n", CASES)
def test_large_m_gemm_matches_oracle_and_gemv(oracle, dtype, m, k, n):
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m + k + n)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=m + n + dtype)
    x = rng.standard_normal((m, k)).astype(np.float32)
    want = oracle.matmul_nt(x, raw, dtype, n)
    try:
        _large_m(True)
        got = ops.matmul_nt(x, raw, dtype, n)
        _large_m(False)
        gemv = ops.matmul_nt(x, raw, dtype, n)
    finally:
        _large_m(1)
    assert got.shape == (m, n) and np.all(np.isfinite(got))
    assert rel_l2(gemv, want) < 3e-4
    err = rel_l2(got, want)
    assert err < 1e-3, err
    assert err < 5e-4, err  # expected ~2e-4 (fp16 operands)
    # every output element, not only the norm: a misplaced tile or a wrong swizzle shows up as O(1) errors
    scale = np.abs(want).max()
    assert np.abs(got - want).max() < 5e-3 * scale


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K, Q8_0])
@pytest.mark.parametrize("m,k,n", CASES + [(32, 4096, 1024), (64, 2048, 640), (200, 4096, 300), (128, 14336, 256)])
def test_exact_operand_mode_is_at_the_level_of_the_integer_path(oracle, dtype, m, k, n):
    """Mode 2: weights and activations each as an fp16 leading part plus remainder, three products per chunk of K. The
    result must sit where the exact integer-digit GEMV sits (2e-5 of the oracle, whose own f32 sums differ by that much
    between summation orders), two hundred times below the fp16-operand mode."""
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m + k + n + 1)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=m + n + dtype + 1)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0, 3] = 250.0   # an outlier, a small row, a row far below the fp16 range and a zero row: rows are scaled by a power
    x[1] *= 1e-3      # of two before they are split, so none of this reaches the fp16 limits
    x[2] *= 1e-30
    x[3] = 0.0
    want = oracle.matmul_nt(x, raw, dtype, n)
    try:
        _large_m(2)
        got = ops.matmul_nt(x, raw, dtype, n)
        again = ops.matmul_nt(x, raw, dtype, n)
    finally:
        _large_m(True)
    assert got.shape == (m, n) and np.all(np.isfinite(got))
    assert np.array_equal(got, again)
    assert np.all(got[3] == 0.0)
    worst = max(rel_l2(got[i], want[i]) for i in range(m) if i != 3)
    assert worst < 2e-5, worst


@pytest.mark.parametrize("m,k,n", [(64, 128, 64), (40, 384, 130), (300, 896, 200), (33, 1152, 272)])
def test_large_m_gemm_q8_0_widths_that_are_odd_multiples_of_128(oracle, m, k, n):
    """Q8_0 rows tiled four blocks at a time (the Qwen2.5-0.5B width 896 is one): one tile per 128-column chunk."""
    rng = np.random.default_rng(m + k + n)
    raw = synth.random_bit_blocks(Q8_0, n * k // 32, seed=m + n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    want = oracle.matmul_nt(x, raw, Q8_0, n)
    got = ops.matmul_nt(x, raw, Q8_0, n)
    assert got.shape == (m, n) and np.all(np.isfinite(got))
    assert rel_l2(got, want) < 5e-4
    assert np.abs(got - want).max() < 5e-3 * np.abs(want).max()


def test_large_m_gemm_quantised_gaussian_weights(oracle):
    """Weights as the synthetic models have them (N(0, 0.02) quantised), activations with a few large entries."""
    import torch

    m, k, n = 64, 1024, 256
    g = torch.Generator().manual_seed(5)
    w = torch.randn(n, k, generator=g) * 0.02
    raw = synth.quantize(Q4_K, w).reshape(-1).numpy()
    x = torch.randn(m, k, generator=g).numpy().astype(np.float32)
    x[3, 17] = 80.0
    got = ops.matmul_nt(x, raw, Q4_K, n)
    want = oracle.matmul_nt(x, raw, Q4_K, n)
    assert rel_l2(got, want) < 5e-4


@pytest.mark.parametrize("dtype,m,k,n", [(Q4_K, 64, 4096, 1024), (Q6_K, 200, 2048, 640), (Q8_0, 32, 4096, 300)])
def test_split_last_wave_is_reproducible_bit_for_bit(oracle, dtype, m, k, n):
    """Grids smaller than the GPU split each weight tile's K range over several CTAs. Their partial tiles are summed in
    part order by the last CTA to arrive, so repeated calls give identical bits (an atomic-add tail would not), and
    the result still meets the operator bar."""
    be, _ = synth.BLOCK[dtype]
    rng = np.random.default_rng(m + k + n)
    raw = synth.random_bit_blocks(dtype, n * k // be, seed=k + n + dtype)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = ops.Weight(dtype, n, k, raw)
    try:
        runs = [w.matmul_nt(x) for _ in range(6)]
    finally:
        w.free()
    for r in runs[1:]:
        assert np.array_equal(r.view(np.uint32), runs[0].view(np.uint32))
    assert rel_l2(runs[0], oracle.matmul_nt(x, raw, dtype, n)) < 5e-4
