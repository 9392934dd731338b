"""Parity of the standalone dequant-matmul at the operator sweep's real shapes (N x K in 4096x4096, 14336x4096,
4096x14336, 128256x4096; Q4_K, Q6_K, Q8_0; M in 1, 16, 32, 512): tile indexing beyond 2^31 bytes, grids several waves
deep and the split-K tail of the large-M GEMM only occur at these sizes.

The CPU oracle would need minutes per full matrix, so each case checks a random subset of output rows — all
activation rows, >= 256 weight rows spread over the whole matrix including its first and last tile — against
`oracle.matmul_nt` (kernels/matmul.rs:862-943,1111-1167,575-689) on exactly those rows' blocks: 1e-3 relative L2
(the operator bar) per activation row, and the dequantised values of the same rows must be bit-identical
(tensor.rs:378-398,468-476).
"""
import numpy as np
import pytest

from helpers import rel_l2
from sapient_b200 import ops, synth

pytestmark = pytest.mark.gpu

DT = {"q4_k": synth.Q4_K, "q6_k": synth.Q6_K, "q8_0": synth.Q8_0}
SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
MS = [1, 16, 32, 512]
ROWS = 256


def _weights(dtype, n, k, seed):
    import torch

    g = torch.Generator(device="cuda").manual_seed(seed)
    rows_per = max(1, (1 << 25) // k)
    parts = []
    for r0 in range(0, n, rows_per):
        w = torch.randn(min(rows_per, n - r0), k, generator=g, device="cuda") * 0.02
        parts.append(synth.quantize(dtype, w))
    return torch.cat(parts, 0).cpu().numpy()  # [n, row_bytes] uint8


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("dtype_name", list(DT))
def test_matmul_nt_at_sweep_shapes(oracle, dtype_name, n, k):
    dtype = DT[dtype_name]
    raw = _weights(dtype, n, k, seed=n + k)
    assert raw.shape[0] == n
    rng = np.random.default_rng(n ^ k)
    pick = np.unique(np.concatenate([np.arange(16), np.arange(n - 16, n), rng.integers(0, n, ROWS)]))
    sub = np.ascontiguousarray(raw[pick])
    w = ops.Weight(dtype, n, k, raw.reshape(-1))
    try:
        # bit-exact dequant of the picked rows (the full matrix is dequantised on the device, only these rows compared)
        deq = w.dequant()[pick]
        want_deq = oracle.dequant(dtype, sub.reshape(-1), pick.size * k).reshape(pick.size, k)
        assert np.array_equal(deq.view(np.uint32), want_deq.view(np.uint32)), "dequantised rows differ in bits"
        del deq, want_deq
        for m in MS:
            x = rng.standard_normal((m, k)).astype(np.float32)
            got = w.matmul_nt(x)[:, pick]
            want = oracle.matmul_nt(x, sub.reshape(-1), dtype, pick.size)
            worst = max(rel_l2(got[i], want[i]) for i in range(m))
            assert worst < 1e-3, (dtype_name, n, k, m, worst)
            if m >= 17:  # the tcgen05 GEMM with operands rounded to fp16 (mode 1) on the same inputs
                ops.set_large_m_gemm(1)
                try:
                    got = w.matmul_nt(x)[:, pick]
                finally:
                    ops.set_large_m_gemm(ops.LARGE_M_DEFAULT)
                worst = max(rel_l2(got[i], want[i]) for i in range(m))
                assert worst < 1e-3, (dtype_name, n, k, m, "tcgen05", worst)
    finally:
        w.free()
