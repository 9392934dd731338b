"""Operator sweep of the standalone dequant-matmul  Y = X · Wᵀ  (weights resident as ggml blocks).

    python -m sapient_b200.sweep                      # the full grid, one JSON line per case
    python -m sapient_b200.sweep --dtype q4_k --n 14336 --k 4096 --m 1 --iters 50

Grid: Q4_K / Q6_K / Q8_0; N x K in {4096x4096, 14336x4096, 4096x14336, 128256x4096};
M in {1, 2, 4, 8, 16, 32, 64, 512}. Weights are random N(0, 0.02) quantised per block,
activations N(0, 1) f32.

Timing: CUDA events on the launching stream around `iters` back-to-back calls after
warm-up; each call uses the next of `rotate` distinct weight buffers whose total size
exceeds the 126 MB L2, so the blocks really come from HBM. Achieved GB/s uses the
algorithmic bytes N·K·bpw + 4·M·K + 4·M·N.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import ops, synth

DTYPES = {"q4_k": synth.Q4_K, "q6_k": synth.Q6_K, "q8_0": synth.Q8_0}
SHAPES = [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]
MS = [1, 2, 4, 8, 16, 32, 64, 512]
L2_BYTES = 126 << 20


def measured_hbm_gbs() -> tuple[float, str]:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def run_case(dtype_name: str, n: int, k: int, m: int, iters: int, warmup: int, rotate: int | None, path: int, seed: int = 0,
             large_m: bool = False, large_m_mode: int | None = None):
    """large_m: calls of 17 rows and more on the tcgen05 GEMM with operands rounded to fp16 instead of its default exact-class
    mode. large_m_mode: the mode number itself (0 integer passes on the mma.sync kernels, 1 fp16-rounded, 2 exact-class)."""
    import torch

    dtype = DTYPES[dtype_name]
    wbytes = synth.byte_count(dtype, n * k)
    if rotate is None:
        rotate = max(2, -(-2 * L2_BYTES // wbytes))
    g = torch.Generator(device="cuda").manual_seed(seed)
    weights = []
    for r in range(rotate):
        rows_per = max(1, (1 << 25) // k)
        parts = []
        for r0 in range(0, n, rows_per):
            w = torch.randn(min(rows_per, n - r0), k, generator=g, device="cuda") * 0.02
            parts.append(synth.quantize(dtype, w))
        raw = torch.cat(parts, 0).reshape(-1).cpu().numpy()
        weights.append(ops.Weight(dtype, n, k, raw))
        del parts, raw
    x = torch.randn(m, k, generator=g, device="cuda", dtype=torch.float32)
    y = torch.empty(m, n, device="cuda", dtype=torch.float32)
    ops.set_gemv_path(path)
    mode = large_m_mode if large_m_mode is not None else (1 if large_m else ops.LARGE_M_DEFAULT)
    ops.set_large_m_gemm(mode)
    warmup = max(warmup, rotate)  # every rotated buffer has made its one-time allocations before the clock starts
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(warmup):
            weights[i % rotate].matmul_nt_dev(x.data_ptr(), m, y.data_ptr(), stream.cuda_stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for i in range(iters):
            weights[i % rotate].matmul_nt_dev(x.data_ptr(), m, y.data_ptr(), stream.cuda_stream)
        e1.record(stream)
        stream.synchronize()
    ops.set_gemv_path(0)
    ops.set_large_m_gemm(ops.LARGE_M_DEFAULT)
    us = e0.elapsed_time(e1) * 1000.0 / iters
    alg = wbytes + 4 * m * k + 4 * m * n
    peak, src = measured_hbm_gbs()
    gbs = alg / us / 1e3
    for w in weights:
        w.free()
    return {"op": "matmul_nt", "dtype": dtype_name, "n": n, "k": k, "m": m, "us": us, "gbs": gbs, "frac_of_8TBs": gbs / 8000.0,
            "frac_of_hbm_peak": gbs / peak, "peak_source": src, "tflops": 2.0 * m * n * k / us / 1e6, "weight_bytes": wbytes,
            "rotate": rotate, "iters": iters,
            "kernel": "cuda-core" if path else ("tcgen05, fp16 operands" if mode == 1 and m >= 17 else
                                                "tcgen05, exact-class operands" if mode == 2 and m >= 17 else
                                                "tensor-core GEMV (mma.sync), exact integer products")}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", choices=list(DTYPES))
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--m", type=int)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rotate", type=int, default=None)
    ap.add_argument("--path", type=int, default=0, help="0 tensor-core GEMV (default), 1 CUDA-core GEMV")
    ap.add_argument("--max-m", type=int, default=512)
    ap.add_argument("--large-m", action="store_true", help="17 rows and more on the tcgen05 GEMM with operands rounded to fp16 (default: exact-class operands)")
    ap.add_argument("--large-m-mode", type=int, choices=[0, 1, 2], default=None,
                    help="17 rows and more: 0 integer passes on the mma.sync kernels, 1 tcgen05 fp16-rounded, 2 tcgen05 exact-class (default)")
    a = ap.parse_args()
    dts = [a.dtype] if a.dtype else list(DTYPES)
    shapes = [(a.n, a.k)] if a.n and a.k else SHAPES
    ms = [a.m] if a.m else [m for m in MS if m <= a.max_m]
    for dt in dts:
        for n, k in shapes:
            for m in ms:
                print(json.dumps(run_case(dt, n, k, m, a.iters, a.warmup, a.rotate, a.path, large_m=a.large_m, large_m_mode=a.large_m_mode)), flush=True)


if __name__ == "__main__":
    main()
