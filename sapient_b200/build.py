"""Builds libsapient_cuda.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m sapient_b200.build [--force]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically
and has no other dependency, so the built file can be copied to a GPU machine.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libsapient_cuda.so")
SOURCES = ["kernels.cu", "attention.cu", "engine.cu", "engine_forward.cu", "engine_layers.cu", "engine_decode.cu", "gemv_imma.cu", "api.cu", "gguf.cu",
           "attention_static.cu", "tp.cu", "gemm_tc5.cu", "gemv_ring.cu", "spec.cu", "batcher.cu", "nccl_arm.cu", "gemv_rows.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--shared",
]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "sapient_cuda.h")]
    return any(os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    from concurrent.futures import ThreadPoolExecutor

    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "sapient_cuda.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)

    def compile_one(src: str) -> str:
        path, obj = os.path.join(CSRC, src), os.path.join(CSRC, src.replace(".cu", ".o"))
        fresh = os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), newest_header)
        if force or verbose or not fresh:
            cmd = ["nvcc", *FLAGS[:-1], "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    subprocess.run(["nvcc", "--shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT, *objs], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
