"""Generates tests/golden/golden_v1.npz (and, with --v2, golden_v2.npz: the block formats and the model family added
later, kept in a file of their own so that the first fixture never has to be regenerated) from the CPU oracle.

    python tests/golden/make_golden.py [--v2]

The reference is Rust and cannot be built in this environment, so these vectors come
from the oracle after it has been pinned against the reference's own known-answer
tests (tests/test_oracle_kat.py). They freeze the oracle's outputs: a later change to
the oracle, the synthetic weight generator or the CUDA path that moves any of them is
caught on CPU (oracle side) and on the GPU (CUDA side).
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle  # noqa: E402
from sapient_b200 import synth  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v1.npz")
MODELS = ["tiny_llama", "tiny_qwen", "tiny_phi2"]


def weights_digest(W) -> str:
    h = hashlib.sha256()
    for k in sorted(W):
        h.update(k.encode())
        h.update(np.ascontiguousarray(W[k][2]).tobytes())
    return h.hexdigest()


def model_case(name):
    cfg, Wt = synth.build_model(synth.CONFIGS[name], seed=7, device="cpu", max_ctx=64)
    W = synth.weights_to_numpy(Wt)
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], 12).astype(np.uint32)
    out = {"ids": ids, "digest": np.frombuffer(weights_digest(W).encode(), np.uint8)}
    for mode, tag in ((0, "ref"), (1, "f16")):
        e = oracle.OracleEngine(cfg, W, kv_mode=mode)
        logits = [e.forward_logits(ids, True)]
        toks = []
        for _ in range(4):
            toks.append(oracle.argmax(logits[-1]))
            logits.append(e.forward_logits([toks[-1]], True))
        out[f"logits_{tag}"] = np.stack(logits)
        out[f"tokens_{tag}"] = np.array(toks, np.uint32)
    return out


OUT2 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v2.npz")


def main_v2():
    """Q4_0 and Q5_K blocks (dequant + matmul) and the Phi-3-shaped tiny model."""
    data = {}
    rng = np.random.default_rng(43)
    for dtype, tag in ((synth.Q4_0, "q4_0"), (synth.Q5_K, "q5_k")):
        n, k, m = 6, 512, 3
        raw = synth.random_bit_blocks(dtype, n * k // synth.BLOCK[dtype][0], seed=dtype)
        x = rng.standard_normal((m, k)).astype(np.float32)
        data[f"{tag}_blocks"] = raw
        data[f"{tag}_x"] = x
        data[f"{tag}_dequant"] = oracle.dequant(dtype, raw, n * k).reshape(n, k)
        data[f"{tag}_y"] = oracle.matmul_nt(x, raw, dtype, n)
    for key, val in model_case("tiny_phi3").items():
        data[f"tiny_phi3_{key}"] = val
    np.savez_compressed(OUT2, **data)
    print(OUT2, os.path.getsize(OUT2), "bytes")


def main():
    if "--v2" in sys.argv:
        return main_v2()
    data = {}
    rng = np.random.default_rng(42)
    for dtype, tag in ((synth.Q4_K, "q4_k"), (synth.Q6_K, "q6_k"), (synth.Q8_0, "q8_0")):
        n, k, m = 6, 512, 3
        raw = synth.random_bit_blocks(dtype, n * k // synth.BLOCK[dtype][0], seed=dtype)
        x = rng.standard_normal((m, k)).astype(np.float32)
        data[f"{tag}_blocks"] = raw
        data[f"{tag}_x"] = x
        data[f"{tag}_dequant"] = oracle.dequant(dtype, raw, n * k).reshape(n, k)
        data[f"{tag}_y"] = oracle.matmul_nt(x, raw, dtype, n)
    for name in MODELS:
        for key, val in model_case(name).items():
            data[f"{name}_{key}"] = val
    np.savez_compressed(OUT, **data)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
