"""Shared helpers of the parity tests."""
import numpy as np

from sapient_b200 import synth


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))


def f16_round(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def tiny_model(name: str, seed: int = 7, max_ctx: int = 64):
    cfg, W = synth.build_model(synth.CONFIGS[name], seed=seed, device="cpu", max_ctx=max_ctx)
    return cfg, synth.weights_to_numpy(W)


def oracle_engine(oracle, cfg, W, kv_mode: int = 0):
    return oracle.OracleEngine(cfg, W, kv_mode=kv_mode)


def has_cuda() -> bool:
    from sapient_b200 import _lib

    return _lib.lib().sp_cuda_device_count() > 0
