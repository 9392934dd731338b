"""Measurements of the other workload shapes of the hot path (bench.py covers batch-1 decode of the
Llama-3-8B shape). One JSON line per case; synthetic seeded weights and token ids throughout.

    python -m sapient_b200.configs_bench c0        Qwen2.5-0.5B shape, batch-1 greedy decode (128-token prompt, 128 steps)
    python -m sapient_b200.configs_bench c2        Phi-2 shape, Q8_0: 512-token prefill, then 256 decode steps
    python -m sapient_b200.configs_bench c3b32     Llama-3-8B shape, 32 sequences decoded together (prompt 256 by default)
    python -m sapient_b200.configs_bench c4        speculative decoding, Qwen2.5-1.5B-shaped target + 0.5B-shaped draft, k = 4
    python -m sapient_b200.configs_bench prefill --model llama8b --prompt 512
                                                   one prompt through an engine whose step holds it whole: time and kernel families

Rooflines: bytes one step must stream (every weight matrix once + the KV entries read) over the measured HBM copy
bandwidth (MEASURED_PEAKS.json next to the package, else 6650 GB/s) and over 8 TB/s.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np

from . import speculative, synth
from .engine import ForwardEngine


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _weight_bytes(cfg, W) -> int:
    total = sum(raw.size for name, (dt, dims, raw) in W.items() if len(dims) == 2 and "embed_tokens" not in name)
    if cfg.get("tied"):
        total += W["model.embed_tokens.weight"][2].size
    return int(total)


def _build(name: str, max_ctx: int, seed: int):
    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=seed, device="cuda", max_ctx=max_ctx)
    Wn = synth.weights_to_numpy(W)
    del W
    torch.cuda.empty_cache()
    return cfg, Wn


def _timed(stream, fn):
    import torch

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def _engine(cfg, W, **kw):
    import torch

    eng = ForwardEngine.from_weights(cfg, W, **kw)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)
    return eng, stream


def _roof(bytes_per_step: float, ms_per_step: float) -> dict:
    peak, src = _peak()
    gbs = bytes_per_step / 1e9 / (ms_per_step / 1e3)
    return {"bytes_per_step": int(bytes_per_step), "achieved_gbs": gbs, "frac_of_measured_peak": gbs / peak, "peak_gbs": peak,
            "peak_source": src, "frac_of_8TBs": gbs / 8000.0}


def decode_case(name: str, prompt_len: int, steps: int, batch: int, label: str, prefill_timed: bool = False, fast: bool = False) -> dict:
    cfg, W = _build(name, max_ctx=prompt_len + steps + 64, seed=1000)
    # rows per forward step: a whole prompt of up to 512 tokens in one step (fewer, fuller launches of the large-M GEMM)
    eng, stream = _engine(cfg, W, max_batch=batch, max_tokens=max(256, min(prompt_len, 512)), fast_large_m=fast)
    rng = np.random.default_rng(0)
    first = np.empty(batch, np.uint32)
    prefill_ms = 0.0
    for s in range(batch):
        ids = rng.integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
        out = {}

        def run(ids=ids, s=s, out=out):
            out["lg"] = eng.forward_slot(s, ids)

        prefill_ms += _timed(stream, run)
        first[s] = int(np.flatnonzero(out["lg"] == out["lg"].max())[-1])
    warm = 8
    toks = eng.decode_greedy(first, list(range(batch)), warm)
    ms = _timed(stream, lambda: eng.decode_greedy(toks[-1], list(range(batch)), steps, fetch=False))
    kv_per_pos = 2 * cfg["n_layers"] * cfg["n_kv_heads"] * cfg["head_dim"] * 2
    ctx_mid = prompt_len + warm + steps // 2
    step_bytes = _weight_bytes(cfg, W) + batch * ctx_mid * kv_per_pos
    line = {"case": label, "model": name, "batch": batch, "prompt_len": prompt_len, "steps": steps, "ms_per_step": ms / steps,
            "tokens_per_s": batch * steps / (ms / 1e3), "roofline": _roof(step_bytes, ms / steps), "data": "synthetic",
            "large_m_path": "tcgen05 GEMM, operands rounded to fp16 (opt-in)" if fast else "tcgen05 GEMM, exact-class operands (default)"}
    if prefill_timed:
        line["prefill_tokens_per_s"] = batch * prompt_len / (prefill_ms / 1e3)
        line["prefill_ms"] = prefill_ms
    eng.close()
    return line


def prefill_case(name: str, prompt_len: int, reps: int = 3, fast: bool = False) -> dict:
    cfg, W = _build(name, max_ctx=prompt_len + 64, seed=3000)
    eng, stream = _engine(cfg, W, max_tokens=min(prompt_len, 1024), fast_large_m=fast)
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], prompt_len).astype(np.uint32)
    eng.forward_logits(ids, False)  # one-time allocations and attribute settings
    ms = min(_timed(stream, lambda: eng.forward_logits(ids, False)) for _ in range(reps))
    eng.set_profile(True)
    eng.forward_logits(ids, False)
    fam = {k: {"ms": round(v[0], 3), "launches": v[1]} for k, v in eng.profile_read().items()}
    eng.set_profile(False)
    eng.close()
    return {"case": "prefill", "model": name, "prompt_len": prompt_len, "ms": ms, "tokens_per_s": prompt_len / (ms / 1e3),
            "families": fam, "data": "synthetic",
            "large_m_path": "tcgen05 GEMM, operands rounded to fp16 (opt-in)" if fast else "tcgen05 GEMM, exact-class operands (default)"}


def spec_case(k: int, prompt_len: int, new_tokens: int) -> dict:
    """Speculative decoding, Qwen2.5-1.5B-shaped target + 0.5B-shaped draft whose embedding / output matrix is the
    target's projected 1536 -> 896, draft length k, greedy accept, batch 1: the loop inside the library
    (sp_cuda_spec_greedy: device-resident draft loop, one k + 1 row verify pass per round, only token ids cross the host
    boundary), beside target-only greedy decoding through the same library (device-resident loop) and the reference's
    two-pass host schedule with rejection sampling."""
    import torch

    (tcfg, tW), (dcfg, dW) = synth.build_spec_pair("qwen15b", "qwen05b", seed=4000, device="cuda", max_ctx=prompt_len + new_tokens + 64)
    tW, dW = synth.weights_to_numpy(tW), synth.weights_to_numpy(dW)
    torch.cuda.empty_cache()
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, tcfg["vocab"], prompt_len).astype(np.uint32)
    out = {"case": "c4", "target": "qwen15b", "draft": "qwen05b (embedding = target's, projected 1536 -> 896)", "k": k, "prompt_len": prompt_len,
           "new_tokens": new_tokens, "data": "synthetic random-init models: whatever acceptance they give is reported"}
    # yardstick: the target alone, greedy, loop resident on the device
    eng, stream = _engine(tcfg, tW, max_tokens=256)
    lg = eng.forward_logits(prompt, True)
    first = speculative.greedy(lg)
    eng.decode_greedy([first], [0], 4)
    eng.truncate_cache(prompt_len)
    t0 = time.perf_counter()
    ref_tokens = [first] + [int(t) for t in eng.decode_greedy([first], [0], new_tokens - 1)[:, 0]]
    out["target_only_tokens_per_s"] = new_tokens / (time.perf_counter() - t0)
    eng.close()
    for tag, cfg_d, W_d in (("projected_draft", dcfg, dW), ("draft_equals_target", tcfg, tW)):
        target, _ = _engine(tcfg, tW, max_tokens=256)
        draft, _ = _engine(cfg_d, W_d, max_tokens=256)
        speculative.generate_greedy_device(target, draft, prompt, 16, k=k)  # warm-up: step graphs of 1 and k + 1 rows
        t0 = time.perf_counter()
        toks, st = speculative.generate_greedy_device(target, draft, prompt, new_tokens, k=k)
        dt = time.perf_counter() - t0  # includes both prefills, like the yardstick does not: reported separately below
        t0 = time.perf_counter()
        target.forward_logits(prompt, False)
        draft.forward_logits(prompt, False)
        prefill = time.perf_counter() - t0
        out[tag] = {"tokens_per_s": len(toks) / max(dt - prefill, 1e-9), "tokens_per_s_with_prefill": len(toks) / dt, "rounds": st.rounds,
                    "drafted": st.drafted, "accepted_drafts": st.accepted_drafts, "acceptance": st.accepted_drafts / max(st.drafted, 1),
                    "tokens_per_round": len(toks) / max(st.rounds, 1), "identical_to_target_greedy": toks == ref_tokens[: len(toks)]}
        target.close()
        draft.close()
    # the reference's schedule (k-row verify + single-token pass, rejection sampling, logits on the host every forward)
    target, _ = _engine(tcfg, tW, max_tokens=256)
    draft, _ = _engine(dcfg, dW, max_tokens=256)
    t0 = time.perf_counter()
    toks, st = speculative.generate(target, draft, prompt, min(new_tokens, 64), k=k, seed=0)
    dt = time.perf_counter() - t0
    out["reference_schedule_host_loop"] = {"tokens_per_s_with_prefill": len(toks) / dt, "rounds": st.rounds, "accepted_drafts": st.accepted_drafts,
                                           "drafted": st.drafted}
    target.close()
    draft.close()
    return out


def load_case(name: str) -> dict:
    """Load path: the model written as a GGUF file (tmpfs when there is one), then sp_cuda_engine_from_gguf timed end to
    end — map the file, parse, stage the tensors through pinned buffers, un-permute / repack on the device, allocate."""
    import tempfile

    import torch

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=3000, device="cuda", max_ctx=512)
    Wc = {k: (dt, dims, t.cpu()) for k, (dt, dims, t) in W.items()}
    del W
    torch.cuda.empty_cache()
    d = "/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir()
    path = os.path.join(d, f"sapient_{name}.gguf")
    t0 = time.perf_counter()
    synth.write_gguf(path, cfg, Wc)
    write_s = time.perf_counter() - t0
    size = os.path.getsize(path)
    out = {"case": "load", "model": name, "file_bytes": size, "write_s": write_s, "runs": []}
    try:
        for _ in range(2):
            t0 = time.perf_counter()
            eng = ForwardEngine.from_gguf(path, max_ctx=512)
            total = time.perf_counter() - t0
            sec, nb = eng.load_stats()
            out["runs"].append({"from_gguf_s": total, "upload_s": sec, "upload_bytes": nb, "upload_gbs": nb / 1e9 / max(sec, 1e-9),
                                "overall_gbs": size / 1e9 / total})
            eng.close()
    finally:
        os.remove(path)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["c0", "c2", "c3b32", "c4", "prefill", "load"])
    ap.add_argument("--model", default="llama8b", choices=sorted(synth.CONFIGS))
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--fast", action="store_true", help="steps of 17 rows and more on the tcgen05 GEMM with operands rounded to fp16 (default: exact-class operands)")
    a = ap.parse_args()
    if a.case == "c0":
        line = decode_case("qwen05b", a.prompt or 128, a.steps or 128, 1, "c0", prefill_timed=True, fast=a.fast)
    elif a.case == "c2":
        line = decode_case("phi2", a.prompt or 512, a.steps or 256, 1, "c2", prefill_timed=True, fast=a.fast)
    elif a.case == "c3b32":
        line = decode_case("llama8b", a.prompt or 256, a.steps or 64, 32, "c3b32", prefill_timed=True, fast=a.fast)
    elif a.case == "prefill":
        line = prefill_case(a.model, a.prompt or 512, fast=a.fast)
    elif a.case == "load":
        line = load_case(a.model)
    else:
        line = spec_case(4, a.prompt or 256, a.steps or 512)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
