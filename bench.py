"""Benchmark of the quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config.workload): batch-1 greedy decode of a Llama-3-8B-shaped decoder with
random-init N(0, 0.02) weights quantised to the Q4_K_M-like GGUF block layout
(Q4_K; Q6_K for output/token_embd and for attn_v/ffn_down on even layers), after a
128-token random prompt. One step = one decode step (one token per sequence).

  value      tokens/s with the loop resident on the device (token ids never leave HBM)
  e2e        tokens/s through ForwardEngine.forward_logits with host buffers: per step the
             token id goes host->device and the full f32 logits come back
  roofline   the dequant-GEMV kernel: algorithmic weight bytes per step / its device time
  cpu_baseline  the CPU restatement of the reference's x86 path on this host's cores

--impl reference times that CPU restatement alone (the reference is Rust and cannot be
built here), same metric/config, all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "llama8b"
NCU_TRAFFIC_RATIO = 1.000  # dram bytes / algorithmic bytes of the GEMV kernel, from the committed ncu summary
PROMPT = 128
CPU_PROMPT = 4


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc, self.thr = gpu_index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.perf_counter(), line.strip()))
        self.thr = threading.Thread(target=pump, daemon=True)
        self.thr.start()

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        sm, mx, reasons, power = [], [], set(), []
        for t, line in self.rows:
            if t < t0 or t > t1 + 0.05:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": float(max(power))}


def build_weights(device: str, seed: int = 3000):
    import torch

    from sapient_b200 import synth

    cfg, W = synth.build_model(synth.CONFIGS[MODEL], seed=seed, device=device, max_ctx=4096)
    Wn = synth.weights_to_numpy(W)
    del W
    if device != "cpu":
        torch.cuda.empty_cache()
    return cfg, Wn


def step_weight_bytes(cfg, W) -> int:
    """Algorithmic weight bytes one decode step streams: every 2-D matrix once (lm_head included; the
    embedding gather touches one row)."""
    total = 0
    for name, (dt, dims, raw) in W.items():
        if len(dims) == 2 and "embed_tokens" not in name:
            total += raw.size
    if cfg.get("tied"):
        total += W["model.embed_tokens.weight"][2].size
    return total


def cpu_decode_rate(cfg, W, steps: int, budget_s: float, prompt_len: int = CPU_PROMPT, prompt_budget_s: float = 0.0):
    """tokens/s of the CPU restatement: `steps` decode steps after a prompt, stopping early at budget_s. The prompt is
    fed 16 tokens at a time until prompt_len tokens are in the cache or prompt_budget_s has passed (at least CPU_PROMPT
    tokens always). All host cores are used whatever OMP_NUM_THREADS the launcher exported.
    Returns (tok/s, decode steps done, threads, prompt tokens fed)."""
    from oracle import oracle

    threads = oracle.use_all_cores()
    eng = oracle.OracleEngine(cfg, W, kv_mode=0)
    ids = np.random.default_rng(1).integers(0, cfg["vocab"], max(prompt_len, CPU_PROMPT)).astype(np.uint32)
    fed, tp0 = 0, time.perf_counter()
    logits = None
    while fed < len(ids):
        n = CPU_PROMPT if fed == 0 else min(16, len(ids) - fed)
        logits = eng.forward_logits(ids[fed:fed + n], True)
        fed += n
        if fed >= CPU_PROMPT and time.perf_counter() - tp0 > prompt_budget_s:
            break
    tok = oracle.argmax(logits)
    done, t0 = 0, time.perf_counter()
    while done < steps:
        logits = eng.forward_logits([tok], True)
        tok = oracle.argmax(logits)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return done / dt, done, threads, fed


B32_BATCH, B32_PROMPT, B32_WARM, B32_STEPS = 32, 1024, 4, 24


def batch32_section(cfg, W, wbytes: int, local: int, rank: int, world: int, stream, barrier, peaks) -> dict:
    """The other half of the metric: 32 sequences with 1024-token prompts decoded together over the paged fp16 KV cache
    (the tensor-parallel configuration of the benchmark at its own sizes; one GPU holds it whole, N GPUs split it).
    Three timings of the same step at context ~1024: the default (tcgen05 GEMM with exact-class operands), the same GEMM
    with operands rounded to fp16 (opt-in) and integer-digit GEMV passes of 10 rows (opt-in). Prompts are prefilled
    untimed on the fastest path in every case."""
    import torch

    from sapient_b200.engine import ForwardEngine

    eng = ForwardEngine.from_weights(cfg, W, device=local, max_batch=B32_BATCH, max_tokens=512, tp_rank=rank, tp_size=world)
    if world > 1:
        eng.tp_connect()
    eng.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(32)
    eng.set_large_m_gemm(1)  # untimed prefill on the fastest path
    first = np.empty(B32_BATCH, np.uint32)
    for s in range(B32_BATCH):
        lg = eng.forward_slot(s, rng.integers(0, cfg["vocab"], B32_PROMPT).astype(np.uint32))
        first[s] = int(np.flatnonzero(lg == lg.max())[-1]) + eng.vocab_first
    if world > 1:
        # every rank must feed the same first tokens: take rank 0's choice of its own vocabulary slice (any valid id does)
        import torch.distributed as dist

        t = torch.from_numpy(first.astype(np.int64)).to(f"cuda:{local}")
        dist.broadcast(t, 0)
        first = t.cpu().numpy().astype(np.uint32)
    slots = list(range(B32_BATCH))
    out = {"batch": B32_BATCH, "prompt_len": B32_PROMPT, "steps": B32_STEPS, "model": MODEL, "kv": "fp16 paged/16"}
    kv_per_pos = 2 * cfg["n_layers"] * cfg["n_kv_heads"] * cfg["head_dim"] * 2
    # exact: the default (tcgen05 GEMM, exact-class operands); tcgen05: its fp16-operand mode; integer_passes: the mma.sync
    # GEMV passes of 10 rows the default replaced
    modes = [("exact", 2), ("tcgen05", 1), ("integer_passes", 0)]
    for tag, fast in modes:
        for s in slots:
            eng.truncate_cache(B32_PROMPT, s)
        eng.set_large_m_gemm(fast)
        toks = eng.decode_greedy(first, slots, B32_WARM)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record(stream)
        eng.decode_greedy(toks[-1], slots, B32_STEPS, fetch=False)
        ev1.record(stream)
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device=f"cuda:{local}", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        ctx_mid = B32_PROMPT + B32_WARM + B32_STEPS // 2
        step_bytes = (wbytes + B32_BATCH * ctx_mid * kv_per_pos) / world
        gbs = step_bytes / 1e9 / (ms / B32_STEPS / 1e3)
        out[tag] = {"tokens_per_s": B32_BATCH * B32_STEPS / (ms / 1e3), "ms_per_step": ms / B32_STEPS, "context": ctx_mid,
                    "bytes_per_step_per_gpu": int(step_bytes), "achieved_gbs_per_gpu": gbs, "frac_of_measured_peak": gbs / peaks["hbm_gbs"],
                    "frac_of_8TBs": gbs / 8000.0}
    out["exact"]["path"] = "tcgen05 / TMEM dequant GEMM, exact-class operands (fp16 leading part + remainder of weights and activations), the default"
    out["tcgen05"]["path"] = "tcgen05 / TMEM dequant GEMM, operands rounded to fp16 (opt-in)"
    out["integer_passes"]["path"] = "integer-digit mma.sync GEMV passes of 10 rows (opt-in)"
    eng.close()
    return out


def sweep_section() -> list:
    """Operator sweep of the standalone dequant-matmul for the four benchmark shapes and the three block formats (weights
    rotated through more than twice the L2, CUDA events on the launching stream): achieved GB/s at M = 1 (tensor-core GEMV)
    and at M = 32 (the default for 17 rows and more: tcgen05 GEMM with exact-class operands) and TFLOP/s at M = 512 on the
    tcgen05 GEMM in both modes (useful flops; the exact-class mode issues three products per useful one)."""
    from sapient_b200 import sweep

    rows = []
    for dt in ("q4_k", "q6_k", "q8_0"):
        for n, k in sweep.SHAPES:
            big = n * k > (1 << 28)
            r1 = sweep.run_case(dt, n, k, 1, 24 if big else 60, 3, None, 0)
            r32 = sweep.run_case(dt, n, k, 32, 16 if big else 40, 3, None, 0)
            r512 = sweep.run_case(dt, n, k, 512, 8 if big else 20, 2, 2 if big else None, 0, large_m=True)
            r512x = sweep.run_case(dt, n, k, 512, 8 if big else 20, 2, 2 if big else None, 0)
            rows.append({"dtype": dt, "n": n, "k": k, "m1_us": round(r1["us"], 2), "m1_gbs": round(r1["gbs"], 1),
                         "m1_frac_of_measured_peak": round(r1["frac_of_hbm_peak"], 3), "m32_us": round(r32["us"], 2),
                         "m32_gbs": round(r32["gbs"], 1), "m32_frac_of_measured_peak": round(r32["frac_of_hbm_peak"], 3),
                         "m512_us": round(r512x["us"], 1), "m512_tflops": round(r512x["tflops"], 1),
                         "m512_fp16_operands_us": round(r512["us"], 1), "m512_fp16_operands_tflops": round(r512["tflops"], 1),
                         "paths": "m1: integer-digit GEMV; m32, m512: tcgen05 GEMM, exact-class operands (default); "
                                  "m512_fp16_operands: the same GEMM with operands rounded to fp16 (opt-in)"})
    return rows


def config_dict(cfg, n_gpus: int, mode: str) -> dict:
    return {"workload": f"{MODEL} (Llama-3-8B-shaped, L32 h4096 32q/8kv hd128 ffn14336 V128256) Q4_K_M-like GGUF blocks, "
                        f"batch-1 greedy decode after a {PROMPT}-token random prompt, fp16 paged KV (16-token pages)",
            "batch": 1, "prompt_len": PROMPT, "kv": "fp16 paged/16", "parallelism": mode if n_gpus > 1 else "single",
            "l2": "each step streams 4.6 GB of weights (>> 126 MB L2), no flush needed"}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    import torch

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    cfg, W = build_weights(dev)
    # bounded sample: at most ~4 minutes of CPU work in total (one warm-up step, up to 90 s of prompt, up to 120 s of decode)
    cpu_decode_rate(cfg, W, 1, 30.0)
    rate, done, threads, fed = cpu_decode_rate(cfg, W, args.steps, 120.0, PROMPT, 90.0)
    sample = (f"{done} decode steps (of {args.steps} requested) after {fed} of the {PROMPT} prompt tokens (prompt feeding is cut at "
              f"90 s; fewer cached keys only shorten the CPU's attention), full model, {threads} threads")
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": rate, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / rate, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(cfg, args.gpus, "replicas"),
            "cpu_baseline": {"value": rate, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": rate, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement (C++) of sapient's x86_64 path; the Rust reference cannot be built without cargo"}
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="prefill + warm-up + timed device loop only (for profiler runs)")
    ap.add_argument("--no-batch32", action="store_true", help="skip the 32-sequence decode section")
    ap.add_argument("--no-sweep", action="store_true", help="skip the operator sweep section")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    from sapient_b200 import ops
    from sapient_b200.engine import ForwardEngine

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        # stdout carries exactly one JSON line: whatever NCCL logs (NCCL_DEBUG as the launcher set it) goes to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    cfg, W = build_weights(f"cuda:{local}")
    wbytes = step_weight_bytes(cfg, W)
    # N > 1: ONE sequence, the model split over the N GPUs (tensor parallel, strong scaling)
    eng = ForwardEngine.from_weights(cfg, W, device=local, max_batch=1, max_tokens=256, tp_rank=rank, tp_size=world)
    if world > 1:
        eng.tp_connect()  # IPC handles over the default process group
    # a real (non-default) stream: CUDA events below are recorded on the stream the kernels run on
    stream = torch.cuda.Stream(device=local)
    torch.cuda.set_stream(stream)
    eng.set_stream(stream.cuda_stream)
    K, Wm = args.steps, args.warmup
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["vocab"], PROMPT).astype(np.uint32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ── value: device-resident greedy loop ──
    if args.quick:
        eng.set_large_m_gemm(1)  # profiler runs: the (untimed) prompt on the path with the fewest launches
    logits = eng.forward_logits(prompt, use_cache=False)
    eng.set_large_m_gemm(2)
    first = np.array([int(np.flatnonzero(logits == logits.max())[-1])], np.uint32)
    toks = eng.decode_greedy(first, [0], Wm)  # warm-up (captures the step graph)
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count()
    barrier()
    t_wall0 = time.perf_counter()
    ev0.record(stream)
    eng.decode_greedy(toks[-1], [0], K, fetch=False)
    ev1.record(stream)
    barrier()
    t_wall1 = time.perf_counter()
    launches = ops.launch_count() - launches0
    dev_ms = ev0.elapsed_time(ev1)
    kv_ctx_mid = PROMPT + Wm + K // 2

    if args.quick:  # launch-list / profiler runs: prefill + warm-up + timed steps only
        sampler.stop()
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": dev_ms / K, "value": K / (dev_ms / 1000.0),
                              "gpu_launches": int(launches)}), flush=True)
        eng.close()
        return

    # ── e2e: public API with host buffers, every step ──
    eng.truncate_cache(PROMPT)
    tok = int(first[0])
    if world == 1:
        # the reference-facing call: token id up, full f32 logits down, arg-max on the host
        def e2e_step(t):
            lg = eng.forward_logits(np.array([t], np.uint32), True)
            return int(lg.argmax())
        e2e_api, e2e_d2h = "ForwardEngine.forward_logits (full f32 logits to host)", cfg["vocab"] * 4
    else:
        # tensor parallel: every rank holds a vocabulary slice; the ranks exchange their arg-max candidates on the
        # device (peer stores) and each returns the global arg-max, so no logits cross PCIe or NCCL
        def e2e_step(t):
            return int(eng.decode_batch(np.array([t], np.uint32), [0], want_logits=False, want_argmax=True)[1][0])
        e2e_api, e2e_d2h = "ForwardEngine.decode_batch (token id up, global arg-max down)", 4
    for _ in range(Wm):
        tok = e2e_step(tok)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = e2e_step(tok)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    time.sleep(0.2)
    sampler.stop()
    clocks = sampler.summary(t_wall0, t_wall1)

    # ── per-family device time: each family's launches of one step replayed alone as a CUDA graph ──
    P = 20
    # (single GPU only: under tensor parallelism a subset would separate the producers of an exchange from its consumers)
    fam_ms = {f: eng.time_families(f, 1, P) for f in eng.PROFILE_FAMILIES} if world == 1 else {}
    fam_ms["all"] = eng.time_families("all", 1, P)
    gemv_ms = fam_ms.get("gemv", 0.0) * P
    gemv_n = (4 * cfg["n_layers"] + 1) * P
    eng.truncate_cache(PROMPT)

    # ── comparison arm under tensor parallelism: the same step with its sums through ncclAllReduce ──
    nccl_arm = None
    if world > 1 and os.environ.get("SAPIENT_BENCH_NCCL_ARM", "1") != "0":
        KN = min(K, 64)
        eng.tp_nccl_init()
        eng.tp_set_allreduce(True)
        t2 = eng.decode_greedy(first, [0], Wm)  # captures this arm's step graph
        barrier()
        ev0.record(stream)
        eng.decode_greedy(t2[-1], [0], KN, fetch=False)
        ev1.record(stream)
        barrier()
        tn = torch.tensor([ev0.elapsed_time(ev1)], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(tn, op=dist.ReduceOp.MAX)
        eng.tp_set_allreduce(False)
        nccl_arm = {"tokens_per_s": KN / (float(tn[0]) / 1000.0), "ms_per_step": float(tn[0]) / KN, "steps": KN,
                    "what": "the same tensor-parallel decode step with the o_proj / down_proj sums through ncclAllReduce "
                            "(partial product to scratch, all-reduce in the step graph, one add) instead of the push fused "
                            "into the GEMV epilogue"}

    # ── the other sections of the metric (extra keys of the same line) ──
    eng.close()
    peaks_now, _ = measured_peaks()
    sections = {}
    if not args.no_batch32:
        sections["batch32"] = batch32_section(cfg, W, wbytes, local, rank, world, stream, barrier, peaks_now)
    if not args.no_sweep and world == 1:
        sections["sweep"] = sweep_section()

    t = torch.tensor([dev_ms, e2e_s * 1000.0], device=f"cuda:{local}", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peaks, peak_src = measured_peaks()
        value = K / (dev_ms / 1000.0)  # one sequence whatever the GPU count
        wbytes_gpu = wbytes / world
        kv_bytes = 2 * cfg["n_layers"] * cfg["n_kv_heads"] * cfg["head_dim"] * 2 * kv_ctx_mid
        achieved = (wbytes_gpu / 1e9) / ((gemv_ms / P) / 1000.0) if gemv_ms > 0 else None  # per GPU
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_dict(cfg, world, f"tp{world}" if world > 1 else "single"),
            "e2e": {"value": K / (e2e_ms / 1000.0), "unit": "tok/s", "h2d_bytes_per_step": 12,
                    "d2h_bytes_per_step": e2e_d2h, "api": e2e_api},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "gemv_imma_kernel<1> (dequant-fused tensor-core GEMV, M=1)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "peak_source": peak_src, "unit": "GB/s",
                         "frac": (achieved / peaks["hbm_gbs"]) if achieved else None,
                         # DRAM bytes per launch: ncu read+write on the 14336x4096 Q4_K and 4096x14336 Q6_K launches is
                         # 0.999x / 1.000x their algorithmic bytes (profiles/gemv_imma_kernel_m1.md), scaled to the
                         # average launch of the step
                         "traffic": NCU_TRAFFIC_RATIO * wbytes_gpu / max(gemv_n / P, 1), "traffic_source": "ncu, scaled by bytes",
                         "algorithmic_bytes_per_step": wbytes_gpu, "launches_per_step": gemv_n / P,
                         "avg_launch_us": (1000.0 * gemv_ms / max(gemv_n, 1)) if gemv_ms > 0 else None},
            "step_roofline": {"bytes_per_step_per_gpu": (wbytes + kv_bytes) / world,
                              "ideal_ms_at_8TBs": (wbytes + kv_bytes) / world / 8e12 * 1e3,
                              "frac_of_8TBs": ((wbytes + kv_bytes) / world / 8e12 * 1e3) / (dev_ms / K),
                              "frac_of_measured_peak": ((wbytes + kv_bytes) / world / (peaks["hbm_gbs"] * 1e9) * 1e3) / (dev_ms / K)},
            "family_ms_per_step": fam_ms,
        }
        if nccl_arm:
            line["tp_allreduce_arm"] = nccl_arm
        if sections.get("batch32"):
            line["batch32"] = sections["batch32"]
        if sections.get("sweep"):
            line["sweep"] = sections["sweep"]
        if not args.no_cpu_baseline:
            rate, done, threads, fed = cpu_decode_rate(cfg, W, 8, 25.0)
            line["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": threads, "kind": "port",
                                    "sample": f"{done} decode steps after a {fed}-token prompt (not the GPU arm's {PROMPT}: the CPU "
                                              f"prefill alone would exceed the sample's time bound), full model"}
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
