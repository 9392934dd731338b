"""Synthetic inputs for the quantized decode path: block quantisers, random-bit
blocks, model weight sets in the layouts the reference's GGUF loader produces,
and a GGUF writer.

The quantisers are simple min/max quantisers of this project (not ggml's search):
both the CUDA path and any CPU checker decode the same bytes, so quantisation
quality does not enter any comparison. Everything is written with torch ops so
the same code builds tiny CPU test models and multi-GB models on a GPU.

Block layouts follow crates/sapient-core/src/dtype.rs:56-69 and the decoders in
crates/sapient-core/src/tensor.rs:378-576 of the reference.
"""
from __future__ import annotations

import numpy as np
import torch

# ggml type codes (crates/sapient-io/src/gguf.rs:88-129).
F32, F16, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 8, 12, 13, 14, 30
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210), F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q5_K: (256, 176), BF16: (1, 2)}
BPW = {Q8_0: 34 / 32, Q4_K: 144 / 256, Q6_K: 210 / 256, F32: 4.0, F16: 2.0, Q4_0: 18 / 32, Q5_K: 176 / 256, BF16: 2.0}
TYPE_NAME = {F32: "f32", F16: "f16", Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k", Q4_0: "q4_0", Q5_K: "q5_k", BF16: "bf16"}


def byte_count(dtype: int, numel: int) -> int:
    be, bb = BLOCK[dtype]
    return numel // be * bb


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """f32 [...] -> uint8 [..., 2] little-endian IEEE half."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """[..., K] f32 -> uint8 [..., K/32*34]."""
    *lead, k = w.shape
    assert k % 32 == 0
    x = w.reshape(-1, k // 32, 32).float()
    amax = x.abs().amax(dim=-1)
    d16 = (amax / 127.0).to(torch.float16)
    d = d16.float()
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(x * inv.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    out = torch.empty(x.shape[0], k // 32, 34, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = d16.contiguous().view(torch.uint8).reshape(x.shape[0], k // 32, 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.reshape(*lead, k // 32 * 34)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """[..., K] f32 -> uint8 [..., K/256*144] (f16 d, f16 dmin, 12 packed 6-bit scale/min bytes, 128 nibble bytes)."""
    *lead, k = w.shape
    assert k % 256 == 0
    x = w.reshape(-1, 8, 32).float()  # [blocks, sub, 32]
    nb = x.shape[0]
    mn = (-x.amin(dim=-1)).clamp_min(0.0)  # offset magnitude, >= 0
    scale = (x.amax(dim=-1) + mn).clamp_min(0.0) / 15.0
    d16 = (scale.amax(dim=-1) / 63.0).to(torch.float16)
    m16 = (mn.amax(dim=-1) / 63.0).to(torch.float16)
    d, dm = d16.float().unsqueeze(-1), m16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale / d), torch.zeros_like(scale)).clamp_(0, 63)
    mq = torch.where(dm > 0, torch.round(mn / dm), torch.zeros_like(mn)).clamp_(0, 63)
    eff = (d * sc).unsqueeze(-1)
    off = (dm * mq).unsqueeze(-1)
    q = torch.where(eff > 0, torch.round((x + off) / eff), torch.zeros_like(x)).clamp_(0, 15).to(torch.uint8)
    sc, mq = sc.to(torch.uint8), mq.to(torch.uint8)
    out = torch.empty(nb, 144, dtype=torch.uint8, device=w.device)
    out[:, 0:2] = d16.contiguous().view(torch.uint8).reshape(nb, 2)
    out[:, 2:4] = m16.contiguous().view(torch.uint8).reshape(nb, 2)
    out[:, 4:8] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (mq[:, 0:4] & 63) | ((mq[:, 4:8] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:8] & 0xF) | ((mq[:, 4:8] & 0xF) << 4)
    qg = q.reshape(nb, 4, 2, 32)  # group, (lo, hi), l
    out[:, 16:144] = (qg[:, :, 0, :] | (qg[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(*lead, k // 256 * 144)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    """[..., K] f32 -> uint8 [..., K/256*210] (ql[128], qh[64], i8 scales[16], f16 d)."""
    *lead, k = w.shape
    assert k % 256 == 0
    x = w.reshape(-1, 16, 16).float()  # [blocks, group, 16]
    nb = x.shape[0]
    gscale = x.abs().amax(dim=-1) / 31.0
    d16 = (gscale.amax(dim=-1) / 127.0).to(torch.float16)
    d = d16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(gscale / d), torch.zeros_like(gscale)).clamp_(-128, 127)
    eff = (d * sc).unsqueeze(-1)
    q = torch.where(eff != 0, torch.round(x / eff), torch.zeros_like(x)).clamp_(-32, 31)
    q = (q + 32).to(torch.uint8).reshape(nb, 2, 4, 32)  # half, quarter, l
    q1, q2, q3, q4 = q[:, :, 0], q[:, :, 1], q[:, :, 2], q[:, :, 3]
    out = torch.empty(nb, 210, dtype=torch.uint8, device=w.device)
    ql = torch.empty(nb, 2, 64, dtype=torch.uint8, device=w.device)
    ql[:, :, 0:32] = (q1 & 0xF) | ((q3 & 0xF) << 4)
    ql[:, :, 32:64] = (q2 & 0xF) | ((q4 & 0xF) << 4)
    out[:, 0:128] = ql.reshape(nb, 128)
    out[:, 128:192] = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).reshape(nb, 64)
    out[:, 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[:, 208:210] = d16.contiguous().view(torch.uint8).reshape(nb, 2)
    return out.reshape(*lead, k // 256 * 210)


def quantize(dtype: int, w: torch.Tensor) -> torch.Tensor:
    if dtype == Q8_0:
        return quantize_q8_0(w)
    if dtype == Q4_K:
        return quantize_q4_k(w)
    if dtype == Q6_K:
        return quantize_q6_k(w)
    if dtype == F32:
        return w.float().contiguous().view(torch.uint8).reshape(*w.shape[:-1], w.shape[-1] * 4)
    if dtype == F16:
        return w.to(torch.float16).contiguous().view(torch.uint8).reshape(*w.shape[:-1], w.shape[-1] * 2)
    if dtype == BF16:
        return w.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(*w.shape[:-1], w.shape[-1] * 2)
    raise ValueError(f"unsupported dtype {dtype}")


def random_bit_blocks(dtype: int, nblocks: int, seed: int) -> np.ndarray:
    """Random-BIT blocks: every payload byte uniformly random, so all bit paths of the
    decoders are exercised (incl. the 6-bit scale packing of Q4_K sub-blocks 4..7); the
    f16 scales are small positive normals so dequantised magnitudes stay O(0.1). Follows
    the recipe of the reference's GPU-vs-CPU block tests
    (crates/sapient-backends/wgpu/tests/resident.rs:600-640,712-740)."""
    rng = np.random.default_rng(seed)
    _, bb = BLOCK[dtype]
    out = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)

    def f16(n, lo):
        return (lo * (1.0 + rng.random(n))).astype(np.float16).view(np.uint8).reshape(n, 2)

    if dtype == Q8_0:
        out[:, 0:2] = f16(nblocks, 1e-3)
    elif dtype == Q4_K:
        out[:, 0:2] = f16(nblocks, 1e-4)
        out[:, 2:4] = f16(nblocks, 1e-4)
    elif dtype == Q6_K:
        out[:, 208:210] = f16(nblocks, 1e-5)
    elif dtype == Q4_0:
        out[:, 0:2] = f16(nblocks, 1e-2)
    elif dtype == Q5_K:
        out[:, 0:2] = f16(nblocks, 1e-4)
        out[:, 2:4] = f16(nblocks, 1e-4)
    else:
        raise ValueError(dtype)
    return out.reshape(-1)


# ── model shapes (BASELINE configs) ──────────────────────────────────────────
CONFIGS = {
    # Qwen2.5-0.5B-shaped
    "qwen05b": dict(arch="qwen2", n_layers=24, hidden=896, n_heads=14, n_kv_heads=2, head_dim=64, ffn=4864,
                    vocab=151936, norm_eps=1e-6, rope_theta=1e6, tied=True, qkv_bias=True),
    # Qwen2.5-1.5B-shaped
    "qwen15b": dict(arch="qwen2", n_layers=28, hidden=1536, n_heads=12, n_kv_heads=2, head_dim=128, ffn=8960,
                    vocab=151936, norm_eps=1e-6, rope_theta=1e6, tied=True, qkv_bias=True),
    # Phi-2-shaped
    "phi2": dict(arch="phi2", n_layers=32, hidden=2560, n_heads=32, n_kv_heads=32, head_dim=80, ffn=10240,
                 vocab=51200, norm_eps=1e-5, rope_theta=1e4, rotary_dim=32, tied=False),
    # Llama-3-8B-shaped
    "llama8b": dict(arch="llama", n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336,
                    vocab=128256, norm_eps=1e-5, rope_theta=5e5, tied=False),
    # tiny shapes for tests
    "tiny_llama": dict(arch="llama", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                       vocab=320, norm_eps=1e-5, rope_theta=1e4, tied=False),
    # splits over 2 ranks on 256-column block boundaries (o_proj K = 512, down_proj K = 1024)
    "tiny_llama_tp": dict(arch="llama", n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024,
                          vocab=320, norm_eps=1e-5, rope_theta=1e4, tied=False),
    "tiny_qwen": dict(arch="qwen2", n_layers=2, hidden=160, n_heads=5, n_kv_heads=1, head_dim=32, ffn=256,
                      vocab=200, norm_eps=1e-6, rope_theta=1e6, tied=True, qkv_bias=True),
    "tiny_phi2": dict(arch="phi2", n_layers=2, hidden=160, n_heads=4, n_kv_heads=4, head_dim=40, ffn=320,
                      vocab=96, norm_eps=1e-5, rope_theta=1e4, rotary_dim=16, tied=False),
    # widths that are multiples of 256 (the 256-column tile kernels) with Phi-2's block: LayerNorm, partial RoPE, GELU,
    # biases, head_dim 80
    "tiny_phi2_wide": dict(arch="phi2", n_layers=2, hidden=640, n_heads=8, n_kv_heads=8, head_dim=80, ffn=1280,
                           vocab=144, norm_eps=1e-5, rope_theta=1e4, rotary_dim=32, tied=False),
    # Phi-3 / Phi-4-mini block: RMSNorm + SwiGLU like Llama, q|k|v and gate|up fused in the GGUF file, grouped-query heads
    "tiny_phi3": dict(arch="phi3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                      vocab=320, norm_eps=1e-5, rope_theta=1e4, tied=False),
    # Llama block whose rows span several 256-column tiles (hidden 768 = 3 tiles, ffn 2048 = 8 tiles)
    "tiny_llama_wide": dict(arch="llama", n_layers=3, hidden=768, n_heads=6, n_kv_heads=2, head_dim=128, ffn=2048,
                            vocab=1000, norm_eps=1e-5, rope_theta=5e5, tied=False),
}


def weight_dtype(cfg: dict, role: str, layer: int, k: int) -> int:
    """"Q4_K_M-like" layout rule: K%256==0 -> Q4_K, except attn_v / ffn_down on even
    layers and token_embd / output -> Q6_K; K%256!=0 -> Q8_0 (the reference's K-quant
    kernels require k % 256 == 0). Phi-2-shaped models are Q8_0 throughout."""
    if cfg["arch"] == "phi2" or k % 256 != 0:
        return Q8_0
    if role in ("embed", "output"):
        return Q6_K
    if cfg["arch"] == "phi3" and role in ("q", "k"):
        role = "v"  # q | k | v are ONE tensor in a Phi-3 file: one format for the three
    if role in ("v", "down") and layer % 2 == 0:
        return Q6_K
    return Q4_K


def build_model(cfg: dict, seed: int, device: str = "cpu", max_ctx: int | None = None, embed_float=None) -> tuple[dict, dict]:
    """Random-init N(0, 0.02) weights quantised per block. Returns (cfg, weights) where
    weights maps HF-style names (the keys the reference's GGUF name map produces,
    crates/sapient-models/src/gguf_weights.rs:360-455) to (dtype, dims, uint8 tensor).
    embed_float: a [vocab, hidden] f32 tensor to quantise as the token embedding (and tied output head) instead of a
    fresh random one."""
    cfg = dict(cfg)
    cfg.setdefault("rotary_dim", cfg["head_dim"])
    cfg["max_ctx"] = max_ctx or cfg.get("max_ctx", 4096)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    H, Hkv, hd, hid, ffn, V = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["hidden"], cfg["ffn"], cfg["vocab"]
    W: dict = {}

    def mat(name, n, k, role, layer=0, dtype=None):
        dt = dtype if dtype is not None else weight_dtype(cfg, role, layer, k)
        # quantise in row chunks to bound temporary memory on large matrices
        rows_per = max(1, (1 << 26) // k)
        parts = []
        for r0 in range(0, n, rows_per):
            r = min(rows_per, n - r0)
            w = torch.randn(r, k, generator=g, device=device, dtype=torch.float32) * 0.02
            parts.append(quantize(dt, w))
        W[name + ".weight"] = (dt, [n, k], torch.cat(parts, 0).reshape(-1))

    def vec(name, n, center, spread):
        v = center + spread * (torch.rand(n, generator=g, device=device, dtype=torch.float32) * 2 - 1)
        W[name] = (F32, [n], v.contiguous().view(torch.uint8).reshape(-1))

    phi = cfg["arch"] == "phi2"
    if embed_float is not None:
        assert tuple(embed_float.shape) == (V, hid)
        dt = weight_dtype(cfg, "embed", 0, hid)
        rows_per = max(1, (1 << 26) // hid)
        parts = [quantize(dt, embed_float[r0:r0 + rows_per].to(device=device, dtype=torch.float32)) for r0 in range(0, V, rows_per)]
        W["model.embed_tokens.weight"] = (dt, [V, hid], torch.cat(parts, 0).reshape(-1))
    else:
        mat("model.embed_tokens", V, hid, "embed")
    for l in range(cfg["n_layers"]):
        p = f"model.layers.{l}"
        vec(p + ".input_layernorm.weight", hid, 1.0, 0.05)
        if phi:
            vec(p + ".input_layernorm.bias", hid, 0.0, 0.02)
        mat(p + ".self_attn.q_proj", H * hd, hid, "q", l)
        mat(p + ".self_attn.k_proj", Hkv * hd, hid, "k", l)
        mat(p + ".self_attn.v_proj", Hkv * hd, hid, "v", l)
        mat(p + ".self_attn.o_proj", hid, H * hd, "o", l)
        if phi or cfg.get("qkv_bias"):
            vec(p + ".self_attn.q_proj.bias", H * hd, 0.0, 0.02)
            vec(p + ".self_attn.k_proj.bias", Hkv * hd, 0.0, 0.02)
            vec(p + ".self_attn.v_proj.bias", Hkv * hd, 0.0, 0.02)
        if phi:
            vec(p + ".self_attn.o_proj.bias", hid, 0.0, 0.02)
            mat(p + ".mlp.fc1", ffn, hid, "up", l)
            vec(p + ".mlp.fc1.bias", ffn, 0.0, 0.02)
            mat(p + ".mlp.fc2", hid, ffn, "down", l)
            vec(p + ".mlp.fc2.bias", hid, 0.0, 0.02)
        else:
            vec(p + ".post_attention_layernorm.weight", hid, 1.0, 0.05)
            mat(p + ".mlp.gate_proj", ffn, hid, "gate", l)
            mat(p + ".mlp.up_proj", ffn, hid, "up", l)
            mat(p + ".mlp.down_proj", hid, ffn, "down", l)
    vec("model.norm.weight", hid, 1.0, 0.05)
    if phi:
        vec("model.norm.bias", hid, 0.0, 0.02)
    if not cfg.get("tied"):
        mat("lm_head", V, hid, "output")
    return cfg, W


def build_spec_pair(target: str = "qwen15b", draft: str = "qwen05b", seed: int = 4000, device: str = "cpu", max_ctx: int | None = None):
    """Target and draft models of the speculative-decoding configuration: both random-init from separate seeds, tied
    embeddings, and the draft's embedding / output matrix is the target's projected by a fixed random
    hidden_t -> hidden_d matrix with N(0, 1 / hidden_t) entries (the projection is applied to the target's f32
    embedding before either is quantised). Returns ((cfg_t, W_t), (cfg_d, W_d))."""
    ct, cd = CONFIGS[target], CONFIGS[draft]
    assert ct["vocab"] == cd["vocab"] and ct.get("tied") and cd.get("tied")
    g = torch.Generator(device=device)
    g.manual_seed(seed + 7)
    V, ht, hd_ = ct["vocab"], ct["hidden"], cd["hidden"]
    emb_t = torch.randn(V, ht, generator=g, device=device, dtype=torch.float32) * 0.02
    proj = torch.randn(ht, hd_, generator=g, device=device, dtype=torch.float32) / (ht ** 0.5)
    emb_d = emb_t @ proj
    t = build_model(ct, seed, device, max_ctx, embed_float=emb_t)
    d = build_model(cd, seed + 1, device, max_ctx, embed_float=emb_d)
    return t, d


def weights_to_numpy(W: dict) -> dict:
    return {k: (dt, dims, t.cpu().numpy()) for k, (dt, dims, t) in W.items()}


def model_bytes(W: dict) -> int:
    return sum(int(t.numel()) for _, _, t in W.values())


# ── GGUF export (names/dim order/permutation the reference loader expects) ────
def _gguf_name(hf: str) -> str:
    fixed = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "model.norm.bias": "output_norm.bias", "lm_head.weight": "output.weight"}
    if hf in fixed:
        return fixed[hf]
    parts = hf.split(".")
    assert parts[0] == "model" and parts[1] == "layers", hf
    l, rest, kind = parts[2], ".".join(parts[3:-1]), parts[-1]
    m = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
         "self_attn.v_proj": "attn_v", "self_attn.qkv_proj": "attn_qkv", "self_attn.o_proj": "attn_output",
         "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
         "mlp.down_proj": "ffn_down", "mlp.fc1": "ffn_up", "mlp.fc2": "ffn_down"}
    return f"blk.{l}.{m[rest]}.{kind}"


def permute_qk_rows_for_gguf(raw: np.ndarray, n_head: int, head_dim: int, row_bytes: int) -> np.ndarray:
    """Forward llama.cpp q/k row permutation: HF row h*D + a*D/2 + b is stored at GGUF
    row h*D + 2b + a (crates/sapient-models/src/gguf_weights.rs:98-141); the loader's
    un-permute must recover the HF order."""
    src = raw.reshape(n_head * head_dim, row_bytes)
    dst = np.empty_like(src)
    half = head_dim // 2
    for h in range(n_head):
        for a in range(2):
            for b in range(half):
                dst[h * head_dim + 2 * b + a] = src[h * head_dim + a * half + b]
    return dst.reshape(-1)


def write_gguf(path: str, cfg: dict, W: dict) -> None:
    """Write a GGUF v3 file the reference's loader accepts: ggml dim order [K, N],
    llama-arch q/k rows permuted, Phi-2 / Phi-3 q/k/v fused into attn_qkv, Phi-3 gate|up fused into ffn_up."""
    import gguf

    arch = cfg["arch"]
    wr = gguf.GGUFWriter(path, arch)
    wr.add_uint32(f"{arch}.vocab_size", cfg["vocab"])
    wr.add_uint32(f"{arch}.embedding_length", cfg["hidden"])
    wr.add_uint32(f"{arch}.block_count", cfg["n_layers"])
    wr.add_uint32(f"{arch}.attention.head_count", cfg["n_heads"])
    wr.add_uint32(f"{arch}.attention.head_count_kv", cfg["n_kv_heads"])
    wr.add_uint32(f"{arch}.feed_forward_length", cfg["ffn"])
    wr.add_uint32(f"{arch}.context_length", cfg["max_ctx"])
    if arch == "phi2":
        wr.add_float32(f"{arch}.attention.layer_norm_epsilon", cfg["norm_eps"])
    else:
        wr.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", cfg["norm_eps"])
    wr.add_float32(f"{arch}.rope.freq_base", cfg["rope_theta"])
    if cfg.get("rotary_dim", cfg["head_dim"]) != cfg["head_dim"]:
        wr.add_uint32(f"{arch}.rope.dimension_count", cfg["rotary_dim"])
    if cfg["head_dim"] * cfg["n_heads"] != cfg["hidden"]:
        wr.add_uint32(f"{arch}.attention.key_length", cfg["head_dim"])
    Wn = {k: (dt, dims, (t.cpu().numpy() if isinstance(t, torch.Tensor) else t)) for k, (dt, dims, t) in W.items()}
    if arch == "phi3":  # fused gate|up rows under the name of up_proj (gguf_weights.rs:322-325)
        for l in range(cfg["n_layers"]):
            p = f"model.layers.{l}.mlp."
            gate, up = Wn.pop(p + "gate_proj.weight"), Wn.pop(p + "up_proj.weight")
            assert gate[0] == up[0]
            Wn[p + "up_proj.weight"] = (gate[0], [gate[1][0] + up[1][0], gate[1][1]], np.concatenate([gate[2], up[2]]))
    if arch in ("phi2", "phi3"):  # fuse q|k|v rows (split again by split_phi_gguf_fused)
        for l in range(cfg["n_layers"]):
            p = f"model.layers.{l}.self_attn."
            for kind in (("weight", "bias") if arch == "phi2" else ("weight",)):
                parts = [Wn.pop(p + f"{x}_proj.{kind}") for x in "qkv"]
                dt = parts[0][0]
                dims = [sum(x[1][0] for x in parts)] + parts[0][1][1:]
                Wn[p + f"qkv_proj.{kind}"] = (dt, dims, np.concatenate([x[2] for x in parts]))
    qt = {F32: gguf.GGMLQuantizationType.F32, F16: gguf.GGMLQuantizationType.F16, Q8_0: gguf.GGMLQuantizationType.Q8_0,
          Q4_K: gguf.GGMLQuantizationType.Q4_K, Q6_K: gguf.GGMLQuantizationType.Q6_K}
    for name, (dt, dims, raw) in Wn.items():
        raw = np.ascontiguousarray(raw).reshape(-1)
        if arch == "llama" and name.endswith(("self_attn.q_proj.weight", "self_attn.k_proj.weight")):
            nh = cfg["n_heads"] if "q_proj" in name else cfg["n_kv_heads"]
            raw = permute_qk_rows_for_gguf(raw, nh, cfg["head_dim"], byte_count(dt, dims[1]))
        gname = _gguf_name(name)
        if dt == F32:
            arr = raw.view(np.float32).reshape(dims)
            wr.add_tensor(gname, arr)
        else:
            rb = byte_count(dt, dims[-1])
            arr = raw.reshape(dims[0], rb) if len(dims) == 2 else raw
            wr.add_tensor(gname, arr, raw_dtype=qt[dt])
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
