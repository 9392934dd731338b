// Minimal GGUF reader and the load-time transforms that turn a GGUF file into the
// HF-named weight map the engine consumes. Restates, for the decoder families on
// this path:
//   header / tensor infos   crates/sapient-io/src/gguf.rs:517-578 (magic, v1-3, alignment)
//   metadata -> model desc  crates/sapient-hub/src/model_info.rs:234-352
//   name map + dim flip     crates/sapient-models/src/gguf_weights.rs:61-96,360-455
//   llama q/k un-permute    crates/sapient-models/src/gguf_weights.rs:114-154 (llama/mistral only)
//   Phi qkv split / renames crates/sapient-models/src/gguf_weights.rs:273-330
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "engine.h"
#include "sp_common.cuh"

namespace {

using sp::set_error;

struct Reader {
    const uint8_t* p;
    size_t n, pos = 0;
    bool ok = true;
    bool take(void* dst, size_t k) {
        if (!ok || pos + k > n) { ok = false; return false; }
        std::memcpy(dst, p + pos, k);
        pos += k;
        return true;
    }
    uint32_t u32() { uint32_t v = 0; take(&v, 4); return v; }
    uint64_t u64() { uint64_t v = 0; take(&v, 8); return v; }
    std::string str() {
        const uint64_t len = u64();
        if (!ok || len > n - pos) { ok = false; return {}; }
        std::string s((const char*)p + pos, (size_t)len);
        pos += (size_t)len;
        return s;
    }
};

struct MetaVal {
    int type = -1;
    double num = 0;       // every scalar numeric type, widened
    std::string s;
    uint64_t arr_len = 0; // arrays are skipped, only their length is kept
};

// value type codes: crates/sapient-io/src/gguf.rs:789-831
bool read_value(Reader& r, int type, MetaVal& v, bool top) {
    v.type = type;
    switch (type) {
        case 0: { uint8_t x = 0; r.take(&x, 1); v.num = x; break; }
        case 1: { int8_t x = 0; r.take(&x, 1); v.num = x; break; }
        case 2: { uint16_t x = 0; r.take(&x, 2); v.num = x; break; }
        case 3: { int16_t x = 0; r.take(&x, 2); v.num = x; break; }
        case 4: { uint32_t x = 0; r.take(&x, 4); v.num = x; break; }
        case 5: { int32_t x = 0; r.take(&x, 4); v.num = x; break; }
        case 6: { float x = 0; r.take(&x, 4); v.num = x; break; }
        case 7: { uint8_t x = 0; r.take(&x, 1); v.num = x; break; }
        case 8: v.s = r.str(); break;
        case 10: { uint64_t x = 0; r.take(&x, 8); v.num = (double)x; break; }
        case 11: { int64_t x = 0; r.take(&x, 8); v.num = (double)x; break; }
        case 12: { double x = 0; r.take(&x, 8); v.num = x; break; }
        case 9: {
            if (!top) { r.ok = false; return false; }
            const int et = (int)r.u32();
            const uint64_t cnt = r.u64();
            v.arr_len = cnt;
            MetaVal tmp;
            for (uint64_t i = 0; i < cnt && r.ok; ++i) read_value(r, et, tmp, false);
            break;
        }
        default: r.ok = false;
    }
    return r.ok;
}

struct TInfo {
    std::string name;
    std::vector<int64_t> dims;  // ggml order: dims[0] is the innermost (in) dimension
    int type = 0;
    uint64_t offset = 0;
};

// map_gguf_tensor_name / map_blk_tensor for dense decoder tensors.
bool map_name(const std::string& g, std::string* hf) {
    if (g == "token_embd.weight" || g == "tok_embeddings.weight") { *hf = "model.embed_tokens.weight"; return true; }
    if (g == "output_norm.weight" || g == "norm.weight") { *hf = "model.norm.weight"; return true; }
    if (g == "output.weight" || g == "lm_head.weight") { *hf = "lm_head.weight"; return true; }
    if (g.rfind("model.", 0) == 0) { *hf = g; return true; }
    if (g.rfind("blk.", 0) != 0) return false;
    const size_t dot = g.find('.', 4);
    if (dot == std::string::npos) return false;
    const std::string layer = g.substr(4, dot - 4);
    if (layer.empty() || layer.find_first_not_of("0123456789") != std::string::npos) return false;
    std::string comp = g.substr(dot + 1), kind;
    auto ends = [&](const char* suf) { const size_t L = std::strlen(suf); return comp.size() > L && comp.compare(comp.size() - L, L, suf) == 0; };
    if (ends(".weight")) { kind = "weight"; comp.resize(comp.size() - 7); }
    else if (ends(".bias")) { kind = "bias"; comp.resize(comp.size() - 5); }
    else return false;
    static const std::map<std::string, std::string> m = {
        {"attn_norm", "input_layernorm"}, {"attn_q", "self_attn.q_proj"}, {"attn_k", "self_attn.k_proj"},
        {"attn_v", "self_attn.v_proj"}, {"attn_qkv", "self_attn.qkv_proj"}, {"attn_output", "self_attn.o_proj"},
        {"ffn_norm", "post_attention_layernorm"}, {"post_attention_norm", "post_attention_layernorm"},
        {"ffn_gate", "mlp.gate_proj"}, {"ffn_up", "mlp.up_proj"}, {"ffn_down", "mlp.down_proj"}};
    auto it = m.find(comp);
    if (it == m.end()) return false;
    *hf = "model.layers." + layer + "." + it->second + "." + kind;
    return true;
}

struct HostTensor {
    int dtype;
    std::vector<int64_t> dims;  // HF order [out, in] / [n]
    const uint8_t* data;        // inside the file mapping
    size_t nbytes;
    int unpermute_heads = 0;    // > 0: llama-order q / k rows, put in place on the device after the upload
};

}  // namespace

int sp_engine_from_gguf_impl(const char* path, int device, int max_ctx, int max_batch, sp::Engine** out) {
    // The file is mapped, not read: tensor bytes go from the page cache straight into the engine's pinned staging
    // buffers (the reference maps its GGUF files as well, crates/sapient-models/src/forward/mod.rs:223-240).
    struct Mapping {
        const uint8_t* p = nullptr;
        size_t n = 0;
        int fd = -1;
        ~Mapping() {
            if (p) munmap((void*)p, n);
            if (fd >= 0) close(fd);
        }
        const uint8_t* data() const { return p; }
        size_t size() const { return n; }
    } buf;
    buf.fd = open(path, O_RDONLY);
    if (buf.fd < 0) { set_error(std::string("cannot open ") + path); return SP_ERR_IO; }
    struct stat sb;
    if (fstat(buf.fd, &sb) != 0 || sb.st_size < 24) { set_error("GGUF file truncated"); return SP_ERR_IO; }
    buf.n = (size_t)sb.st_size;
    void* mp = mmap(nullptr, buf.n, PROT_READ, MAP_PRIVATE, buf.fd, 0);
    if (mp == MAP_FAILED) { buf.n = 0; set_error(std::string("cannot map ") + path); return SP_ERR_IO; }
    buf.p = (const uint8_t*)mp;
    madvise(mp, buf.n, MADV_SEQUENTIAL);

    Reader r{buf.data(), buf.size()};
    if (r.u32() != 0x46554747u) { set_error("bad GGUF magic"); return SP_ERR_IO; }
    const uint32_t version = r.u32();
    if (version < 1 || version > 3) { set_error("unsupported GGUF version " + std::to_string(version) + " (expected 1-3)"); return SP_ERR_IO; }
    const uint64_t tensor_count = r.u64(), kv_count = r.u64();
    if (tensor_count > (1u << 24) || kv_count > (1u << 24)) { set_error("implausible GGUF counts"); return SP_ERR_IO; }
    std::map<std::string, MetaVal> meta;
    for (uint64_t i = 0; i < kv_count && r.ok; ++i) {
        std::string key = r.str();
        const int type = (int)r.u32();
        MetaVal v;
        if (!read_value(r, type, v, true)) break;
        meta[key] = v;
    }
    std::vector<TInfo> infos;
    for (uint64_t i = 0; i < tensor_count && r.ok; ++i) {
        TInfo t;
        t.name = r.str();
        const uint32_t nd = r.u32();
        if (nd > 4) { r.ok = false; break; }
        for (uint32_t k = 0; k < nd; ++k) t.dims.push_back((int64_t)r.u64());
        t.type = (int)r.u32();
        t.offset = r.u64();
        infos.push_back(t);
    }
    if (!r.ok) { set_error("GGUF header truncated or malformed"); return SP_ERR_IO; }
    uint64_t alignment = 32;
    if (meta.count("general.alignment")) {
        const double a = meta["general.alignment"].num;
        // a power of two of sane size: anything else could wrap the offset arithmetic below
        if (!(a >= 1 && a <= 65536) || ((uint64_t)a & ((uint64_t)a - 1)) != 0 || (double)(uint64_t)a != a) {
            set_error("GGUF general.alignment must be a power of two in 1..65536");
            return SP_ERR_IO;
        }
        alignment = (uint64_t)a;
    }
    const uint64_t data_start64 = ((uint64_t)r.pos + alignment - 1) / alignment * alignment;
    if (data_start64 > buf.size()) { set_error("GGUF data section starts past the end of the file"); return SP_ERR_IO; }
    const size_t data_start = (size_t)data_start64;

    // ── metadata -> description ──
    const std::string arch = meta.count("general.architecture") ? meta["general.architecture"].s : "llama";
    auto num = [&](const std::string& key, double dflt) { auto it = meta.find(arch + "." + key); return it == meta.end() ? dflt : it->second.num; };
    auto has = [&](const std::string& key) { return meta.count(arch + "." + key) != 0; };
    SpModelDesc d{};
    const bool is_phi = arch == "phi" || arch == "phi2";
    // Phi-3 / 3.5 / 4-mini: PhiForward's sequential block — RMSNorm, fused q|k|v, fused gate|up SwiGLU
    // (crates/sapient-models/src/forward/phi.rs:391-503,559-604) — which is the Llama block once the fused tensors are cut
    const bool is_phi3 = arch == "phi3";
    const bool is_llama_family = is_phi3 || arch == "llama" || arch == "mistral" || arch == "qwen2" || arch == "qwen3" || arch == "idefics3";
    if (!is_phi && !is_llama_family) { set_error("architecture '" + arch + "' is not supported by the CUDA engine"); return SP_ERR_DTYPE; }
    if (num("expert_count", 0) > 0) { set_error("MoE models are not supported by the CUDA engine"); return SP_ERR_DTYPE; }
    d.arch = is_phi ? 1 : 0;
    double vocab = 32000;
    if (has("vocab_size")) vocab = num("vocab_size", 32000);
    else if (meta.count("tokenizer.ggml.tokens")) vocab = (double)meta["tokenizer.ggml.tokens"].arr_len;
    d.vocab = (int32_t)vocab;
    d.hidden = (int32_t)num("embedding_length", 4096);
    d.n_layers = (int32_t)num("block_count", 32) - (int32_t)num("nextn_predict_layers", 0);
    d.n_heads = (int32_t)num("attention.head_count", 32);
    d.n_kv_heads = (int32_t)num("attention.head_count_kv", d.n_heads);
    d.ffn = (int32_t)num("feed_forward_length", 11008);
    const int ctx_file = (int)num("context_length", 4096);
    d.norm_eps = (float)(has("attention.layer_norm_rms_epsilon") ? num("attention.layer_norm_rms_epsilon", 1e-5)
                                                                 : num("attention.layer_norm_epsilon", 1e-5));
    d.rope_theta = (float)num("rope.freq_base", 10000.0);
    d.head_dim = has("attention.key_length") ? (int32_t)num("attention.key_length", 0) : d.hidden / std::max(1, d.n_heads);
    // partial rotary factor = rope.dimension_count / head_dim; rotary_dim rule of each forward engine
    // (llama.rs:470-472: round(hd*pf) & !1; phi.rs:388-389: round(pf*hd).clamp(2, hd)).
    double pf = has("rope.dimension_count") ? num("rope.dimension_count", 0) / (double)d.head_dim : 1.0;
    if (is_phi || is_phi3) {
        long rd = std::lround(pf * (double)d.head_dim);
        d.rotary_dim = (int32_t)std::min<long>(std::max<long>(rd, 2), d.head_dim);
    } else {
        d.rotary_dim = pf < 1.0 ? (int32_t)(std::lround((double)d.head_dim * pf) & ~1L) : d.head_dim;
    }
    // kv_cache_ctx (crates/sapient-models/src/forward/common.rs:25-37): min(model max, 8192) unless overridden
    d.max_ctx = max_ctx > 0 ? std::min(max_ctx, ctx_file) : std::min(ctx_file, 8192);
    if (d.max_ctx < 1) d.max_ctx = 1;
    d.max_batch = max_batch > 0 ? max_batch : 1;
    d.max_tokens = 256;
    d.device = device;
    d.tp_rank = 0;
    d.tp_size = 1;

    // ── tensors -> HF-named map ──
    std::map<std::string, HostTensor> W;
    for (const TInfo& t : infos) {
        std::string hf;
        if (!map_name(t.name, &hf)) continue;  // unknown tensors are skipped, as the reference does
        const int bb = sp::block_bytes(t.type), be = sp::block_elems(t.type);
        if (bb == 0) { set_error("tensor '" + t.name + "' has unsupported ggml type " + std::to_string(t.type)); return SP_ERR_DTYPE; }
        // dims and offset are raw 64-bit words of a downloaded file: every product and sum is checked before use
        if (t.dims.empty()) { set_error("tensor '" + t.name + "' has no dimensions"); return SP_ERR_SHAPE; }
        uint64_t numel = 1;
        bool bad = false;
        for (auto v : t.dims) {
            if (v <= 0) { bad = true; break; }
            if (numel > (uint64_t)INT64_MAX / (uint64_t)v) { bad = true; break; }
            numel *= (uint64_t)v;
        }
        if (bad) { set_error("tensor '" + t.name + "' has a non-positive or overflowing shape"); return SP_ERR_SHAPE; }
        if (t.dims[0] % be != 0) { set_error("tensor '" + t.name + "' inner dim is not a multiple of its block size"); return SP_ERR_SHAPE; }
        const uint64_t nblocks = numel / (uint64_t)be;
        const uint64_t avail = (uint64_t)buf.size() - data_start;
        if (t.offset > avail || nblocks > (avail - t.offset) / (uint64_t)bb) {
            set_error("tensor '" + t.name + "' data out of file bounds");
            return SP_ERR_IO;
        }
        const size_t nbytes = (size_t)(nblocks * (uint64_t)bb);
        HostTensor h;
        h.dtype = t.type;
        h.data = buf.data() + data_start + t.offset;
        h.nbytes = nbytes;
        const bool is_w = hf.size() > 7 && hf.compare(hf.size() - 7, 7, ".weight") == 0;
        if (is_w && t.dims.size() == 2) h.dims = {t.dims[1], t.dims[0]};  // ggml [in, out] -> HF [out, in]; bytes untouched
        else h.dims = t.dims;
        if (W.count(hf)) { set_error("duplicate mapped weight key '" + hf + "'"); return SP_ERR_IO; }
        W[hf] = std::move(h);
    }
    if (!W.count("model.embed_tokens.weight")) { set_error("GGUF file missing token embedding weights (token_embd.weight)"); return SP_ERR_STATE; }

    if (arch == "llama" || arch == "mistral" || arch == "idefics3") {
        for (auto& kv : W) {
            int nh = 0;
            const std::string& nm = kv.first;
            auto ends = [&](const char* suf) { const size_t L = std::strlen(suf); return nm.size() >= L && nm.compare(nm.size() - L, L, suf) == 0; };
            if (ends("self_attn.q_proj.weight")) nh = d.n_heads;
            else if (ends("self_attn.k_proj.weight")) nh = d.n_kv_heads;
            if (!nh) continue;
            HostTensor& h = kv.second;
            const int hd = d.head_dim;
            if (h.dims.size() != 2 || hd < 2 || hd % 2 != 0 || (int64_t)nh * hd != h.dims[0]) continue;  // left as is
            h.unpermute_heads = nh;
        }
    }
    if (is_phi || is_phi3) {
        const int64_t q_rows = (int64_t)d.n_heads * d.head_dim, kv_rows = (int64_t)d.n_kv_heads * d.head_dim;
        std::vector<std::string> fused;
        for (auto& kv : W) if (kv.first.find("self_attn.qkv_proj.") != std::string::npos) fused.push_back(kv.first);
        for (const std::string& key : fused) {
            HostTensor t = std::move(W[key]);
            W.erase(key);
            const size_t at = key.find("qkv_proj.");
            const std::string base = key.substr(0, at), suffix = key.substr(at + 9);
            if (t.dims[0] != q_rows + 2 * kv_rows) { set_error("Phi qkv split for '" + key + "': unexpected row count"); return SP_ERR_SHAPE; }
            // a 1-D tensor (bias) splits by elements: only unquantised types can be cut at any element
            if (t.dims.size() != 2 && sp::block_elems(t.dtype) != 1) { set_error("Phi qkv split for '" + key + "': quantised 1-D tensor"); return SP_ERR_SHAPE; }
            const int64_t rb = t.dims.size() == 2 ? sp::row_bytes(t.dtype, t.dims[1]) : sp::block_bytes(t.dtype);
            if ((uint64_t)t.dims[0] * (uint64_t)rb != (uint64_t)t.nbytes) { set_error("Phi qkv split for '" + key + "': byte count does not match the shape"); return SP_ERR_SHAPE; }
            const int64_t starts[3] = {0, q_rows, q_rows + kv_rows}, rows[3] = {q_rows, kv_rows, kv_rows};
            const char* nm[3] = {"q_proj.", "k_proj.", "v_proj."};
            for (int i = 0; i < 3; ++i) {
                HostTensor s;
                s.dtype = t.dtype;
                s.dims = t.dims;
                s.dims[0] = rows[i];
                s.data = t.data + starts[i] * rb;  // a row range of the same mapped bytes: nothing is copied on the host
                s.nbytes = (size_t)(rows[i] * rb);
                W[base + nm[i] + suffix] = std::move(s);
            }
        }
        // Phi-3: `ffn_up` holds the fused gate|up rows (gguf_weights.rs:322-325); the engine cuts it at set_tensor
        std::vector<std::pair<std::string, std::string>> ren;
        if (is_phi3) {
            for (auto& kv : W) {
                size_t at;
                if ((at = kv.first.find("mlp.up_proj.")) != std::string::npos) ren.push_back({kv.first, kv.first.substr(0, at) + "mlp.gate_up_proj." + kv.first.substr(at + 12)});
            }
        } else
        for (auto& kv : W) {
            size_t at;
            if ((at = kv.first.find("mlp.up_proj.")) != std::string::npos) ren.push_back({kv.first, kv.first.substr(0, at) + "mlp.fc1." + kv.first.substr(at + 12)});
            else if ((at = kv.first.find("mlp.down_proj.")) != std::string::npos) ren.push_back({kv.first, kv.first.substr(0, at) + "mlp.fc2." + kv.first.substr(at + 14)});
        }
        for (auto& pr : ren) { W[pr.second] = std::move(W[pr.first]); W.erase(pr.first); }
    }

    sp::Engine* eng = new sp::Engine(d);
    for (auto& kv : W) {
        HostTensor& h = kv.second;
        int st = eng->set_tensor_ex(kv.first.c_str(), h.dtype, h.dims.data(), (int)h.dims.size(), h.data, h.nbytes, h.unpermute_heads);
        if (st != SP_OK) { delete eng; return st; }
    }
    int st = eng->finalize();
    if (st != SP_OK) { delete eng; return st; }
    *out = eng;
    return SP_OK;
}
