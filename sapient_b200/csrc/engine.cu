// Resident CUDA engine for Llama/Qwen- and Phi-2-shaped quantized decoders (host side).
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <chrono>
#include <thread>
#include <cstring>

#include "sp_common.cuh"

namespace sp {

static thread_local std::string g_err;
void set_error(const std::string& msg) { g_err = msg; }
const char* get_error() { return g_err.c_str(); }

// IEEE half <-> float on the host (round-to-nearest-even), used only at load time.
static float h2f_host(uint16_t h) { return __half2float(__ushort_as_half(h)); }
static uint16_t f2h_host(float f) { return __half_as_ushort(__float2half_rn(f)); }

// quantize_q8_0_block (crates/sapient-backends/cpu/src/kernels/quant.rs:223-235): used for the online
// F16/BF16 -> Q8_0 conversion of 2-D linears at load (crates/sapient-models/src/forward/common.rs:48-86).
static void quantize_q8_0_block_host(const float* x, uint8_t* out) {
    float max_abs = 0.0f;
    for (int i = 0; i < 32; ++i) max_abs = std::fmax(max_abs, std::fabs(x[i]));
    const float scale = max_abs / 127.0f;
    const uint16_t dh = f2h_host(scale);
    const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    out[0] = (uint8_t)(dh & 0xFF);
    out[1] = (uint8_t)(dh >> 8);
    for (int i = 0; i < 32; ++i) {
        float r = std::round(x[i] * inv);
        r = std::fmin(std::fmax(r, -127.0f), 127.0f);
        out[2 + i] = (uint8_t)(int8_t)r;
    }
}

Engine::Engine(const SpModelDesc& desc) : d(desc) {
    if (d.max_batch <= 0) d.max_batch = 1;
    if (d.max_tokens <= 0) d.max_tokens = 256;
    if (d.tp_size <= 0) d.tp_size = 1;
    if (d.rotary_dim <= 0) d.rotary_dim = d.head_dim;
    g = d;
    if (d.tp_size > 1) {  // from here on d describes this rank's shard (validated in finalize)
        d.n_heads /= d.tp_size;
        d.n_kv_heads /= d.tp_size;
        d.ffn /= d.tp_size;
    }
    seq_len.assign(d.max_batch, 0);
}

Engine::~Engine() {
    cudaSetDevice(d.device);
    if (stream) cudaStreamSynchronize(stream);
    for (auto& g : step_graphs_) cudaGraphExecDestroy(g.second);
    for (auto& r : prof_recs_) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (cudaEvent_t ev : prof_pool_) cudaEventDestroy(ev);
    if (d_tokens_) cudaFree(d_tokens_);
    for (auto& kv : tensors_) { if (kv.second.d) cudaFree(kv.second.d); if (kv.second.tiled) cudaFree(kv.second.tiled); }
    ws_.release();
    tp_nccl_release();
    tp_release();
    if (att_scratch_) cudaFree(att_scratch_);
    if (argmax_scratch_) cudaFree(argmax_scratch_);
    ring_.release();
    rows_.release();
    for (void* p : owned_) cudaFree(p);
    void* bufs[] = {kv_.pool, d_page_table_, x_, h_, qkv_, attn_, gu_, mid_, sel_, logits_, trace_, d_ids_, d_argmax_,
                    d_tok_slot_, d_tok_pos_, cos_sin_};
    for (void* p : bufs) if (p) cudaFree(p);
    void* pinned[] = {p_ids_, p_slot_, p_pos_, p_logits_, p_argmax_};
    for (void* p : pinned) if (p) cudaFreeHost(p);
    if (own_stream) cudaStreamDestroy(own_stream);
    release_staging();
}

// dst[r] = src[map(r)] for rows of row_bytes bytes (a multiple of 2): the llama q/k un-permute as a gather.
// HF row h*D + a*half + b comes from GGUF row h*D + 2b + a.
__global__ void unpermute_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t row_bytes, int head_dim) {
    const int half = head_dim / 2;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int64_t h = r / head_dim, in_head = r - h * head_dim;
        const int a = (int)(in_head / half), b = (int)(in_head - (int64_t)a * half);
        const int64_t from = h * head_dim + 2 * b + a;
        const uint16_t* s = reinterpret_cast<const uint16_t*>(src + from * row_bytes);
        uint16_t* t = reinterpret_cast<uint16_t*>(dst + r * row_bytes);
        for (int64_t i = threadIdx.x; i < row_bytes / 2; i += blockDim.x) t[i] = s[i];
    }
}

int Engine::upload_staged(uint8_t* dst, const uint8_t* src, size_t nbytes) {
    if (!load_stream_) {
        SP_CUDA_TRY(cudaStreamCreateWithFlags(&load_stream_, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            SP_CUDA_TRY(cudaMallocHost((void**)&stage_[i], STAGE_BYTES));
            SP_CUDA_TRY(cudaEventCreateWithFlags(&stage_ev_[i], cudaEventDisableTiming));
        }
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (size_t off = 0; off < nbytes; off += STAGE_BYTES) {
        const size_t n = std::min(STAGE_BYTES, nbytes - off);
        const int b = stage_next_;
        stage_next_ ^= 1;
        SP_CUDA_TRY(cudaEventSynchronize(stage_ev_[b]));  // the copy that last used this buffer has left it
        // page-cache / mmap pages -> pinned memory; one host thread moves ~10 GB/s, less than the link takes, so large
        // pieces are copied by four
        if (n >= (8u << 20)) {
            constexpr int NT = 4;
            std::thread th[NT - 1];
            const size_t per = (n / NT + 4095) & ~(size_t)4095;
            for (int i = 1; i < NT; ++i) {
                const size_t o = std::min(n, per * i), e = std::min(n, per * (i + 1));
                th[i - 1] = std::thread([=] { if (e > o) std::memcpy(stage_[b] + o, src + off + o, e - o); });
            }
            std::memcpy(stage_[b], src + off, std::min(n, per));
            for (auto& t : th) t.join();
        } else {
            std::memcpy(stage_[b], src + off, n);
        }
        SP_CUDA_TRY(cudaMemcpyAsync(dst + off, stage_[b], n, cudaMemcpyHostToDevice, load_stream_));
        SP_CUDA_TRY(cudaEventRecord(stage_ev_[b], load_stream_));
    }
    load_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    load_bytes += nbytes;
    return SP_OK;
}

void Engine::release_staging() {
    if (load_stream_) cudaStreamSynchronize(load_stream_);
    for (int i = 0; i < 2; ++i) {
        if (stage_[i]) cudaFreeHost(stage_[i]);
        if (stage_ev_[i]) cudaEventDestroy(stage_ev_[i]);
        stage_[i] = nullptr;
        stage_ev_[i] = nullptr;
    }
    if (load_stream_) cudaStreamDestroy(load_stream_);
    load_stream_ = nullptr;
}

int Engine::set_tensor(const char* name, int dtype, const int64_t* dims, int ndim, const void* bytes, size_t nbytes) {
    return set_tensor_ex(name, dtype, dims, ndim, bytes, nbytes, 0);
}

int Engine::set_tensor_ex(const char* name, int dtype, const int64_t* dims, int ndim, const void* bytes, size_t nbytes, int unpermute_heads) {
    if (!name || !dims || !bytes || ndim < 1 || ndim > 2) { set_error("set_tensor: bad argument"); return SP_ERR_ARG; }
    if (finalized) { set_error("set_tensor after finalize"); return SP_ERR_STATE; }
    {
        // Phi-3's fused `mlp.gate_up_proj` (rows 0..ffn gate, ffn..2 ffn up: forward/phi.rs:559-604) is kept as two
        // matrices: two row ranges of the caller's bytes, nothing is copied on the host
        const std::string nm(name);
        const size_t at = nm.find("mlp.gate_up_proj.weight");
        if (at != std::string::npos && at + 23 == nm.size()) {
            const int bbq = block_bytes(dtype), beq = block_elems(dtype);
            if (ndim != 2 || bbq == 0 || dims[0] != 2 * (int64_t)g.ffn || dims[1] % beq != 0 ||
                (uint64_t)nbytes != (uint64_t)dims[0] * (uint64_t)(dims[1] / beq * bbq)) {
                set_error("set_tensor: fused gate_up_proj must be [2 * ffn, hidden] with matching bytes");
                return SP_ERR_SHAPE;
            }
            const int64_t half[2] = {dims[0] / 2, dims[1]};
            const std::string base = nm.substr(0, at);
            int st = set_tensor_ex((base + "mlp.gate_proj.weight").c_str(), dtype, half, 2, bytes, nbytes / 2, 0);
            if (st != SP_OK) return st;
            return set_tensor_ex((base + "mlp.up_proj.weight").c_str(), dtype, half, 2, (const uint8_t*)bytes + nbytes / 2, nbytes / 2, 0);
        }
    }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    DevTensor t;
    t.dtype = dtype;
    t.dims.assign(dims, dims + ndim);
    const int bb = block_bytes(dtype), be = block_elems(dtype);
    if (bb == 0) { set_error(std::string("unsupported dtype for ") + name); return SP_ERR_DTYPE; }
    const int64_t inner = t.dims.back();
    if (inner % be != 0) { set_error(std::string("inner dim not a multiple of the block size: ") + name); return SP_ERR_SHAPE; }
    const int64_t want = t.numel() / be * bb;
    if ((int64_t)nbytes != want) { set_error(std::string("byte size mismatch for ") + name); return SP_ERR_SHAPE; }
    std::string nm(name);
    std::vector<uint8_t> conv, shard;
    const uint8_t* src = (const uint8_t*)bytes;
    if (d.tp_size > 1) {
        if (d.tp_size > TP_MAX_RANKS || d.tp_rank < 0 || d.tp_rank >= d.tp_size) { set_error("bad tensor-parallel rank / size"); return SP_ERR_ARG; }
        std::vector<int64_t> sd;
        bool sharded = false;
        const int st = tp_shard_tensor(nm, dtype, dims, ndim, src, d.tp_rank, d.tp_size, d.vocab, shard, sd, sharded);
        if (st != SP_OK) return st;
        if (sharded) {
            t.dims = sd;
            src = shard.data();
            nbytes = shard.size();
        }
    }
    const int64_t inner_l = t.dims.back();
    const bool skip = nm.find("norm") != std::string::npos || nm.find("bias") != std::string::npos ||
                      nm.find("embed") != std::string::npos || nm.find("lm_head") != std::string::npos;
    if (ndim == 2 && !skip && (dtype == T_F16 || dtype == T_BF16) && t.numel() >= 32 && t.numel() % 32 == 0 &&
        inner_l % 32 == 0) {
        // online Q8_0 quantisation, block by block along rows
        const int64_t n = t.numel();
        conv.resize((size_t)(n / 32 * 34));
        float tmp[32];
        const uint16_t* h = (const uint16_t*)src;
        for (int64_t b = 0; b < n / 32; ++b) {
            for (int i = 0; i < 32; ++i) {
                const uint16_t v = h[b * 32 + i];
                if (dtype == T_F16) tmp[i] = h2f_host(v);
                else { uint32_t u = (uint32_t)v << 16; std::memcpy(&tmp[i], &u, 4); }
            }
            quantize_q8_0_block_host(tmp, &conv[(size_t)(b * 34)]);
        }
        t.dtype = T_Q8_0;
        src = conv.data();
        nbytes = conv.size();
    }
    t.nbytes = nbytes;
    SP_CUDA_TRY(cudaMalloc((void**)&t.d, nbytes + 16));
    if (unpermute_heads > 0 && ndim == 2) {
        // rows arrive in the GGUF llama order: upload as they are, put them in place on the device
        const int heads_here = unpermute_heads / (d.tp_size > 1 ? d.tp_size : 1);  // a row shard keeps whole heads
        const int64_t rows = t.dims[0], rb = row_bytes(t.dtype, t.dims[1]);
        if (heads_here <= 0 || rows % heads_here != 0 || ((rows / heads_here) & 1) || (rb & 1)) {
            cudaFree(t.d);
            set_error(std::string("un-permute: rows of ") + name + " do not form whole heads");
            return SP_ERR_SHAPE;
        }
        uint8_t* tmp = nullptr;
        SP_CUDA_TRY(cudaMalloc((void**)&tmp, nbytes + 16));
        int st = upload_staged(tmp, src, nbytes);
        if (st == SP_OK) {
            unpermute_rows_kernel<<<(unsigned)std::min<int64_t>(rows, 4096), 128, 0, load_stream_>>>(tmp, t.d, rows, rb, (int)(rows / heads_here));
            if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(load_stream_) != cudaSuccess) { set_error("un-permute kernel failed"); st = SP_ERR_CUDA; }
        }
        cudaFree(tmp);
        if (st != SP_OK) { cudaFree(t.d); return st; }
    } else {
        const int st = upload_staged(t.d, src, nbytes);
        if (st != SP_OK) { cudaFree(t.d); return st; }
        // conv / shard are host temporaries of this call: the copy out of them must have been staged (it has: every byte
        // went through memcpy into pinned memory before upload_staged returned)
    }
    auto it = tensors_.find(nm);
    if (it != tensors_.end()) { cudaStreamSynchronize(load_stream_); cudaFree(it->second.d); weight_bytes -= it->second.nbytes; }
    weight_bytes += nbytes;
    tensors_[nm] = t;
    return SP_OK;
}

const DevTensor* Engine::find(const std::string& name) const {
    auto it = tensors_.find(name);
    if (it != tensors_.end()) return &it->second;
    it = tensors_.find("model." + name);
    return it == tensors_.end() ? nullptr : &it->second;
}

// Norm weights and biases as f32 device vectors (F16/BF16 sources are converted once).
const float* Engine::find_f32(const std::string& name, int64_t n) {
    const DevTensor* t = find(name);
    if (!t) return nullptr;
    if (t->numel() != n) return nullptr;
    if (t->dtype == T_F32) return (const float*)t->d;
    float* out = nullptr;
    if (cudaMalloc((void**)&out, (size_t)n * 4) != cudaSuccess) return nullptr;
    owned_.push_back(out);
    if (launch_dequant(t->dtype, t->d, 1, n, out, 0) != cudaSuccess) return nullptr;
    cudaStreamSynchronize(0);
    return out;
}

// Tile-repack every quantised matrix for the tensor-core GEMV. The raw blocks are kept only for the
// embedding table (rows are gathered from it); a tied output head therefore holds both layouts.
int Engine::repack_weights() {
    int kmax = 256;
    for (auto& kv : tensors_) {
        DevTensor& t = kv.second;
        if (t.dims.size() != 2 || t.tiled) continue;
        const int64_t n = t.dims[0], k = t.dims[1];
        kmax = std::max<int>(kmax, (int)k);
        if (!imma_supported(t.dtype, k)) continue;
        const bool is_embed = &t == embed_;
        if (is_embed && lm_head_ != embed_) continue;  // gather only
        t.tiled_bytes = imma_tiled_bytes(t.dtype, n, k);
        SP_CUDA_TRY(cudaMalloc((void**)&t.tiled, t.tiled_bytes + 16));
        SP_CUDA_TRY(launch_repack(t.dtype, t.d, n, k, t.tiled, 0));
        SP_CUDA_TRY(cudaStreamSynchronize(0));
        weight_bytes += t.tiled_bytes;
        if (!is_embed) {
            cudaFree(t.d);
            t.d = nullptr;
            weight_bytes -= t.nbytes;
        }
    }
    SP_CUDA_TRY(ws_.alloc(kmax));
    if (d.max_tokens >= TC5_MIN_M) SP_CUDA_TRY(ws_.ensure_xh((size_t)2 * d.max_tokens * kmax));  // x 2: leading parts + remainders of the exact mode
    {
        // tile rows of the widest launch: q|k|v, gate|up (two segments), lm_head
        const int64_t widest = std::max<int64_t>({(int64_t)d.vocab, 2 * (int64_t)d.ffn, (int64_t)(d.n_heads + 2 * d.n_kv_heads) * d.head_dim, (int64_t)d.hidden});
        SP_CUDA_TRY(ring_device_init());
        SP_CUDA_TRY(ring_.alloc((int)(widest / 16 + 8)));
    }
    if (d.max_tokens > imma_rows_per_pass()) SP_CUDA_TRY(rows_.alloc());
    return SP_OK;
}

int Engine::finalize() {
    if (finalized) return SP_OK;
    SP_CUDA_TRY(cudaSetDevice(d.device));
    if (load_stream_) SP_CUDA_TRY(cudaStreamSynchronize(load_stream_));  // every weight has landed
    release_staging();
    if (d.tp_size > 1) {
        if (d.arch != 0) { set_error("tensor parallelism covers the Llama/Qwen block only"); return SP_ERR_ARG; }
        if (g.n_heads % d.tp_size || g.n_kv_heads % d.tp_size || g.ffn % d.tp_size || g.vocab % d.tp_size ||
            (g.vocab / d.tp_size) % 16 != 0) {
            set_error("tensor parallel: heads, kv heads, ffn and vocab / 16 must divide by the rank count");
            return SP_ERR_SHAPE;
        }
        if (d.max_tokens > 0 && std::min<int>(32, d.max_tokens) > TP_ARGMAX_ROWS) { set_error("internal: logit rows"); return SP_ERR_STATE; }
    }
    vocab_l_ = d.vocab / d.tp_size;
    vocab_off_ = d.tp_rank * vocab_l_;
    if (d.n_layers <= 0 || d.hidden <= 0 || d.n_heads <= 0 || d.n_kv_heads <= 0 || d.head_dim <= 0 || d.vocab <= 0 ||
        d.max_ctx <= 0 || d.n_heads % d.n_kv_heads != 0 || d.head_dim % 2 != 0 || d.head_dim > 256 ||
        d.rotary_dim % 2 != 0 || d.rotary_dim > d.head_dim || d.hidden % 4 != 0 || d.ffn % 4 != 0) {
        set_error("finalize: invalid model description");
        return SP_ERR_ARG;
    }
    const int H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim, hid = d.hidden;
    auto need = [&](const std::string& nm, int64_t n, int64_t k) -> const DevTensor* {
        const DevTensor* t = find(nm);
        if (!t) { set_error("missing weight '" + nm + "'"); return nullptr; }
        if (t->dims.size() != 2 || t->dims[0] != n || t->dims[1] != k) {
            set_error("shape mismatch for '" + nm + "'");
            return nullptr;
        }
        return t;
    };
    embed_ = find("model.embed_tokens.weight");
    if (!embed_ || embed_->dims.size() != 2 || embed_->dims[0] < d.vocab || embed_->dims[1] != hid) {
        set_error("missing or mis-shaped embedding weights (model.embed_tokens.weight)");
        return SP_ERR_STATE;
    }
    lm_head_ = find("lm_head.weight");  // tied fallback: crates/sapient-models/src/weights.rs:88-109
    if (!lm_head_) lm_head_ = embed_;
    if (d.tp_size > 1 && lm_head_ == embed_) { set_error("tensor parallel: tied output head is not supported"); return SP_ERR_ARG; }
    if (lm_head_->dims.size() != 2 || lm_head_->dims[1] != hid || lm_head_->dims[0] < vocab_l_) {
        set_error("mis-shaped lm_head.weight");
        return SP_ERR_STATE;
    }
    const bool phi = d.arch == 1;
    layers_.resize(d.n_layers);
    for (int l = 0; l < d.n_layers; ++l) {
        LayerW& w = layers_[l];
        const std::string p = "model.layers." + std::to_string(l) + ".";
        w.n1w = find_f32(p + "input_layernorm.weight", hid);
        w.n1b = find_f32(p + "input_layernorm.bias", hid);
        if (!w.n1w) { set_error("missing " + p + "input_layernorm.weight"); return SP_ERR_STATE; }
        if (!(w.q = need(p + "self_attn.q_proj.weight", (int64_t)H * hd, hid))) return SP_ERR_STATE;
        if (!(w.k = need(p + "self_attn.k_proj.weight", (int64_t)Hkv * hd, hid))) return SP_ERR_STATE;
        if (!(w.v = need(p + "self_attn.v_proj.weight", (int64_t)Hkv * hd, hid))) return SP_ERR_STATE;
        const std::string oname = find(p + "self_attn.dense.weight") ? "self_attn.dense" : "self_attn.o_proj";
        if (!(w.o = need(p + oname + ".weight", hid, (int64_t)H * hd))) return SP_ERR_STATE;
        w.qb = find_f32(p + "self_attn.q_proj.bias", (int64_t)H * hd);
        w.kb = find_f32(p + "self_attn.k_proj.bias", (int64_t)Hkv * hd);
        w.vb = find_f32(p + "self_attn.v_proj.bias", (int64_t)Hkv * hd);
        w.ob = find_f32(p + oname + ".bias", hid);
        if (phi) {
            if (!(w.up = need(p + "mlp.fc1.weight", d.ffn, hid))) return SP_ERR_STATE;
            if (!(w.down = need(p + "mlp.fc2.weight", hid, d.ffn))) return SP_ERR_STATE;
            w.upb = find_f32(p + "mlp.fc1.bias", d.ffn);
            w.downb = find_f32(p + "mlp.fc2.bias", hid);
        } else {
            w.n2w = find_f32(p + "post_attention_layernorm.weight", hid);
            if (!w.n2w) { set_error("missing " + p + "post_attention_layernorm.weight"); return SP_ERR_STATE; }
            if (!(w.gate = need(p + "mlp.gate_proj.weight", d.ffn, hid))) return SP_ERR_STATE;
            if (!(w.up = need(p + "mlp.up_proj.weight", d.ffn, hid))) return SP_ERR_STATE;
            if (!(w.down = need(p + "mlp.down_proj.weight", hid, d.ffn))) return SP_ERR_STATE;
        }
    }
    {
        const int st = repack_weights();
        if (st != SP_OK) return st;
    }
    // KV pages
    const int pages_per_seq = (d.max_ctx + KV_PAGE - 1) / KV_PAGE;
    int64_t n_pages = d.kv_pages > 0 ? d.kv_pages : (int64_t)d.max_batch * pages_per_seq;
    kv_.n_pages = (int)n_pages;
    kv_.n_kv = Hkv;
    kv_.head_dim = hd;
    kv_.max_pages = pages_per_seq;
    kv_bytes = (uint64_t)d.n_layers * n_pages * 2 * Hkv * KV_PAGE * hd * sizeof(__half);
    SP_CUDA_TRY(cudaMalloc((void**)&kv_.pool, kv_bytes));
    SP_CUDA_TRY(cudaMalloc((void**)&d_page_table_, (size_t)d.max_batch * pages_per_seq * 4));
    SP_CUDA_TRY(cudaMemset(d_page_table_, 0, (size_t)d.max_batch * pages_per_seq * 4));
    kv_.page_table = d_page_table_;
    pages.init(d.max_batch, pages_per_seq, (int)n_pages);
    // activations
    const size_t T = (size_t)d.max_tokens;
    const size_t qkv_ld = (size_t)(H + 2 * Hkv) * hd;
    SP_CUDA_TRY(cudaMalloc((void**)&x_, T * hid * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&h_, T * hid * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&qkv_, T * qkv_ld * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&attn_, T * (size_t)H * hd * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&gu_, T * (size_t)d.ffn * 2 * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&mid_, T * (size_t)d.ffn * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&sel_, T * hid * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&att_scratch_, attention_scratch_floats(ATT_SPLIT_TOKENS, H, ATT_SPLITS, hd) * 4));
    logit_rows_ = std::min<int>(32, d.max_tokens);
    SP_CUDA_TRY(cudaMalloc((void**)&logits_, (size_t)logit_rows_ * vocab_l_ * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&d_ids_, T * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&d_argmax_, T * 4));
    SP_CUDA_TRY(cudaMalloc(&argmax_scratch_, argmax_scratch_bytes()));
    SP_CUDA_TRY(cudaMemset(argmax_scratch_, 0, argmax_scratch_bytes()));
    SP_CUDA_TRY(cudaMalloc((void**)&d_tok_slot_, T * 4));
    SP_CUDA_TRY(cudaMalloc((void**)&d_tok_pos_, T * 4));
    SP_CUDA_TRY(cudaMallocHost((void**)&p_ids_, T * 4));
    SP_CUDA_TRY(cudaMallocHost((void**)&p_slot_, T * 4));
    SP_CUDA_TRY(cudaMallocHost((void**)&p_pos_, T * 4));
    SP_CUDA_TRY(cudaMallocHost((void**)&p_logits_, (size_t)logit_rows_ * vocab_l_ * 4));
    {
        const int st = tp_alloc();
        if (st != SP_OK) return st;
    }
    SP_CUDA_TRY(cudaMallocHost((void**)&p_argmax_, T * 4));
    // RoPE table: theta = pos / base^(2i/rotary_dim) in f32, as crates/sapient-backends/cpu/src/kernels/rope.rs:40-43,118-121.
    const int half = d.rotary_dim / 2;
    std::vector<float2> cs((size_t)d.max_ctx * half);
    for (int pos = 0; pos < d.max_ctx; ++pos)
        for (int i = 0; i < half; ++i) {
            const float freq = ((float)pos / 1.0f) / powf(d.rope_theta, 2.0f * (float)i / (float)d.rotary_dim);
            cs[(size_t)pos * half + i] = make_float2(cosf(freq), sinf(freq));
        }
    SP_CUDA_TRY(cudaMalloc((void**)&cos_sin_, std::max<size_t>(cs.size(), 1) * sizeof(float2)));
    SP_CUDA_TRY(cudaMemcpy(cos_sin_, cs.data(), cs.size() * sizeof(float2), cudaMemcpyHostToDevice));
    // Final norm: `final_layernorm` else `norm` (crates/sapient-models/src/forward/phi.rs:351-360).
    const std::string fn = find("model.final_layernorm.weight") ? "model.final_layernorm" : "model.norm";
    final_w_ = find_f32(fn + ".weight", hid);
    final_b_ = phi ? find_f32(fn + ".bias", hid) : nullptr;
    if (!final_w_) { set_error("missing final norm weight"); return SP_ERR_STATE; }
    lm_bias_ = phi ? find_f32("lm_head.bias", lm_head_->dims[0]) : nullptr;
    SP_CUDA_TRY(cudaStreamCreateWithFlags(&own_stream, cudaStreamNonBlocking));
    stream = own_stream;
    SP_CUDA_TRY(cudaDeviceSynchronize());
    finalized = true;
    return SP_OK;
}

}  // namespace sp
