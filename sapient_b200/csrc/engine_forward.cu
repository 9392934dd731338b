// Forward pass of the resident engine: token table + paged-KV bookkeeping on the host,
// then the per-layer kernel sequence. Layer wiring follows
//   Llama/Qwen: crates/sapient-models/src/forward/llama.rs:400-539
//   Phi-2     : crates/sapient-models/src/forward/phi.rs:373-503
#include <algorithm>
#include <cstring>

#include "engine.h"
#include "sp_common.cuh"

namespace sp {

#define SP_TRY(expr)                  \
    do {                              \
        int _s = (expr);              \
        if (_s != SP_OK) return _s;   \
    } while (0)

// Launch `expr` (a cudaError_t) bracketed by profiling events of kernel family `fam`.
#define SP_LAUNCH(fam, expr)              \
    do {                                  \
        if (fam_mask & (1u << (fam))) {   \
            prof_begin(fam);              \
            SP_CUDA_TRY(expr);            \
            prof_end(fam);                \
        }                                 \
    } while (0)

int Engine::alloc_pages(int slot, int new_len) {
    if (!pages.grow(slot, new_len)) { set_error("KV page pool exhausted"); return SP_ERR_KV_FULL; }
    return SP_OK;
}

int Engine::sync_page_table() {
    if (pages.dirty) {
        SP_CUDA_TRY(cudaMemcpyAsync(d_page_table_, pages.table.data(), pages.table.size() * 4, cudaMemcpyHostToDevice, stream));
        pages.dirty = false;
    }
    return SP_OK;
}

// One page of one layer is a contiguous run of 2 * n_kv * 16 * head_dim halves; the layers are n_pages such runs apart.
int Engine::privatise_tail(int slot) {
    int from = 0, to = 0;
    const int r = pages.privatise_tail(slot, seq_len[slot], &from, &to);
    if (r < 0) { set_error("KV page pool exhausted"); return SP_ERR_KV_FULL; }
    if (r == 0) return SP_OK;
    const size_t run = (size_t)2 * kv_.n_kv * KV_PAGE * kv_.head_dim * sizeof(__half);
    const size_t pitch = run * (size_t)kv_.n_pages;
    const uint8_t* base = reinterpret_cast<const uint8_t*>(kv_.pool);
    SP_CUDA_TRY(cudaMemcpy2DAsync(const_cast<uint8_t*>(base) + run * (size_t)to, pitch, base + run * (size_t)from, pitch, run, (size_t)d.n_layers,
                                  cudaMemcpyDeviceToDevice, stream));
    return SP_OK;
}

int Engine::adopt_prefix(int slot, const int32_t* page_ids, int n) {
    if (slot < 0 || slot >= d.max_batch || n < 0 || (n > 0 && !page_ids)) { set_error("adopt_prefix: bad argument"); return SP_ERR_ARG; }
    if (seq_len[slot] != 0 || !pages.adopt(slot, page_ids, n)) { set_error("adopt_prefix: the slot is not empty or a page is not live"); return SP_ERR_STATE; }
    seq_len[slot] = n * KV_PAGE;
    return SP_OK;
}

int Engine::reset(int slot) {
    size_t kept;
    if (slot < 0) {
        for (int s = 0; s < d.max_batch; ++s) SP_TRY(truncate(s, 0, &kept));
        return SP_OK;
    }
    return truncate(slot, 0, &kept);
}

// truncate_cache (crates/sapient-models/src/forward/llama.rs:307-313): kept = min(n, current). Rollback is
// O(1): the page-table tail is returned to the pool, the kept pages stay where they are.
int Engine::truncate(int slot, size_t n, size_t* kept) {
    if (slot < 0 || slot >= d.max_batch) { set_error("slot out of range"); return SP_ERR_ARG; }
    const int k = (int)std::min<size_t>(n, (size_t)seq_len[slot]);
    seq_len[slot] = k;
    const int keep_pages = (k + KV_PAGE - 1) / KV_PAGE;
    pages.shrink(slot, keep_pages);
    if (kept) *kept = (size_t)k;
    return SP_OK;
}

int Engine::enqueue_layers(int T) {
    const int hid = d.hidden;
    SP_LAUNCH(F_EMBED, launch_embed(embed_->dtype, embed_->d, hid, d_ids_, T, x_, stream));
    for (int l = 0; l < d.n_layers; ++l) {
        SP_TRY(d.arch == 1 ? layer_phi(layers_[l], l, T) : layer_llama(layers_[l], l, T));
        if (trace_on) SP_TRY(tp_resolve(T));
        if (trace_on)
            SP_CUDA_TRY(cudaMemcpyAsync(trace_ + (size_t)l * d.max_tokens * hid, x_, (size_t)T * hid * 4, cudaMemcpyDeviceToDevice, stream));
    }
    trace_tokens_ = T;
    return SP_OK;
}

// lm_head over rows [r0, r0+rc) of the normalised selection sel_, plus their argmax.
int Engine::enqueue_head(int rows_from, int r0, int rc, const ImmaArgs* pre) {
    (void)rows_from;
    const int V = vocab_l_, hid = d.hidden;
    // lm_head rows beyond the vocabulary (if the table is larger) are not computed: n = V (this rank's slice under
    // tensor parallelism)
    DevTensor head = *lm_head_;
    head.dims[0] = V;
    SP_TRY(gemv(sel_ + (size_t)r0 * hid, hid, rc, hid, &head, lm_bias_, logits_, V, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                nullptr, pre));
    SP_LAUNCH(F_ARGMAX, launch_argmax(logits_, rc, V, V, d_argmax_, stream, argmax_scratch_));
    if (d.tp_size > 1) {
        if (!tp_connected_) { set_error("tensor-parallel engine used before tp_connect"); return SP_ERR_STATE; }
        SP_LAUNCH(F_ARGMAX, launch_tp_argmax(logits_, V, rc, vocab_off_, d_argmax_, d_tp_, stream));
    }
    return SP_OK;
}

int Engine::enqueue_decode_step(int T) {
    const int hid = d.hidden;
    SP_TRY(enqueue_layers(T));
    ImmaArgs ia;
    {
        DevTensor head = *lm_head_;
        head.dims[0] = vocab_l_;
        bool ringed = false;
        SP_TRY(try_ring(&ringed, T, hid, d.arch == 1 ? RING_SRC_LN : RING_SRC_RMS, x_, hid, final_w_, final_b_, &head, lm_bias_, logits_, vocab_l_));
        if (ringed) {
            SP_LAUNCH(F_ARGMAX, launch_argmax(logits_, T, vocab_l_, vocab_l_, d_argmax_, stream, argmax_scratch_));
            return SP_OK;
        }
    }
    if (lm_head_->tiled && plan_digits(T, hid, ia)) {
        SP_LAUNCH(F_NORM, launch_norm_quant(x_, hid, final_w_, final_b_, d.arch == 1, d.norm_eps, nullptr, 0, ia, stream, tp_take()));
        return enqueue_head(0, 0, T, &ia);
    }
    SP_TRY(tp_resolve(T));
    if (d.arch == 1) SP_LAUNCH(F_NORM, launch_layer_norm(x_, final_w_, final_b_, T, hid, d.norm_eps, sel_, stream));
    else SP_LAUNCH(F_NORM, launch_rms_norm(x_, final_w_, T, hid, d.norm_eps, sel_, stream));
    return enqueue_head(0, 0, T);
}

// One chunk of T <= max_tokens tokens whose (slot, pos) are already staged in p_slot_/p_pos_.
// Logits are produced for chunk rows [rows_from, T).
int Engine::run_chunk(const uint32_t* ids, const int32_t* slots, int T, int rows_from, float* logits_out,
                      uint32_t* argmax_out) {
    (void)slots;
    std::memcpy(p_ids_, ids, (size_t)T * 4);
    SP_CUDA_TRY(cudaMemcpyAsync(d_ids_, p_ids_, (size_t)T * 4, cudaMemcpyHostToDevice, stream));
    SP_CUDA_TRY(cudaMemcpyAsync(d_tok_slot_, p_slot_, (size_t)T * 4, cudaMemcpyHostToDevice, stream));
    SP_CUDA_TRY(cudaMemcpyAsync(d_tok_pos_, p_pos_, (size_t)T * 4, cudaMemcpyHostToDevice, stream));
    SP_TRY(sync_page_table());
    const int hid = d.hidden, V = vocab_l_;
    if (trace_on && !trace_) SP_CUDA_TRY(cudaMalloc((void**)&trace_, (size_t)d.n_layers * d.max_tokens * hid * 4));
    const int rows = T - rows_from;
    const bool want = rows > 0 && (logits_out || argmax_out);
    if (want && rows_from == 0 && T <= logit_rows_) {
        // decode-shaped call: the whole step is one (graph) launch
        SP_TRY(launch_decode_step(T));
        if (argmax_out) SP_CUDA_TRY(cudaMemcpyAsync(p_argmax_, d_argmax_, (size_t)T * 4, cudaMemcpyDeviceToHost, stream));
        if (logits_out) SP_CUDA_TRY(cudaMemcpyAsync(p_logits_, logits_, (size_t)T * V * 4, cudaMemcpyDeviceToHost, stream));
        SP_CUDA_TRY(cudaStreamSynchronize(stream));
        if (logits_out) std::memcpy(logits_out, p_logits_, (size_t)T * V * 4);
        if (argmax_out) std::memcpy(argmax_out, p_argmax_, (size_t)T * 4);
        SP_TRY(prof_flush());
        return device_check();
    }
    SP_TRY(enqueue_layers(T));
    SP_TRY(tp_resolve(T));
    if (want) {
        const float* src = x_ + (size_t)rows_from * hid;
        if (d.arch == 1) SP_LAUNCH(F_NORM, launch_layer_norm(src, final_w_, final_b_, rows, hid, d.norm_eps, sel_, stream));
        else SP_LAUNCH(F_NORM, launch_rms_norm(src, final_w_, rows, hid, d.norm_eps, sel_, stream));
        for (int r0 = 0; r0 < rows; r0 += logit_rows_) {
            const int rc = std::min(logit_rows_, rows - r0);
            SP_TRY(enqueue_head(rows_from, r0, rc));
            if (argmax_out) SP_CUDA_TRY(cudaMemcpyAsync(p_argmax_, d_argmax_, (size_t)rc * 4, cudaMemcpyDeviceToHost, stream));
            if (logits_out) SP_CUDA_TRY(cudaMemcpyAsync(p_logits_, logits_, (size_t)rc * V * 4, cudaMemcpyDeviceToHost, stream));
            SP_CUDA_TRY(cudaStreamSynchronize(stream));
            if (logits_out) std::memcpy(logits_out + (size_t)r0 * V, p_logits_, (size_t)rc * V * 4);
            if (argmax_out) std::memcpy(argmax_out + r0, p_argmax_, (size_t)rc * 4);
        }
    }
    SP_CUDA_TRY(cudaStreamSynchronize(stream));
    SP_TRY(prof_flush());
    return device_check();
}

int Engine::forward(const uint32_t* ids, const int32_t* slots, int64_t n, bool want_all, float* logits_out,
                    uint32_t* argmax_out) {
    if (!finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    if (!ids || !slots || n <= 0) { set_error("empty input"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_TRY(drain_async());
    // validate everything before touching any state
    std::vector<int> add(d.max_batch, 0);
    for (int64_t i = 0; i < n; ++i) {
        if (slots[i] < 0 || slots[i] >= d.max_batch) { set_error("slot out of range"); return SP_ERR_ARG; }
        if ((int64_t)ids[i] >= (int64_t)d.vocab) { set_error("token id " + std::to_string(ids[i]) + " out of vocab range"); return SP_ERR_VOCAB; }
        add[slots[i]]++;
    }
    for (int s = 0; s < d.max_batch; ++s)
        if (seq_len[s] + add[s] > d.max_ctx) { set_error("KV cache full"); return SP_ERR_KV_FULL; }
    {
        int need = 0;  // fresh pages, plus one per slot whose partly filled last page is shared (copy-on-write)
        for (int s = 0; s < d.max_batch; ++s)
            if (add[s])
                need += pages.missing(s, seq_len[s] + add[s]) +
                        ((seq_len[s] % KV_PAGE) && pages.ref[pages.page_of(s, seq_len[s] / KV_PAGE)] > 1 ? 1 : 0);
        if (need > pages.available()) { set_error("KV page pool exhausted"); return SP_ERR_KV_FULL; }
    }
    for (int s = 0; s < d.max_batch; ++s)
        if (add[s]) SP_TRY(privatise_tail(s));
    const int C = d.max_tokens;
    for (int64_t c0 = 0; c0 < n; c0 += C) {
        const int T = (int)std::min<int64_t>(C, n - c0);
        for (int i = 0; i < T; ++i) {
            const int s = slots[c0 + i];
            p_slot_[i] = s;
            p_pos_[i] = seq_len[s]++;
            SP_TRY(alloc_pages(s, seq_len[s]));
        }
        step_ctx_ = 0;
        for (int i = 0; i < T; ++i) step_ctx_ = std::max(step_ctx_, p_pos_[i] + 1);
        const bool last_chunk = c0 + T >= n;
        int rows_from;
        float* lo = nullptr;
        uint32_t* ao = nullptr;
        if (want_all) {
            rows_from = 0;
            lo = logits_out ? logits_out + (size_t)c0 * vocab_l_ : nullptr;
            ao = argmax_out ? argmax_out + c0 : nullptr;
        } else {
            rows_from = last_chunk ? T - 1 : T;
            if (last_chunk) { lo = logits_out; ao = argmax_out; }
        }
        SP_TRY(run_chunk(ids + c0, slots + c0, T, rows_from, lo, ao));
    }
    return SP_OK;
}

int Engine::debug_layer_out(int layer, float* out, size_t cap, int32_t* n_tokens) {
    if (!trace_ || layer < 0 || layer >= d.n_layers) { set_error("no trace (enable tracing before the forward)"); return SP_ERR_STATE; }
    const size_t n = (size_t)trace_tokens_ * d.hidden;
    if (cap < n) { set_error("trace buffer too small"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_CUDA_TRY(cudaMemcpy(out, trace_ + (size_t)layer * d.max_tokens * d.hidden, n * 4, cudaMemcpyDeviceToHost));
    if (n_tokens) *n_tokens = trace_tokens_;
    return SP_OK;
}

}  // namespace sp
