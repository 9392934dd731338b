// Decode-step CUDA graphs, the device-resident greedy loop and per-family profiling.
//
// A decode step launches ~9 kernels per layer; at batch 1 each lasts a few
// microseconds, so the step is captured once per token count into a CUDA graph and
// replayed (the reference's CPU engine pays a thread-pool dispatch per matmul instead,
// crates/sapient-backends/cpu/src/kernels/matmul.rs:486-534). All kernel arguments are
// fixed device buffers; positions, slots, token ids and the page table are read from
// device memory, so one graph serves every step.
#include <algorithm>
#include <cstring>

#include "engine.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

#define SP_TRY(expr)                  \
    do {                              \
        int _s = (expr);              \
        if (_s != SP_OK) return _s;   \
    } while (0)

// After a greedy step: the argmax becomes the next input token, positions advance, the token is logged.
__global__ void advance_greedy_kernel(const uint32_t* __restrict__ argmax, uint32_t* __restrict__ ids,
                                      int32_t* __restrict__ pos, uint32_t* __restrict__ log, int b) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < b) {
        const uint32_t t = argmax[i];
        ids[i] = t;
        pos[i] += 1;
        log[i] = t;
    }
}

void Engine::prof_begin(int fam) {
    if (!profile_on) return;
    ProfRec r{fam, nullptr, nullptr};
    for (cudaEvent_t* e : {&r.a, &r.b}) {
        if (!prof_pool_.empty()) { *e = prof_pool_.back(); prof_pool_.pop_back(); }
        else cudaEventCreate(e);
    }
    cudaEventRecord(r.a, stream);
    prof_recs_.push_back(r);
}

void Engine::prof_end(int fam) {
    (void)fam;
    if (!profile_on || prof_recs_.empty()) return;
    cudaEventRecord(prof_recs_.back().b, stream);
}

// Resolve the recorded event pairs (the stream has been synchronised by the caller).
int Engine::prof_flush() {
    if (prof_recs_.empty()) return SP_OK;
    for (ProfRec& r : prof_recs_) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            prof_ms_[r.fam] += ms;
            prof_n_[r.fam] += 1;
        } else {
            cudaGetLastError();
        }
        prof_pool_.push_back(r.a);
        prof_pool_.push_back(r.b);
    }
    prof_recs_.clear();
    return SP_OK;
}

int Engine::profile_read(double* ms, uint64_t* launches, int cap) {
    for (int i = 0; i < std::min<int>(cap, F_COUNT); ++i) {
        if (ms) ms[i] = prof_ms_[i];
        if (launches) launches[i] = prof_n_[i];
    }
    return F_COUNT;
}

void Engine::profile_reset() {
    for (int i = 0; i < F_COUNT; ++i) { prof_ms_[i] = 0; prof_n_[i] = 0; }
}

void Engine::drop_graphs() {
    if (stream) cudaStreamSynchronize(stream);
    for (auto& g : step_graphs_) cudaGraphExecDestroy(g.second);
    step_graphs_.clear();
    step_graph_kernels_.clear();
}

int Engine::drain_async() {
    if (!async_pending_) return SP_OK;
    async_pending_ = false;
    SP_CUDA_TRY(cudaStreamSynchronize(stream));
    SP_TRY(prof_flush());
    return device_check();
}

int Engine::launch_decode_step(int T) {
    if (!use_graphs || profile_on || trace_on) return enqueue_decode_step(T);
    const int key = T * 64 + step_splits(T);
    auto it = step_graphs_.find(key);
    if (it == step_graphs_.end()) {
        cudaGraph_t graph = nullptr;
        const uint64_t before = launch_count();
        SP_CUDA_TRY(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        graph_step_ = true;
        const int st = enqueue_decode_step(T);
        graph_step_ = false;
        const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
        const int64_t captured = (int64_t)(launch_count() - before);
        adjust_launch_count(-captured);  // captured, not executed
        step_graph_kernels_[key] = captured;
        if (st != SP_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (ce != cudaSuccess) { set_error(std::string("graph capture: ") + cudaGetErrorString(ce)); return SP_ERR_CUDA; }
        cudaGraphExec_t exec = nullptr;
        const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) { set_error(std::string("graph instantiate: ") + cudaGetErrorString(ie)); return SP_ERR_CUDA; }
        it = step_graphs_.emplace(key, exec).first;
    }
    SP_CUDA_TRY(cudaGraphLaunch(it->second, stream));
    adjust_launch_count(step_graph_kernels_[key]);
    return SP_OK;
}

int Engine::time_families(unsigned mask, int T, int reps, float* ms_per_step) {
    if (!finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    if (T <= 0 || T > logit_rows_ || reps <= 0 || !ms_per_step) { set_error("time_families: bad argument"); return SP_ERR_ARG; }
    if (d.tp_size > 1 && (mask & ((1u << F_COUNT) - 1)) != (1u << F_COUNT) - 1) {
        // a subset would run the producers of an exchange without its consumers (or the reverse)
        set_error("time_families: under tensor parallelism only the whole step can be timed");
        return SP_ERR_ARG;
    }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_TRY(drain_async());
    SP_CUDA_TRY(cudaStreamSynchronize(stream));
    const bool prof = profile_on, tr = trace_on;
    profile_on = false;
    trace_on = false;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    const uint64_t before = launch_count();
    fam_mask = mask;
    cudaError_t ce = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    int st = SP_OK;
    if (ce == cudaSuccess) {
        graph_step_ = true;  // as in launch_decode_step: captured kernels take positions from device memory only
        st = enqueue_decode_step(T);
        graph_step_ = false;
        ce = cudaStreamEndCapture(stream, &graph);
    }
    fam_mask = 0xFFFFFFFFu;
    profile_on = prof;
    trace_on = tr;
    const int64_t nodes = (int64_t)(launch_count() - before);
    adjust_launch_count(-nodes);
    if (st != SP_OK) { if (graph) cudaGraphDestroy(graph); return st; }
    if (ce != cudaSuccess || !graph) { set_error(std::string("time_families capture: ") + cudaGetErrorString(ce)); return SP_ERR_CUDA; }
    ce = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) { set_error(std::string("time_families instantiate: ") + cudaGetErrorString(ce)); return SP_ERR_CUDA; }
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    for (int i = 0; i < 3; ++i) cudaGraphLaunch(exec, stream);
    cudaEventRecord(a, stream);
    for (int i = 0; i < reps; ++i) cudaGraphLaunch(exec, stream);
    cudaEventRecord(b, stream);
    ce = cudaStreamSynchronize(stream);
    float ms = 0.f;
    if (ce == cudaSuccess) ce = cudaEventElapsedTime(&ms, a, b);
    adjust_launch_count(nodes * (reps + 3));
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    cudaGraphExecDestroy(exec);
    if (ce != cudaSuccess) { set_error(std::string("time_families: ") + cudaGetErrorString(ce)); return SP_ERR_CUDA; }
    *ms_per_step = ms / reps;
    return SP_OK;
}

int Engine::decode_greedy(const uint32_t* first_ids, const int32_t* slots, int b, int steps, uint32_t* tokens_out) {
    if (!finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    if (!first_ids || !slots || b <= 0 || steps <= 0) { set_error("empty input"); return SP_ERR_ARG; }
    if (b > logit_rows_ || b > d.max_tokens) { set_error("decode_greedy: batch larger than the decode step capacity"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_TRY(drain_async());
    for (int i = 0; i < b; ++i) {
        if (slots[i] < 0 || slots[i] >= d.max_batch) { set_error("slot out of range"); return SP_ERR_ARG; }
        for (int j = 0; j < i; ++j) if (slots[i] == slots[j]) { set_error("decode_greedy: a slot appears twice"); return SP_ERR_ARG; }
        if ((int64_t)first_ids[i] >= (int64_t)d.vocab) { set_error("token id out of vocab range"); return SP_ERR_VOCAB; }
        if (seq_len[slots[i]] + steps > d.max_ctx) { set_error("KV cache full"); return SP_ERR_KV_FULL; }
    }
    {
        int need = 0;
        for (int i = 0; i < b; ++i) {
            const int s = slots[i];
            need += pages.missing(s, seq_len[s] + steps) + ((seq_len[s] % KV_PAGE) && pages.ref[pages.page_of(s, seq_len[s] / KV_PAGE)] > 1 ? 1 : 0);
        }
        if (need > pages.available()) { set_error("KV page pool exhausted"); return SP_ERR_KV_FULL; }
    }
    for (int i = 0; i < b; ++i) SP_TRY(privatise_tail(slots[i]));
    // pages for every step up front, so nothing on the host has to happen between steps
    for (int i = 0; i < b; ++i) {
        SP_TRY(alloc_pages(slots[i], seq_len[slots[i]] + steps));
        p_slot_[i] = slots[i];
        p_pos_[i] = seq_len[slots[i]];
        p_ids_[i] = first_ids[i];
    }
    const size_t need_tok = (size_t)b * steps;
    if (need_tok > d_tokens_cap_) {
        if (d_tokens_) cudaFree(d_tokens_);
        d_tokens_ = nullptr;
        d_tokens_cap_ = 0;
        SP_CUDA_TRY(cudaMalloc((void**)&d_tokens_, need_tok * 4));
        d_tokens_cap_ = need_tok;
    }
    SP_CUDA_TRY(cudaMemcpyAsync(d_ids_, p_ids_, (size_t)b * 4, cudaMemcpyHostToDevice, stream));
    SP_CUDA_TRY(cudaMemcpyAsync(d_tok_slot_, p_slot_, (size_t)b * 4, cudaMemcpyHostToDevice, stream));
    SP_CUDA_TRY(cudaMemcpyAsync(d_tok_pos_, p_pos_, (size_t)b * 4, cudaMemcpyHostToDevice, stream));
    SP_TRY(sync_page_table());
    int done = 0, st = SP_OK, ctx0 = 0;
    for (int i = 0; i < b; ++i) ctx0 = std::max(ctx0, seq_len[slots[i]]);
    for (; done < steps && st == SP_OK; ++done) {
        step_ctx_ = ctx0 + done + 1;
        st = launch_decode_step(b);
        if (st != SP_OK) break;
        cudaError_t ce = launch_pdl(advance_greedy_kernel, dim3((b + 127) / 128), dim3(128), 0, stream, (const uint32_t*)d_argmax_, d_ids_,
                                    d_tok_pos_, d_tokens_ + (size_t)done * b, b);
        if (ce == cudaSuccess) ce = cudaGetLastError();
        if (ce != cudaSuccess) { set_error(std::string("advance_greedy_kernel: ") + cudaGetErrorString(ce)); st = SP_ERR_CUDA; break; }
        adjust_launch_count(1);
    }
    // the sequences now hold the steps that were enqueued completely; on an error the pages reserved for the rest go
    // back to the pool (truncate to the length reached)
    for (int i = 0; i < b; ++i) seq_len[slots[i]] += done;
    if (st != SP_OK) {
        cudaStreamSynchronize(stream);
        for (int i = 0; i < b; ++i) { size_t kept; truncate(slots[i], (size_t)seq_len[slots[i]], &kept); }
        return st;
    }
    if (tokens_out) {
        std::vector<uint32_t> tmp(need_tok);
        SP_CUDA_TRY(cudaMemcpyAsync(tmp.data(), d_tokens_, need_tok * 4, cudaMemcpyDeviceToHost, stream));
        SP_CUDA_TRY(cudaStreamSynchronize(stream));
        std::memcpy(tokens_out, tmp.data(), need_tok * 4);
        SP_TRY(prof_flush());
        return device_check();
    }
    async_pending_ = true;  // asynchronous: the caller synchronises the stream; the next call of this engine drains it
    return SP_OK;
}

}  // namespace sp
