// Tensor parallelism: weight sharding at load, the communication block, and the two exchange kernels
// (see tp.cuh for the protocol).
#include "tp.cuh"

#include <algorithm>
#include <cstddef>
#include <cstring>

#include "engine.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

// ───────────────────────────── sharding (host) ─────────────────────────────
// Which slice of a full tensor a rank keeps. Names are the HF names the reference's GGUF name map produces
// (crates/sapient-models/src/gguf_weights.rs:360-455).
enum ShardKind { SHARD_NONE = 0, SHARD_ROWS, SHARD_COLS, SHARD_VOCAB_ROWS };

static bool ends_with(const std::string& s, const char* suf) {
    const size_t n = std::strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

static ShardKind shard_kind(const std::string& nm) {
    for (const char* p : {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj"})
        if (ends_with(nm, (std::string(p) + ".weight").c_str()) || ends_with(nm, (std::string(p) + ".bias").c_str())) return SHARD_ROWS;
    if (ends_with(nm, "self_attn.o_proj.weight") || ends_with(nm, "mlp.down_proj.weight")) return SHARD_COLS;
    if (nm == "lm_head.weight") return SHARD_VOCAB_ROWS;
    return SHARD_NONE;
}

// Slices `bytes` (dims [n, k] or [n]) for rank `rank` of `size`; vocab limits the rows of the output head.
// Returns SP_OK with out/out_dims filled, or an error (indivisible sizes). SHARD_NONE copies nothing (out empty).
int tp_shard_tensor(const std::string& nm, int dtype, const int64_t* dims, int ndim, const uint8_t* bytes, int rank, int size,
                    int64_t vocab, std::vector<uint8_t>& out, std::vector<int64_t>& out_dims, bool& sharded) {
    sharded = false;
    out.clear();
    out_dims.assign(dims, dims + ndim);
    const ShardKind kind = shard_kind(nm);
    if (kind == SHARD_NONE || size <= 1) return SP_OK;
    const int bb = block_bytes(dtype), be = block_elems(dtype);
    if (bb == 0) { set_error("unsupported dtype for " + nm); return SP_ERR_DTYPE; }
    if (ndim == 1) {  // bias of a row-split matrix
        if (dims[0] % size != 0 || (dims[0] / size) % be != 0) { set_error("tensor parallel: cannot split " + nm); return SP_ERR_SHAPE; }
        const int64_t nl = dims[0] / size;
        out.assign(bytes + rank * nl / be * bb, bytes + (rank + 1) * nl / be * bb);
        out_dims[0] = nl;
        sharded = true;
        return SP_OK;
    }
    const int64_t n = dims[0], k = dims[1];
    const int64_t row_b = k / be * bb;
    if (kind == SHARD_ROWS || kind == SHARD_VOCAB_ROWS) {
        const int64_t rows = kind == SHARD_VOCAB_ROWS ? std::min<int64_t>(n, vocab) : n;
        if (rows % size != 0) { set_error("tensor parallel: rows of " + nm + " do not divide by the rank count"); return SP_ERR_SHAPE; }
        const int64_t nl = rows / size;
        out.assign(bytes + rank * nl * row_b, bytes + (rank + 1) * nl * row_b);
        out_dims[0] = nl;
    } else {
        if (k % size != 0 || (k / size) % be != 0) {
            set_error("tensor parallel: columns of " + nm + " do not split on block boundaries");
            return SP_ERR_SHAPE;
        }
        const int64_t kl = k / size, seg_b = kl / be * bb;
        out.resize((size_t)(n * seg_b));
        for (int64_t r = 0; r < n; ++r) std::memcpy(&out[(size_t)(r * seg_b)], bytes + r * row_b + rank * seg_b, (size_t)seg_b);
        out_dims[1] = kl;
    }
    sharded = true;
    return SP_OK;
}

// ───────────────────────────── exchange kernels ─────────────────────────────
// x[row, :] += sum over ranks of the partial rows that the column-split GEMV pushed; one block per activation row.
// Used where the next kernel is not the fused norm (prefill-shaped steps, tracing).
__global__ void __launch_bounds__(256) tp_reduce_kernel(float* __restrict__ x, int ldx, int dim, const TpDev* __restrict__ tpp) {
    pdl_wait();
    pdl_trigger();
    const TpDev& tp = *tpp;
    const uint32_t epoch = tp_consume_row(tp, x, (int64_t)blockIdx.x * ldx, blockIdx.x, dim);
    tp_consume_done(tp, epoch, gridDim.x);
}

cudaError_t launch_tp_reduce(float* x, int ldx, int rows, int dim, const TpDev* tp, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (dim % 4 != 0) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(tp_reduce_kernel, dim3(rows), dim3(256), 0, st, x, ldx, dim, tp);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

// Partial rows of a column-split product computed by a kernel that cannot push them itself (the tcgen05 GEMM): two
// elements per thread, one 128-bit store per peer, each element tagged with the exchange number like the GEMV's.
__global__ void __launch_bounds__(256) tp_push_kernel(const float* __restrict__ part, int ld, int rows, int dim, const TpDev* __restrict__ tpp) {
    pdl_wait();
    pdl_trigger();
    const TpDev& tp = *tpp;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tp.ar_seq) + 1u;
    const int slot = (int)(epoch & 1u);
    const int64_t pairs = (int64_t)rows * dim / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = (2 * i) / dim, c = 2 * i - r * dim;
        const float2 v = *reinterpret_cast<const float2*>(part + r * ld + c);
        ulonglong2 w;
        w.x = tp_word(v.x, epoch);
        w.y = tp_word(v.y, epoch);
        for (int p = 0; p < tp.size; ++p) *reinterpret_cast<ulonglong2*>(tp_recv(tp, p, slot, tp.rank) + r * dim + c) = w;
    }
}

cudaError_t launch_tp_push(const float* part, int ld, int rows, int dim, const TpDev* tp, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (dim % 2 != 0 || ld % 2 != 0) return cudaErrorInvalidValue;
    const int64_t pairs = (int64_t)rows * dim / 2;
    cudaError_t le = launch_pdl(tp_push_kernel, dim3((unsigned)std::min<int64_t>((pairs + 255) / 256, 148 * 8)), dim3(256), 0, st, part, ld, rows, dim, tp);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

// Global arg-max of `rows` logit rows whose vocabulary is split over the ranks: every rank publishes
// (max value, global index) of its slice, then all pick the largest value, the largest index among equals
// (the reference's tie rule: the last maximum wins, crates/sapient-generate/src/sampler.rs:161-168).
__global__ void __launch_bounds__(32) tp_argmax_kernel(const float* __restrict__ logits, int ld, int rows, int vocab_off,
                                                       uint32_t* __restrict__ argmax, const TpDev* __restrict__ tpp) {
    pdl_wait();
    pdl_trigger();
    const TpDev& tp = *tpp;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tp.am_seq) + 1u;
    const int slot = (int)(epoch & 1u), lane = threadIdx.x;
    if (lane < rows) {
        const uint32_t li = argmax[lane];
        const float2 cand = make_float2(logits[(int64_t)lane * ld + li], __uint_as_float(li + (uint32_t)vocab_off));
        for (int p = 0; p < tp.size; ++p)
            reinterpret_cast<float2*>(tp.base[p] + TP_OFF_AM_VALS)[((int64_t)slot * TP_MAX_RANKS + tp.rank) * TP_ARGMAX_ROWS + lane] = cand;
    }
    __threadfence_system();
    __syncwarp();
    if (lane < tp.size) *tp_flag(tp, TP_OFF_AM_FLAGS, lane, slot, tp.rank) = epoch;
    if (lane < tp.size) {
        const bool already = *reinterpret_cast<volatile int*>(tp.timeout) != 0;  // an earlier wait expired: do not wait again
        if (!already && !tp_wait_flag(tp_flag(tp, TP_OFF_AM_FLAGS, tp.rank, slot, lane), epoch, tp.wait_ns)) atomicExch(tp.timeout, 1);
        __threadfence_system();
    }
    __syncwarp();
    if (lane < rows) {
        float best = -INFINITY;
        uint32_t best_i = 0;
        bool have = false;
        for (int s = 0; s < tp.size; ++s) {
            const float2 c = __ldcg(reinterpret_cast<const float2*>(tp.base[tp.rank] + TP_OFF_AM_VALS) +
                                    ((int64_t)slot * TP_MAX_RANKS + s) * TP_ARGMAX_ROWS + lane);
            const uint32_t ci = __float_as_uint(c.y);
            // sources are visited in rank order = ascending index: ">=" keeps the last maximum; NaN compares equal
            // to everything in the reference's partial_cmp fallback, so it replaces the running best as well
            if (!have || !(c.x < best)) { best = c.x; best_i = ci; have = true; }
        }
        argmax[lane] = best_i;
    }
    __syncwarp();
    if (lane == 0) *reinterpret_cast<volatile uint32_t*>(tp.am_seq) = epoch;
}

cudaError_t launch_tp_argmax(const float* logits, int ld, int rows, int vocab_off, uint32_t* argmax, const TpDev* tp, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (rows > TP_ARGMAX_ROWS) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(tp_argmax_kernel, dim3(1), dim3(32), 0, st, logits, ld, rows, vocab_off, argmax, tp);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

// ───────────────────────────── engine side ─────────────────────────────
size_t Engine::tp_block_bytes() const { return TP_OFF_RECV + (size_t)2 * d.tp_size * d.max_tokens * d.hidden * 8; }

int Engine::tp_alloc() {
    if (d.tp_size <= 1) return SP_OK;
    SP_CUDA_TRY(cudaMalloc((void**)&tp_block_, tp_block_bytes()));
    SP_CUDA_TRY(cudaMemset(tp_block_, 0, tp_block_bytes()));
    SP_CUDA_TRY(cudaMalloc((void**)&tp_state_, 64));
    SP_CUDA_TRY(cudaMemset(tp_state_, 0, 64));
    SP_CUDA_TRY(cudaMalloc((void**)&d_tp_, sizeof(TpDev)));
    return SP_OK;
}

void Engine::tp_release() {
    for (int r = 0; r < TP_MAX_RANKS; ++r)
        if (tp_peer_[r] && r != d.tp_rank) cudaIpcCloseMemHandle(tp_peer_[r]);
    if (tp_block_) cudaFree(tp_block_);
    if (tp_state_) cudaFree(tp_state_);
    if (d_tp_) cudaFree(d_tp_);
}

int Engine::tp_handle(void* out, size_t cap) {
    if (d.tp_size <= 1 || !tp_block_) { set_error("engine is not tensor parallel (or not finalised)"); return SP_ERR_STATE; }
    if (!out || cap < sizeof(cudaIpcMemHandle_t)) { set_error("tp_handle: buffer too small"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    cudaIpcMemHandle_t h;
    SP_CUDA_TRY(cudaIpcGetMemHandle(&h, tp_block_));
    std::memcpy(out, &h, sizeof(h));
    return SP_OK;
}

int Engine::tp_connect(const void* handles, int n) {
    if (d.tp_size <= 1 || !tp_block_) { set_error("engine is not tensor parallel (or not finalised)"); return SP_ERR_STATE; }
    if (!handles || n != d.tp_size) { set_error("tp_connect: need one handle per rank"); return SP_ERR_ARG; }
    if (tp_connected_) { set_error("tp_connect: already connected"); return SP_ERR_STATE; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    TpDev h{};
    h.rank = d.tp_rank;
    h.size = d.tp_size;
    h.slot_floats = (int64_t)d.max_tokens * d.hidden;
    for (int r = 0; r < n; ++r) {
        if (r == d.tp_rank) { tp_peer_[r] = tp_block_; }
        else {
            cudaIpcMemHandle_t mh;
            std::memcpy(&mh, (const uint8_t*)handles + (size_t)r * sizeof(mh), sizeof(mh));
            void* p = nullptr;
            SP_CUDA_TRY(cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess));
            tp_peer_[r] = (uint8_t*)p;
        }
        h.base[r] = tp_peer_[r];
    }
    uint32_t* st = (uint32_t*)tp_state_;
    h.ar_seq = st; h.am_seq = st + 1; h.done = st + 2; h.timeout = (int*)(st + 3);
    h.wait_ns = tp_wait_ns_;
    SP_CUDA_TRY(cudaMemcpy(d_tp_, &h, sizeof(h), cudaMemcpyHostToDevice));
    tp_connected_ = true;
    return SP_OK;
}

int Engine::tp_connect_ptrs(void* const* blocks, int n) {
    if (d.tp_size <= 1 || !tp_block_) { set_error("engine is not tensor parallel (or not finalised)"); return SP_ERR_STATE; }
    if (!blocks || n != d.tp_size) { set_error("tp_connect: need one block per rank"); return SP_ERR_ARG; }
    if (tp_connected_) { set_error("tp_connect: already connected"); return SP_ERR_STATE; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    TpDev h{};
    h.rank = d.tp_rank;
    h.size = d.tp_size;
    h.slot_floats = (int64_t)d.max_tokens * d.hidden;
    for (int r = 0; r < n; ++r) {
        if (!blocks[r]) { set_error("tp_connect: null block"); return SP_ERR_ARG; }
        h.base[r] = r == d.tp_rank ? tp_block_ : (uint8_t*)blocks[r];  // tp_peer_ stays empty: nothing to close
    }
    uint32_t* st = (uint32_t*)tp_state_;
    h.ar_seq = st; h.am_seq = st + 1; h.done = st + 2; h.timeout = (int*)(st + 3);
    h.wait_ns = tp_wait_ns_;
    SP_CUDA_TRY(cudaMemcpy(d_tp_, &h, sizeof(h), cudaMemcpyHostToDevice));
    tp_connected_ = true;
    return SP_OK;
}

// A new bound for the waits on peers (takes effect with the next launch; captured step graphs read it from device memory).
int Engine::tp_set_wait_ms(int ms) {
    if (ms <= 0) { set_error("tp_set_wait_ms: the bound must be positive"); return SP_ERR_ARG; }
    tp_wait_ns_ = (uint64_t)ms * 1000000ull;
    if (!tp_connected_) return SP_OK;
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_CUDA_TRY(cudaStreamSynchronize(stream));
    SP_CUDA_TRY(cudaMemcpy((uint8_t*)d_tp_ + offsetof(TpDev, wait_ns), &tp_wait_ns_, sizeof(uint64_t), cudaMemcpyHostToDevice));
    return SP_OK;
}

// After SP_ERR_COMM (or to restart cleanly): exchange counters, arrival marks and the sticky flag back to their initial
// state. Every rank must call it, with a host barrier before (no rank still inside a step) and after (no rank starts a
// step before all have cleared): the epochs of the ranks must agree again.
int Engine::tp_reset() {
    if (d.tp_size <= 1 || !tp_block_) { set_error("engine is not tensor parallel (or not finalised)"); return SP_ERR_STATE; }
    SP_CUDA_TRY(cudaSetDevice(d.device));
    SP_CUDA_TRY(cudaStreamSynchronize(stream));
    SP_CUDA_TRY(cudaMemset(tp_block_, 0, tp_block_bytes()));
    SP_CUDA_TRY(cudaMemset(tp_state_, 0, 64));
    tp_pending_ = false;
    SP_CUDA_TRY(cudaDeviceSynchronize());
    return SP_OK;
}

int Engine::device_check() {
    const int a = tc5_take_timeout(), b = imma_take_timeout();
    if (a < 0 || b < 0) { set_error("could not read the kernels' timeout flags"); return SP_ERR_CUDA; }
    if (a > 0) { set_error("tcgen05 GEMM: a bounded mbarrier wait expired, the outputs of that launch are not valid"); return SP_ERR_CUDA; }
    if (b > 0) { set_error("streaming GEMV: a bounded mbarrier wait expired, the outputs of that launch are not valid"); return SP_ERR_CUDA; }
    return tp_check();
}

int Engine::tp_check() {
    if (d.tp_size <= 1) return SP_OK;
    int flag = 0;
    SP_CUDA_TRY(cudaMemcpy(&flag, (uint8_t*)tp_state_ + 12, 4, cudaMemcpyDeviceToHost));
    if (flag) { set_error("tensor-parallel exchange timed out waiting for a peer"); return SP_ERR_COMM; }
    return SP_OK;
}

}  // namespace sp
