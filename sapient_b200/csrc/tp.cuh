// Tensor-parallel exchange over peer memory (one process per GPU, NVLink / NVSwitch).
//
// Megatron-style split of a Llama-shaped decoder: q/k/v, gate/up and lm_head are split by output rows, o_proj and
// down_proj by input columns, so each layer needs two sums over the ranks of a [rows, hidden] partial result, and
// the greedy loop one arg-max over the ranks' vocabulary slices.
//
// Every rank owns one communication block (a single cudaMalloc, exported with a CUDA IPC handle and mapped by
// every peer):
//     ar_flags[2][8]   u32   all-reduce arrival flags, indexed [slot][source rank]
//     am_flags[2][8]   u32   arg-max arrival flags
//     am_vals [2][8][32] float2 (value, index bits) arg-max candidates per logit row
//     recv    [2][size][max_tokens * hidden] f32   partial sums pushed by every source rank
// The sum is a push: the row-split GEMV stores each output element straight into recv[slot][my rank] of EVERY rank
// (plain stores to peer pointers from the tensor-core kernel's epilogue); the kernel that consumes the sum then
// raises this rank's flag on every peer, waits (bounded) until all sources have raised theirs here, and adds the
// partials from LOCAL memory in rank order, so every rank computes bit-identical activations.
// slot = epoch & 1 where epoch counts the exchanges; a rank cannot be more than one exchange ahead of a peer
// (it needs that peer's flag to finish the current one), so two slots are enough.
// Waits are bounded: after TP_SPIN_LIMIT polls a kernel records the failure in `timeout` and goes on, the host
// reports SP_ERR_COMM. Peer memory is only ever written, with plain stores; nothing is loaded from a peer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sp {

constexpr int TP_MAX_RANKS = 8;
constexpr int TP_ARGMAX_ROWS = 32;
constexpr int TP_SPIN_LIMIT = 1 << 22;  // polls of ~0.25 us each: about a second

constexpr size_t TP_OFF_AR_FLAGS = 0;
constexpr size_t TP_OFF_AM_FLAGS = 256;
constexpr size_t TP_OFF_AM_VALS = 512;
constexpr size_t TP_OFF_RECV = 8192;

struct TpDev {
    int rank, size;
    int64_t slot_floats;               // floats of one (slot, source) region: max_tokens * hidden
    uint8_t* base[TP_MAX_RANKS];       // every rank's communication block (base[rank] is the local one)
    uint32_t* ar_seq;                  // local: exchanges completed so far
    uint32_t* am_seq;
    uint32_t* done;                    // local: block counter of the consuming kernel
    int* timeout;                      // local: set when a wait gave up
};

__device__ __forceinline__ float* tp_recv(const TpDev& tp, int on_rank, int slot, int src) {
    return reinterpret_cast<float*>(tp.base[on_rank] + TP_OFF_RECV) + ((int64_t)slot * tp.size + src) * tp.slot_floats;
}
__device__ __forceinline__ volatile uint32_t* tp_flag(const TpDev& tp, size_t off, int on_rank, int slot, int src) {
    return reinterpret_cast<volatile uint32_t*>(tp.base[on_rank] + off) + slot * TP_MAX_RANKS + src;
}

// Polls a flag in local memory until it holds `epoch`; false after TP_SPIN_LIMIT polls.
__device__ __forceinline__ bool tp_wait_flag(volatile uint32_t* f, uint32_t epoch) {
    for (int i = 0; i < TP_SPIN_LIMIT; ++i) {
        if (*f == epoch) return true;
        __nanosleep(200);
    }
    return false;
}

cudaError_t launch_tp_reduce(float* x, int ldx, int rows, int dim, const TpDev* tp, cudaStream_t st);
cudaError_t launch_tp_argmax(const float* logits, int ld, int rows, int vocab_off, uint32_t* argmax, const TpDev* tp, cudaStream_t st);

}  // namespace sp
