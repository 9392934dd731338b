// Tensor-parallel exchange over peer memory (one process per GPU, NVLink / NVSwitch).
//
// Megatron-style split of a Llama-shaped decoder: q/k/v, gate/up and lm_head are split by output rows, o_proj and
// down_proj by input columns, so each layer needs two sums over the ranks of a [rows, hidden] partial result, and
// the greedy loop one arg-max over the ranks' vocabulary slices.
//
// Every rank owns one communication block (a single cudaMalloc, exported with a CUDA IPC handle and mapped by
// every peer):
//     am_flags[2][8]   u32   arg-max arrival flags, indexed [slot][source rank]
//     am_vals [2][8][32] float2 (value, index bits) arg-max candidates per logit row
//     recv    [2][size][max_tokens * hidden] u64   partial sums pushed by every source rank
// The sum is a push with the arrival flag inside the data: the column-split GEMV stores each output element
// straight into recv[slot][my rank] of EVERY rank (plain 64-bit stores to peer pointers from the tensor-core
// kernel's epilogue) as one word = (exchange number << 32) | float bits. A 64-bit store is a single copy, so a
// reader that sees the exchange number also sees the value: no fence, no separate flag, no extra kernel. The
// kernel that consumes the sum — the following RMSNorm, or a small stand-alone kernel — polls (bounded) the
// words of its row in LOCAL memory until all carry the current exchange number and adds the values in rank
// order, so every rank computes bit-identical activations.
// slot = epoch & 1 where epoch counts the exchanges; a rank cannot be more than one exchange ahead of a peer
// (it needs that peer's words to finish the current one), so two slots are enough, and a word left over from
// two exchanges ago never matches.
// Waits are bounded in time (TpDev::wait_ns of the device's global timer, 5 s unless the host sets another bound: long
// enough for a peer that is still capturing its first step graph, short enough to end a step whose peer has gone): a
// kernel whose wait runs out records the failure in `timeout` and goes on, the host reports SP_ERR_COMM. Peer memory is only ever written, with plain stores; nothing is loaded from a peer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sp {

constexpr int TP_MAX_RANKS = 8;
constexpr int TP_ARGMAX_ROWS = 32;
constexpr uint64_t TP_WAIT_NS_DEFAULT = 5ull * 1000 * 1000 * 1000;  // how long a kernel waits for a peer before it gives up

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
    uint64_t wait_ns;                  // bound of every wait, in nanoseconds of the device's global timer
};

__device__ __forceinline__ uint64_t tp_now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned long long* tp_recv(const TpDev& tp, int on_rank, int slot, int src) {
    return reinterpret_cast<unsigned long long*>(tp.base[on_rank] + TP_OFF_RECV) + ((int64_t)slot * tp.size + src) * tp.slot_floats;
}
__device__ __forceinline__ unsigned long long tp_word(float v, uint32_t epoch) {
    return ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
}
__device__ __forceinline__ volatile uint32_t* tp_flag(const TpDev& tp, size_t off, int on_rank, int slot, int src) {
    return reinterpret_cast<volatile uint32_t*>(tp.base[on_rank] + off) + slot * TP_MAX_RANKS + src;
}

// Polls a flag in local memory until it holds `epoch`; false once wait_ns have passed.
__device__ __forceinline__ bool tp_wait_flag(volatile uint32_t* f, uint32_t epoch, uint64_t wait_ns) {
    const uint64_t t0 = tp_now_ns();
    for (;;) {
        if (*f == epoch) return true;
        if (tp_now_ns() - t0 > wait_ns) return false;
        __nanosleep(200);
    }
}

// Consumer side of one exchange, called by every thread of a block after the grid-dependency wait: adds the
// partial rows of all sources to x[row, 0..dim) (dim % 4 == 0), polling each word until it carries this exchange's
// number. Returns the epoch for tp_consume_done.
__device__ __forceinline__ uint32_t tp_consume_row(const TpDev& tp, float* x, int64_t row_off_x, int row, int dim) {
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tp.ar_seq) + 1u;
    const int slot = (int)(epoch & 1u);
    // once any wait of this engine has expired (now or in an earlier kernel) nothing waits again: the step finishes
    // with undefined values, the host sees the flag and reports SP_ERR_COMM
    bool ok = *reinterpret_cast<volatile int*>(tp.timeout) == 0;
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
        float4 acc = *reinterpret_cast<const float4*>(x + row_off_x + i);
        // the words of all sources are requested together (one round trip to memory, not one per source); only sources
        // whose words are still from an earlier exchange are read again
        unsigned long long w[TP_MAX_RANKS][4];
        unsigned pending = (1u << tp.size) - 1u;
        uint64_t t0 = 0;  // read on the first miss only: the common case costs no timer access
        for (;;) {
#pragma unroll
            for (int s = 0; s < TP_MAX_RANKS; ++s) {
                if (s < tp.size && (pending >> s & 1u)) {
                    const volatile ulonglong2* src = reinterpret_cast<const volatile ulonglong2*>(tp_recv(tp, tp.rank, slot, s) + (int64_t)row * dim + i);
                    w[s][0] = src[0].x; w[s][1] = src[0].y; w[s][2] = src[1].x; w[s][3] = src[1].y;
                }
            }
#pragma unroll
            for (int s = 0; s < TP_MAX_RANKS; ++s) {
                if (s < tp.size && (pending >> s & 1u) && (uint32_t)(w[s][0] >> 32) == epoch && (uint32_t)(w[s][1] >> 32) == epoch &&
                    (uint32_t)(w[s][2] >> 32) == epoch && (uint32_t)(w[s][3] >> 32) == epoch)
                    pending &= ~(1u << s);
            }
            if (pending == 0u || !ok) break;
            const uint64_t now = tp_now_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > tp.wait_ns) { ok = false; break; }
            __nanosleep(100);
        }
#pragma unroll
        for (int s = 0; s < TP_MAX_RANKS; ++s) {  // rank order: every rank adds the same values in the same order
            if (s < tp.size) {
                acc.x += __uint_as_float((uint32_t)w[s][0]); acc.y += __uint_as_float((uint32_t)w[s][1]);
                acc.z += __uint_as_float((uint32_t)w[s][2]); acc.w += __uint_as_float((uint32_t)w[s][3]);
            }
        }
        *reinterpret_cast<float4*>(x + row_off_x + i) = acc;
    }
    if (!ok) atomicExch(tp.timeout, 1);
    __syncthreads();  // the block's own stores to x are visible to all its threads from here on
    return epoch;
}
// After every block of the consuming grid has called tp_consume_row: the last one publishes the new sequence number.
__device__ __forceinline__ void tp_consume_done(const TpDev& tp, uint32_t epoch, unsigned n_blocks) {
    if (threadIdx.x == 0 && atomicAdd(tp.done, 1u) == n_blocks - 1) {
        *tp.done = 0u;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(tp.ar_seq) = epoch;  // every block has read the old value by now
    }
}

cudaError_t launch_tp_reduce(float* x, int ldx, int rows, int dim, const TpDev* tp, cudaStream_t st);
// Pushes the partial rows part[rows][dim] (row stride ld) of a column-split product into every rank's receive area, as
// the GEMV epilogue does for its own outputs; the consumer is launch_tp_reduce or the fused norm.
cudaError_t launch_tp_push(const float* part, int ld, int rows, int dim, const TpDev* tp, cudaStream_t st);
cudaError_t launch_tp_argmax(const float* logits, int ld, int rows, int vocab_off, uint32_t* argmax, const TpDev* tp, cudaStream_t st);

}  // namespace sp
