// Split-K paged attention for callers that must not allocate device memory.
//
// sp_cuda_attention builds a cache from host buffers and allocates what it needs on every call. Some callers
// cannot afford that: a serving loop that has handed all device memory to its own pool (a cudaMalloc there can
// fail or fragment the pool), or code running between other streams' work, where an allocation's implicit
// device-wide synchronisation would stall everyone. This entry point takes device pointers for everything the
// caller owns and keeps the one temporary it needs — the per-split partial results (m, l, o[head_dim]) of the
// split-K kernel — in a fixed-size array that is part of the loaded module.
//
// The array is one per device and shared by every call: two calls that overlap in time (different streams or
// threads) race on it, so callers serialise them. It keeps the contents of the last call; nothing has to start
// at zero, because the split kernel writes every partial the merge kernel reads before the merge runs.
// The first call on a device looks the array's address up (cudaGetSymbolAddress); make that call before any
// stream capture begins.
#include <mutex>
#include <string>

#include <cmath>

#include "engine.h"

namespace sp {

constexpr size_t STATIC_SCRATCH_FLOATS = SP_ATTENTION_STATIC_MAX_FLOATS;
static __device__ __align__(256) float g_static_split_scratch[STATIC_SCRATCH_FLOATS];

constexpr int STATIC_MAX_DEVICES = 64;
static std::mutex g_static_mu;
static float* g_static_ptr[STATIC_MAX_DEVICES] = {};

// Device address of the array on the current device. The array's name is a host-side handle, not a device
// address, so it is resolved once per device and cached.
static int static_scratch(int device, float** out) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[device]) {
        void* p = nullptr;
        SP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_split_scratch));
        if (!p) { set_error("static scratch: no device address"); return SP_ERR_CUDA; }
        g_static_ptr[device] = static_cast<float*>(p);
    }
    *out = g_static_ptr[device];
    return SP_OK;
}

}  // namespace sp

using namespace sp;

extern "C" int32_t sp_cuda_attention_paged_static(int32_t device, const float* d_q, int32_t ldq, float* d_out, int32_t ldo,
                                                  int32_t n_tok, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                                  const int32_t* d_tok_slot, const int32_t* d_tok_pos, const void* d_kv_pool,
                                                  const int32_t* d_page_table, int32_t n_pages, int32_t max_pages, int32_t layer,
                                                  int32_t n_splits, void* stream) {
    try {
        if (!d_q || !d_out || !d_tok_slot || !d_tok_pos || !d_kv_pool || !d_page_table) { set_error("null argument"); return SP_ERR_ARG; }
        if (device < 0 || device >= STATIC_MAX_DEVICES) { set_error("device index out of range"); return SP_ERR_ARG; }
        if (n_tok < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || head_dim <= 0 || head_dim % 2 != 0 ||
            head_dim > 256 || ldq < n_heads * head_dim || ldo < n_heads * head_dim || n_pages <= 0 || max_pages <= 0 || layer < 0) {
            set_error("bad attention shape");
            return SP_ERR_SHAPE;
        }
        if (n_splits < 1 || n_splits > 64) { set_error("n_splits must be 1..64"); return SP_ERR_ARG; }
        const size_t need = attention_scratch_floats(n_tok, n_heads, n_splits, head_dim);
        if (need > STATIC_SCRATCH_FLOATS) {
            set_error("split scratch of " + std::to_string(need) + " floats exceeds the static buffer of " +
                      std::to_string(STATIC_SCRATCH_FLOATS) + " floats; use fewer tokens or splits per call");
            return SP_ERR_SHAPE;
        }
        if (n_tok == 0) return SP_OK;
        SP_CUDA_TRY(cudaSetDevice(device));
        float* scratch = nullptr;
        const int st = static_scratch(device, &scratch);
        if (st != SP_OK) return st;
        KvGeom g{};
        g.pool = static_cast<__half*>(const_cast<void*>(d_kv_pool));  // read only here
        g.page_table = d_page_table;
        g.n_pages = n_pages;
        g.n_kv = n_kv_heads;
        g.head_dim = head_dim;
        g.max_pages = max_pages;
        SP_CUDA_TRY(launch_attention(d_q, ldq, d_out, ldo, n_tok, n_heads, d_tok_slot, d_tok_pos, g, layer, 1.0f / sqrtf((float)head_dim),
                                     n_splits, scratch, static_cast<cudaStream_t>(stream)));
        return SP_OK;
    } catch (...) {
        set_error("internal error");
        return SP_ERR_ARG;
    }
}
