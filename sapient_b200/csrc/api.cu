// extern "C" surface of libsapient_cuda.so (declarations: include/sapient_cuda.h).
// No exception leaves this file; every entry sets the CUDA device it works on.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "batcher.h"
#include "engine.h"
#include "sp_common.cuh"

using namespace sp;

struct SpWeight {
    int device;
    int dtype;
    int64_t n, k;
    uint8_t* d;
    size_t nbytes;
    uint8_t* tiled = nullptr;  // tile-repacked copy for the tensor-core GEMV (quantised types)
    ActWorkspace ws;           // activation digits for up to 16 rows
    RingScratch ring;          // shared-row scratch of the ring GEMV (calls of 1-4 rows)
    RowsScratch rows;          // K-split partials of the one-pass many-row GEMV
};
struct SpEngine {
    Engine* e;
};

int sp_engine_from_gguf_impl(const char* path, int device, int max_ctx, int max_batch, Engine** out);  // gguf.cu
namespace sp {
int nccl_unique_id(const char* libpath, void* out, size_t cap);  // nccl_arm.cu
int spec_greedy(Engine* target, Engine* draft, const uint32_t* prompt, size_t n_prompt, int k, size_t max_new, const uint32_t* eos,
                int n_eos, uint32_t* tokens_out, size_t* n_out, uint64_t* stats);  // spec.cu
}

namespace {

std::atomic<int> g_gemv_path{0};  // 0: tensor-core GEMV on tiled weights; 1: CUDA-core GEMV on raw blocks
std::atomic<int> g_rows{1};       // calls of 11 rows and more on the one-pass many-row GEMV (path 2 turns it off: passes of 10 rows)
std::atomic<int> g_ring{0};       // calls of 1-5 rows on the bulk-copy ring GEMV where it fits (path 4)

#define API_BEGIN try {
#define API_END                                                     \
    }                                                               \
    catch (const std::bad_alloc&) {                                 \
        set_error("host allocation failed");                        \
        return SP_ERR_OOM;                                          \
    }                                                               \
    catch (const std::exception& ex) {                              \
        set_error(std::string("internal error: ") + ex.what());     \
        return SP_ERR_ARG;                                          \
    }                                                               \
    catch (...) {                                                   \
        set_error("internal error");                                \
        return SP_ERR_ARG;                                          \
    }

// RAII device scratch for the host-buffer op entry points.
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 16); }
    template <class T> T* as() { return (T*)p; }
};

int check_weight_shape(int dtype, int64_t n, int64_t k, size_t nbytes) {
    const int be = block_elems(dtype), bb = block_bytes(dtype);
    if (bb == 0) { set_error("unsupported dtype"); return SP_ERR_DTYPE; }
    if (n < 0 || k <= 0) { set_error("bad shape"); return SP_ERR_SHAPE; }
    if (dtype == T_Q4_K || dtype == T_Q5_K || dtype == T_Q6_K) {
        if (k % 256 != 0) { set_error("k must be a multiple of 256"); return SP_ERR_SHAPE; }
    } else if (dtype == T_Q8_0 || dtype == T_Q4_0) {
        if (k % 32 != 0) { set_error("k must be a multiple of the block size (32)"); return SP_ERR_SHAPE; }
    } else if (k % 4 != 0) {
        set_error("k must be a multiple of 4");
        return SP_ERR_SHAPE;
    }
    if ((size_t)(n * k / be * bb) != nbytes) { set_error("byte size does not match dtype and shape"); return SP_ERR_SHAPE; }
    return SP_OK;
}

int unary_op(int device, const float* x, int64_t n, float* y, cudaError_t (*fn)(float*, int64_t, cudaStream_t)) {
    if (!x || !y || n < 0) { set_error("null argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(device));
    DevBuf b;
    SP_CUDA_TRY(b.alloc((size_t)n * 4));
    SP_CUDA_TRY(cudaMemcpy(b.p, x, (size_t)n * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(fn(b.as<float>(), n, 0));
    SP_CUDA_TRY(cudaMemcpy(y, b.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
}

int binary_op(int device, const float* a, const float* b, int64_t n, float* y,
              cudaError_t (*fn)(const float*, const float*, float*, int64_t, cudaStream_t)) {
    if (!a || !b || !y || n < 0) { set_error("null argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(device));
    DevBuf da, db;
    SP_CUDA_TRY(da.alloc((size_t)n * 4));
    SP_CUDA_TRY(db.alloc((size_t)n * 4));
    SP_CUDA_TRY(cudaMemcpy(da.p, a, (size_t)n * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(db.p, b, (size_t)n * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(fn(da.as<float>(), db.as<float>(), da.as<float>(), n, 0));
    SP_CUDA_TRY(cudaMemcpy(y, da.p, (size_t)n * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
}

// RoPE table for arbitrary positions: row i holds the angles of positions[i].
std::vector<float2> rope_rows(const int64_t* positions, int64_t seq, float base, int64_t rotary_dim) {
    const int64_t half = rotary_dim / 2;
    std::vector<float2> cs((size_t)(seq * half));
    for (int64_t s = 0; s < seq; ++s)
        for (int64_t i = 0; i < half; ++i) {
            const float freq = ((float)positions[s] / 1.0f) / powf(base, 2.0f * (float)i / (float)rotary_dim);
            cs[(size_t)(s * half + i)] = make_float2(cosf(freq), sinf(freq));
        }
    return cs;
}

}  // namespace

extern "C" {

const char* sp_cuda_last_error(void) { return get_error(); }

int32_t sp_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

uint64_t sp_cuda_launch_count(void) { return launch_count(); }

int32_t sp_cuda_engine_set_kv_rounding(SpEngine* e, int32_t mode) {
    API_BEGIN
    if (!e || mode < 0 || mode > 1) { set_error("bad argument"); return SP_ERR_ARG; }
    for (int len : e->e->seq_len)
        if (len != 0) { set_error("set_kv_rounding: the KV cache is not empty"); return SP_ERR_STATE; }
    if (e->e->kv_round != mode) {
        e->e->kv_round = mode;
        e->e->drop_graphs();
    }
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_tp_handle(SpEngine* e, void* out, size_t cap) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_handle(out, cap);
    API_END
}

int32_t sp_cuda_engine_tp_connect(SpEngine* e, const void* handles, int32_t n_ranks) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_connect(handles, n_ranks);
    API_END
}

int32_t sp_cuda_engine_tp_block(SpEngine* e, void** block) {
    API_BEGIN
    if (!e || !block) { set_error("null argument"); return SP_ERR_ARG; }
    *block = e->e->tp_block();
    if (!*block) { set_error("engine is not tensor parallel (or not finalised)"); return SP_ERR_STATE; }
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_tp_connect_local(SpEngine* e, void* const* blocks, int32_t n_ranks) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_connect_ptrs(blocks, n_ranks);
    API_END
}

int32_t sp_cuda_engine_vocab_local(const SpEngine* e, int32_t* rows, int32_t* first) {
    API_BEGIN
    if (!e || !rows) { set_error("null argument"); return SP_ERR_ARG; }
    *rows = e->e->vocab_local();
    if (first) *first = e->e->d.tp_rank * e->e->vocab_local();
    return SP_OK;
    API_END
}

int32_t sp_cuda_tp_shard(const char* hf_name, int32_t dtype, const int64_t* dims, int32_t ndim, const void* bytes, size_t nbytes,
                         int32_t rank, int32_t size, int64_t vocab, void* out, size_t out_cap, int64_t* out_dims, size_t* out_bytes) {
    API_BEGIN
    if (!hf_name || !dims || !bytes || !out_dims || !out_bytes || ndim < 1 || ndim > 2 || size < 1 || rank < 0 || rank >= size) {
        set_error("tp_shard: bad argument");
        return SP_ERR_ARG;
    }
    const int bb = block_bytes(dtype), be = block_elems(dtype);
    if (bb == 0) { set_error("unsupported dtype"); return SP_ERR_DTYPE; }
    int64_t numel = 1;
    for (int i = 0; i < ndim; ++i) numel *= dims[i];
    if (dims[ndim - 1] % be != 0 || (size_t)(numel / be * bb) != nbytes) { set_error("byte size does not match dtype and shape"); return SP_ERR_SHAPE; }
    std::vector<uint8_t> sh;
    std::vector<int64_t> sd;
    bool sharded = false;
    const int st = tp_shard_tensor(hf_name, dtype, dims, ndim, (const uint8_t*)bytes, rank, size, vocab, sh, sd, sharded);
    if (st != SP_OK) return st;
    for (int i = 0; i < ndim; ++i) out_dims[i] = sd[i];
    *out_bytes = sharded ? sh.size() : nbytes;
    if (out) {
        if (out_cap < *out_bytes) { set_error("tp_shard: output buffer too small"); return SP_ERR_ARG; }
        std::memcpy(out, sharded ? sh.data() : (const uint8_t*)bytes, *out_bytes);
    }
    return SP_OK;
    API_END
}

static std::atomic<int> g_tc5{2};  // op-level matmuls of 17 rows and more: 2 tcgen05 GEMM with exact-class operands (default), 1 fp16 operands, 0 integer passes

int32_t sp_cuda_set_large_m_gemm(int32_t on) {
    if (on < 0 || on > 2) { set_error("large-M mode must be 0, 1 or 2"); return SP_ERR_ARG; }
    g_tc5.store(on);
    return SP_OK;
}

int32_t sp_cuda_set_activation_digits(int32_t mode) {
    if (mode < 0 || mode > 1) { set_error("activation digit mode must be 0 or 1"); return SP_ERR_ARG; }
    imma_set_digit_mode(mode);
    return SP_OK;
}

int32_t sp_cuda_set_gemv_path(int32_t path) {
    if (path < 0 || path > 4) { set_error("gemv path must be 0..4"); return SP_ERR_ARG; }
    g_gemv_path.store(path == 1 ? 1 : 0);
    g_rows.store(path == 2 ? 0 : 1);
    g_ring.store(path == 4 ? 1 : 0);
    imma_select_kernel(path == 3 ? 3 : 0);
    return SP_OK;
}

int32_t sp_cuda_upload_weight(int32_t device, int32_t dtype, int64_t n, int64_t k, const void* host_blocks, size_t nbytes,
                              SpWeight** out) {
    API_BEGIN
    if (!host_blocks || !out) { set_error("null argument"); return SP_ERR_ARG; }
    int st = check_weight_shape(dtype, n, k, nbytes);
    if (st != SP_OK) return st;
    SP_CUDA_TRY(cudaSetDevice(device));
    SpWeight* w = new SpWeight{device, dtype, n, k, nullptr, nbytes};
    cudaError_t ce = cudaMalloc((void**)&w->d, nbytes + 16);
    if (ce == cudaSuccess) ce = cudaMemcpy(w->d, host_blocks, nbytes, cudaMemcpyHostToDevice);
    if (ce == cudaSuccess && imma_supported(dtype, k) && n > 0) {
        ce = cudaMalloc((void**)&w->tiled, imma_tiled_bytes(dtype, n, k) + 16);
        if (ce == cudaSuccess) ce = launch_repack(dtype, w->d, n, k, w->tiled, 0);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(0);
        if (ce == cudaSuccess) ce = w->ws.alloc((int)k);
        if (ce == cudaSuccess) ce = ring_device_init();
        if (ce == cudaSuccess) ce = w->ring.alloc((int)((n + 15) / 16));
        if (ce == cudaSuccess) ce = w->rows.alloc();
    }
    if (ce != cudaSuccess) {
        set_error(std::string("upload_weight: ") + cudaGetErrorString(ce));
        if (w->d) cudaFree(w->d);
        if (w->tiled) cudaFree(w->tiled);
        w->ws.release();
        w->ring.release();
        w->rows.release();
        delete w;
        return ce == cudaErrorMemoryAllocation ? SP_ERR_OOM : SP_ERR_CUDA;
    }
    *out = w;
    return SP_OK;
    API_END
}

void sp_cuda_free_weight(SpWeight* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    cudaFree(w->d);
    if (w->tiled) cudaFree(w->tiled);
    w->ws.release();
    w->ring.release();
    w->rows.release();
    delete w;
}

int32_t sp_cuda_weight_info(const SpWeight* w, int32_t* dtype, int64_t* n, int64_t* k, size_t* nbytes) {
    if (!w) { set_error("null weight"); return SP_ERR_ARG; }
    if (dtype) *dtype = w->dtype;
    if (n) *n = w->n;
    if (k) *k = w->k;
    if (nbytes) *nbytes = w->nbytes;
    return SP_OK;
}

int32_t sp_cuda_dequant(const SpWeight* w, float* out_host) {
    API_BEGIN
    if (!w || !out_host) { set_error("null argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(w->device));
    DevBuf o;
    SP_CUDA_TRY(o.alloc((size_t)(w->n * w->k) * 4));
    SP_CUDA_TRY(launch_dequant(w->dtype, w->d, w->n, w->k, o.as<float>(), 0));
    SP_CUDA_TRY(cudaMemcpy(out_host, o.p, (size_t)(w->n * w->k) * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
    API_END
}

int32_t sp_cuda_matmul_nt_dev(const SpWeight* w, const float* x_dev, int64_t m, float* y_dev, void* stream) {
    API_BEGIN
    if (!w || !x_dev || !y_dev || m < 0) { set_error("null argument"); return SP_ERR_ARG; }
    if (((uintptr_t)x_dev & 15) != 0) { set_error("x must be 16-byte aligned"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(w->device));
    if (w->tiled && g_gemv_path.load() == 0 && g_tc5.load() && m >= TC5_MIN_M && tc5_supported(w->dtype, w->k)) {
        SpWeight* wm = const_cast<SpWeight*>(w);
        const bool exact = g_tc5.load() == 2;
        SP_CUDA_TRY(wm->ws.ensure_xh((size_t)m * w->k * (exact ? 2 : 1)));
        if (exact && m > ActWorkspace::XSCALE_ROWS) { set_error("matmul: more than 4096 rows in the exact tensor-core mode"); return SP_ERR_SHAPE; }
        if (exact) SP_CUDA_TRY(launch_x_to_f16_hilo(x_dev, (int)w->k, (int)m, (int)w->k, wm->ws.xh, wm->ws.xscale, (cudaStream_t)stream));
        else SP_CUDA_TRY(launch_x_to_f16(x_dev, (int)w->k, (int)m, (int)w->k, wm->ws.xh, (cudaStream_t)stream));
        SP_CUDA_TRY(launch_gemm_tc5(w->tiled, w->dtype, (int)w->n, (int)w->k, wm->ws.xh, (int)m, y_dev, (int)w->n, nullptr, nullptr, 0,
                                    (cudaStream_t)stream, &wm->ws.tc5, exact ? wm->ws.xscale : nullptr));
        return SP_OK;
    }
    if (w->tiled && g_gemv_path.load() == 0 && g_ring.load() && m >= 1 && m <= RING_MAX_M) {
        RingArgs ra{};
        ra.nseg = 1;
        ra.seg[0].wt = w->tiled; ra.seg[0].y = y_dev; ra.seg[0].dtype = w->dtype; ra.seg[0].n = (int)w->n; ra.seg[0].ldy = (int)w->n; ra.seg[0].bpt = 8;
        ra.k = (int)w->k; ra.m = (int)m; ra.src = RING_SRC_PLAIN; ra.x = x_dev; ra.ldx = (int)w->k;
        if (ring_plan(ra, w->ring)) {
            SP_CUDA_TRY(launch_gemv_ring(ra, (cudaStream_t)stream));
            return SP_OK;
        }
    }
    if (w->tiled && g_gemv_path.load() == 0 && g_rows.load() && m > imma_rows_per_pass() && rows_supported(w->dtype, w->k) &&
        (w->dtype != T_Q8_0 || imma_q8_bpt(w->k) == 8)) {
        // 11 rows and more: passes of up to 32 rows, each reading the weights once
        for (int64_t m0 = 0; m0 < m; m0 += IMMA_ROWS_MAX) {
            ImmaArgs ia{};
            ia.k = (int)w->k; ia.m = (int)std::min<int64_t>(IMMA_ROWS_MAX, m - m0); ia.nseg = 1;
            ia.seg[0].wt = w->tiled; ia.seg[0].y = y_dev + m0 * w->n; ia.seg[0].dtype = w->dtype; ia.seg[0].n = (int)w->n;
            ia.seg[0].ldy = (int)w->n; ia.seg[0].bpt = 8;
            imma_plan_rows(ia, w->ws);
            SP_CUDA_TRY(launch_act_quant(x_dev + m0 * w->k, (int)w->k, ia, (cudaStream_t)stream));
            SP_CUDA_TRY(launch_gemv_rows(ia, w->rows, (cudaStream_t)stream));
        }
        return SP_OK;
    }
    if (w->tiled && g_gemv_path.load() == 0) {
        const int pass = imma_rows_per_pass();
        for (int64_t m0 = 0; m0 < m; m0 += pass) {
            ImmaArgs ia{};
            ia.k = (int)w->k; ia.m = (int)std::min<int64_t>(pass, m - m0); ia.nseg = 1;
            ia.seg[0].wt = w->tiled; ia.seg[0].y = y_dev + m0 * w->n; ia.seg[0].dtype = w->dtype; ia.seg[0].n = (int)w->n;
            ia.seg[0].ldy = (int)w->n; ia.seg[0].bpt = imma_q8_bpt(w->k);
            SP_CUDA_TRY(launch_quant_gemv(x_dev + m0 * w->k, (int)w->k, ia, w->ws, true, (cudaStream_t)stream));
        }
        return SP_OK;
    }
    GemvArgs a{};
    a.x = x_dev; a.ldx = (int)w->k; a.m = (int)m; a.k = (int)w->k; a.nseg = 1;
    a.seg[0].w = w->d; a.seg[0].y = y_dev; a.seg[0].dtype = w->dtype; a.seg[0].n = (int)w->n; a.seg[0].ldy = (int)w->n;
    SP_CUDA_TRY(launch_gemv(a, (cudaStream_t)stream));
    return SP_OK;
    API_END
}

static int check_kernel_flags() {
    const int a = tc5_take_timeout(), b = imma_take_timeout();
    if (a < 0 || b < 0) { set_error("could not read the kernels' timeout flags"); return SP_ERR_CUDA; }
    if (a > 0) { set_error("tcgen05 GEMM: a bounded mbarrier wait expired, the outputs of that launch are not valid"); return SP_ERR_CUDA; }
    if (b > 0) { set_error("streaming GEMV: a bounded mbarrier wait expired, the outputs of that launch are not valid"); return SP_ERR_CUDA; }
    return SP_OK;
}

int32_t sp_cuda_check_kernels(int32_t device) {
    API_BEGIN
    SP_CUDA_TRY(cudaSetDevice(device));
    SP_CUDA_TRY(cudaDeviceSynchronize());
    return check_kernel_flags();
    API_END
}

int32_t sp_cuda_matmul_nt(const SpWeight* w, const float* x_host, int64_t m, float* y_host) {
    API_BEGIN
    if (!w || !x_host || !y_host || m < 0) { set_error("null argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(w->device));
    DevBuf x, y;
    SP_CUDA_TRY(x.alloc((size_t)(m * w->k) * 4));
    SP_CUDA_TRY(y.alloc((size_t)(m * w->n) * 4));
    SP_CUDA_TRY(cudaMemcpy(x.p, x_host, (size_t)(m * w->k) * 4, cudaMemcpyHostToDevice));
    int st = sp_cuda_matmul_nt_dev(w, x.as<float>(), m, y.as<float>(), nullptr);
    if (st != SP_OK) return st;
    SP_CUDA_TRY(cudaMemcpy(y_host, y.p, (size_t)(m * w->n) * 4, cudaMemcpyDeviceToHost));
    return check_kernel_flags();
    API_END
}

int32_t sp_cuda_rms_norm(int32_t device, const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y) {
    API_BEGIN
    if (!x || !y || rows < 0 || dim <= 0) { set_error("bad argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(device));
    DevBuf dx, dw, dy;
    SP_CUDA_TRY(dx.alloc((size_t)(rows * dim) * 4));
    SP_CUDA_TRY(dy.alloc((size_t)(rows * dim) * 4));
    SP_CUDA_TRY(cudaMemcpy(dx.p, x, (size_t)(rows * dim) * 4, cudaMemcpyHostToDevice));
    if (w) { SP_CUDA_TRY(dw.alloc((size_t)dim * 4)); SP_CUDA_TRY(cudaMemcpy(dw.p, w, (size_t)dim * 4, cudaMemcpyHostToDevice)); }
    SP_CUDA_TRY(launch_rms_norm(dx.as<float>(), w ? dw.as<float>() : nullptr, (int)rows, (int)dim, eps, dy.as<float>(), 0));
    SP_CUDA_TRY(cudaMemcpy(y, dy.p, (size_t)(rows * dim) * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
    API_END
}

int32_t sp_cuda_layer_norm(int32_t device, const float* x, const float* w, const float* b, int64_t rows, int64_t dim,
                           float eps, float* y) {
    API_BEGIN
    if (!x || !y || rows < 0 || dim <= 0) { set_error("bad argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(device));
    DevBuf dx, dw, db, dy;
    SP_CUDA_TRY(dx.alloc((size_t)(rows * dim) * 4));
    SP_CUDA_TRY(dy.alloc((size_t)(rows * dim) * 4));
    SP_CUDA_TRY(cudaMemcpy(dx.p, x, (size_t)(rows * dim) * 4, cudaMemcpyHostToDevice));
    if (w) { SP_CUDA_TRY(dw.alloc((size_t)dim * 4)); SP_CUDA_TRY(cudaMemcpy(dw.p, w, (size_t)dim * 4, cudaMemcpyHostToDevice)); }
    if (b) { SP_CUDA_TRY(db.alloc((size_t)dim * 4)); SP_CUDA_TRY(cudaMemcpy(db.p, b, (size_t)dim * 4, cudaMemcpyHostToDevice)); }
    SP_CUDA_TRY(launch_layer_norm(dx.as<float>(), w ? dw.as<float>() : nullptr, b ? db.as<float>() : nullptr, (int)rows, (int)dim,
                                  eps, dy.as<float>(), 0));
    SP_CUDA_TRY(cudaMemcpy(y, dy.p, (size_t)(rows * dim) * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
    API_END
}

int32_t sp_cuda_rope(int32_t device, const float* x, int64_t n_heads, int64_t seq, int64_t head_dim, const int64_t* positions,
                     float base, int64_t rotary_dim, float* y) {
    API_BEGIN
    if (!x || !y || !positions) { set_error("null argument"); return SP_ERR_ARG; }
    // error behaviour of crates/sapient-backends/cpu/src/kernels/rope.rs:98-108
    if (rotary_dim <= 0 || rotary_dim > head_dim) { set_error("rotary_dim must be in 1..=head_dim"); return SP_ERR_SHAPE; }
    if (rotary_dim % 2 != 0) { set_error("RoPE requires even rotary_dim"); return SP_ERR_SHAPE; }
    SP_CUDA_TRY(cudaSetDevice(device));
    // device layout is token-major [seq, n_heads*head_dim]; transpose on the host
    const size_t total = (size_t)(n_heads * seq * head_dim);
    std::vector<float> tm(total);
    for (int64_t h = 0; h < n_heads; ++h)
        for (int64_t s = 0; s < seq; ++s)
            std::memcpy(&tm[(size_t)((s * n_heads + h) * head_dim)], &x[(size_t)((h * seq + s) * head_dim)], (size_t)head_dim * 4);
    std::vector<float2> cs = rope_rows(positions, seq, base, rotary_dim);
    std::vector<int32_t> pos((size_t)seq);
    for (int64_t s = 0; s < seq; ++s) pos[(size_t)s] = (int32_t)s;  // row index into the per-call table
    DevBuf dx, dcs, dpos;
    SP_CUDA_TRY(dx.alloc(total * 4));
    SP_CUDA_TRY(dcs.alloc(cs.size() * sizeof(float2)));
    SP_CUDA_TRY(dpos.alloc((size_t)seq * 4));
    SP_CUDA_TRY(cudaMemcpy(dx.p, tm.data(), total * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dcs.p, cs.data(), cs.size() * sizeof(float2), cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dpos.p, pos.data(), (size_t)seq * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(launch_rope(dx.as<float>(), (int)seq, (int)n_heads, (int)head_dim, (int)rotary_dim, dcs.as<float2>(),
                            dpos.as<int32_t>(), (int)(n_heads * head_dim), 0));
    SP_CUDA_TRY(cudaMemcpy(tm.data(), dx.p, total * 4, cudaMemcpyDeviceToHost));
    for (int64_t h = 0; h < n_heads; ++h)
        for (int64_t s = 0; s < seq; ++s)
            std::memcpy(&y[(size_t)((h * seq + s) * head_dim)], &tm[(size_t)((s * n_heads + h) * head_dim)], (size_t)head_dim * 4);
    return SP_OK;
    API_END
}

int32_t sp_cuda_attention(int32_t device, const float* q, const float* k, const float* v, int64_t H, int64_t Hkv, int64_t sq,
                          int64_t sk, int64_t hd, float* out) {
    API_BEGIN
    if (!q || !k || !v || !out) { set_error("null argument"); return SP_ERR_ARG; }
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || hd <= 0 || hd % 2 != 0 || hd > 256 || sq <= 0 || sk < sq) {
        set_error("bad attention shape");
        return SP_ERR_SHAPE;
    }
    SP_CUDA_TRY(cudaSetDevice(device));
    // Build a one-slot paged fp16 cache holding k/v, with an identity page table.
    const int n_pages = (int)((sk + KV_PAGE - 1) / KV_PAGE);
    const size_t pool_halfs = (size_t)n_pages * 2 * Hkv * KV_PAGE * hd;
    std::vector<__half> pool(pool_halfs, __float2half_rn(0.f));
    for (int64_t h = 0; h < Hkv; ++h)
        for (int64_t s = 0; s < sk; ++s) {
            const int64_t pg = s / KV_PAGE, off = s % KV_PAGE;
            __half* kd = &pool[(size_t)((((pg * 2 + 0) * Hkv + h) * KV_PAGE + off) * hd)];
            __half* vd = &pool[(size_t)((((pg * 2 + 1) * Hkv + h) * KV_PAGE + off) * hd)];
            for (int64_t e = 0; e < hd; ++e) {
                kd[e] = __float2half_rn(k[(size_t)((h * sk + s) * hd + e)]);
                vd[e] = __float2half_rn(v[(size_t)((h * sk + s) * hd + e)]);
            }
        }
    std::vector<int32_t> pt((size_t)n_pages), slot((size_t)sq, 0), pos((size_t)sq);
    for (int i = 0; i < n_pages; ++i) pt[(size_t)i] = i;
    for (int64_t t = 0; t < sq; ++t) pos[(size_t)t] = (int32_t)(sk - sq + t);
    std::vector<float> qt((size_t)(sq * H * hd));
    for (int64_t h = 0; h < H; ++h)
        for (int64_t t = 0; t < sq; ++t)
            std::memcpy(&qt[(size_t)((t * H + h) * hd)], &q[(size_t)((h * sq + t) * hd)], (size_t)hd * 4);
    DevBuf dpool, dpt, dslot, dpos, dq, dout;
    SP_CUDA_TRY(dpool.alloc(pool_halfs * 2));
    SP_CUDA_TRY(dpt.alloc((size_t)n_pages * 4));
    SP_CUDA_TRY(dslot.alloc((size_t)sq * 4));
    SP_CUDA_TRY(dpos.alloc((size_t)sq * 4));
    SP_CUDA_TRY(dq.alloc(qt.size() * 4));
    SP_CUDA_TRY(dout.alloc(qt.size() * 4));
    SP_CUDA_TRY(cudaMemcpy(dpool.p, pool.data(), pool_halfs * 2, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dpt.p, pt.data(), (size_t)n_pages * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dslot.p, slot.data(), (size_t)sq * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dpos.p, pos.data(), (size_t)sq * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(cudaMemcpy(dq.p, qt.data(), qt.size() * 4, cudaMemcpyHostToDevice));
    KvGeom g{};
    g.pool = dpool.as<__half>(); g.page_table = dpt.as<int32_t>(); g.n_pages = n_pages; g.n_kv = (int)Hkv;
    g.head_dim = (int)hd; g.max_pages = n_pages;
    // decode-shaped calls split the keys over several blocks, like the engine does
    const int splits = sq <= 4 ? 8 : 1;
    DevBuf dscr;
    SP_CUDA_TRY(dscr.alloc(attention_scratch_floats((int)sq, (int)H, splits, (int)hd) * 4));
    SP_CUDA_TRY(launch_attention(dq.as<float>(), (int)(H * hd), dout.as<float>(), (int)(H * hd), (int)sq, (int)H,
                                 dslot.as<int32_t>(), dpos.as<int32_t>(), g, 0, 1.0f / sqrtf((float)hd), splits,
                                 dscr.as<float>(), 0, (int)sk));
    SP_CUDA_TRY(cudaMemcpy(qt.data(), dout.p, qt.size() * 4, cudaMemcpyDeviceToHost));
    for (int64_t h = 0; h < H; ++h)
        for (int64_t t = 0; t < sq; ++t)
            std::memcpy(&out[(size_t)((h * sq + t) * hd)], &qt[(size_t)((t * H + h) * hd)], (size_t)hd * 4);
    return SP_OK;
    API_END
}

int32_t sp_cuda_silu(int32_t device, const float* x, int64_t n, float* y) { API_BEGIN return unary_op(device, x, n, y, launch_silu); API_END }
int32_t sp_cuda_gelu(int32_t device, const float* x, int64_t n, float* y) { API_BEGIN return unary_op(device, x, n, y, launch_gelu); API_END }
int32_t sp_cuda_add(int32_t device, const float* a, const float* b, int64_t n, float* y) { API_BEGIN return binary_op(device, a, b, n, y, launch_add); API_END }
int32_t sp_cuda_mul(int32_t device, const float* a, const float* b, int64_t n, float* y) { API_BEGIN return binary_op(device, a, b, n, y, launch_mul); API_END }

int32_t sp_cuda_embed(const SpWeight* table, const uint32_t* ids, int64_t n, float* out_host) {
    API_BEGIN
    if (!table || !ids || !out_host || n < 0) { set_error("null argument"); return SP_ERR_ARG; }
    for (int64_t i = 0; i < n; ++i)
        if ((int64_t)ids[i] >= table->n) { set_error("token id " + std::to_string(ids[i]) + " out of vocab range"); return SP_ERR_VOCAB; }
    SP_CUDA_TRY(cudaSetDevice(table->device));
    DevBuf di, dout;
    SP_CUDA_TRY(di.alloc((size_t)n * 4));
    SP_CUDA_TRY(dout.alloc((size_t)(n * table->k) * 4));
    SP_CUDA_TRY(cudaMemcpy(di.p, ids, (size_t)n * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(launch_embed(table->dtype, table->d, table->k, di.as<uint32_t>(), (int)n, dout.as<float>(), 0));
    SP_CUDA_TRY(cudaMemcpy(out_host, dout.p, (size_t)(n * table->k) * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
    API_END
}

int32_t sp_cuda_argmax(int32_t device, const float* logits, int64_t rows, int64_t n, uint32_t* out) {
    API_BEGIN
    if (!logits || !out || rows < 0 || n <= 0) { set_error("bad argument"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(device));
    DevBuf dl, dout;
    SP_CUDA_TRY(dl.alloc((size_t)(rows * n) * 4));
    SP_CUDA_TRY(dout.alloc((size_t)rows * 4));
    SP_CUDA_TRY(cudaMemcpy(dl.p, logits, (size_t)(rows * n) * 4, cudaMemcpyHostToDevice));
    SP_CUDA_TRY(launch_argmax(dl.as<float>(), (int)rows, (int)n, (int)n, dout.as<uint32_t>(), 0));
    SP_CUDA_TRY(cudaMemcpy(out, dout.p, (size_t)rows * 4, cudaMemcpyDeviceToHost));
    return SP_OK;
    API_END
}

// ── engine ──────────────────────────────────────────────────────────────────
int32_t sp_cuda_engine_create(const SpModelDesc* desc, SpEngine** out) {
    API_BEGIN
    if (!desc || !out) { set_error("null argument"); return SP_ERR_ARG; }
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || desc->device < 0 || desc->device >= n) {
        cudaGetLastError();
        set_error("no such CUDA device");
        return SP_ERR_CUDA;
    }
    *out = new SpEngine{new Engine(*desc)};
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_set_tensor(SpEngine* e, const char* hf_name, int32_t dtype, const int64_t* dims, int32_t ndim,
                                  const void* host_bytes, size_t nbytes) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->set_tensor(hf_name, dtype, dims, ndim, host_bytes, nbytes);
    API_END
}

int32_t sp_cuda_engine_finalize(SpEngine* e) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->finalize();
    API_END
}

int32_t sp_cuda_engine_from_gguf(const char* path, int32_t device, int32_t max_ctx, int32_t max_batch, SpEngine** out) {
    API_BEGIN
    if (!path || !out) { set_error("null argument"); return SP_ERR_ARG; }
    Engine* eng = nullptr;
    int st = sp_engine_from_gguf_impl(path, device, max_ctx, max_batch, &eng);
    if (st != SP_OK) return st;
    *out = new SpEngine{eng};
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_desc(const SpEngine* e, SpModelDesc* out) {
    if (!e || !out) { set_error("null argument"); return SP_ERR_ARG; }
    *out = e->e->g;  // as given at creation (under tensor parallelism the engine works on its shard of it)
    return SP_OK;
}

void sp_cuda_engine_destroy(SpEngine* e) {
    if (!e) return;
    try { delete e->e; } catch (...) {}
    delete e;
}

int32_t sp_cuda_engine_set_stream(SpEngine* e, void* stream) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    e->e->stream = stream ? (cudaStream_t)stream : e->e->own_stream;
    return SP_OK;
}

int32_t sp_cuda_engine_set_trace(SpEngine* e, int32_t on) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    e->e->trace_on = on != 0;
    return SP_OK;
}

static int forward_slot(SpEngine* e, int slot, const uint32_t* ids, size_t n, bool all, float* out) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!ids || n == 0) { set_error("empty input"); return SP_ERR_ARG; }
    std::vector<int32_t> slots(n, slot);
    return e->e->forward(ids, slots.data(), (int64_t)n, all, out, nullptr);
}

int32_t sp_cuda_forward_logits(SpEngine* e, const uint32_t* ids, size_t n, int32_t use_cache, float* logits_out) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!ids || n == 0) { set_error("empty input"); return SP_ERR_ARG; }
    if (!use_cache) { int st = e->e->reset(0); if (st != SP_OK) return st; }
    return forward_slot(e, 0, ids, n, false, logits_out);
    API_END
}

int32_t sp_cuda_forward_all_logits(SpEngine* e, const uint32_t* ids, size_t n, float* out) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!ids || n == 0) { set_error("empty input"); return SP_ERR_ARG; }
    int st = e->e->reset(0);
    if (st != SP_OK) return st;
    return forward_slot(e, 0, ids, n, true, out);
    API_END
}

int32_t sp_cuda_forward_all_logits_cached(SpEngine* e, const uint32_t* ids, size_t n, float* out) {
    API_BEGIN
    return forward_slot(e, 0, ids, n, true, out);
    API_END
}

int32_t sp_cuda_forward_slot(SpEngine* e, int32_t slot, const uint32_t* ids, size_t n, int32_t all_positions, float* logits_out) {
    API_BEGIN
    return forward_slot(e, slot, ids, n, all_positions != 0, logits_out);
    API_END
}

int32_t sp_cuda_decode_batch(SpEngine* e, const uint32_t* ids, const int32_t* slots, int32_t b, float* logits_out,
                             uint32_t* argmax_out) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!ids || !slots || b <= 0) { set_error("empty input"); return SP_ERR_ARG; }
    for (int i = 0; i < b; ++i)
        for (int j = 0; j < i; ++j)
            if (slots[i] == slots[j]) { set_error("decode_batch: a slot appears twice"); return SP_ERR_ARG; }
    return e->e->forward(ids, slots, b, true, logits_out, argmax_out);
    API_END
}

int32_t sp_cuda_decode_greedy(SpEngine* e, const uint32_t* first_ids, const int32_t* slots, int32_t b, int32_t steps,
                              uint32_t* tokens_out) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->decode_greedy(first_ids, slots, b, steps, tokens_out);
    API_END
}

int32_t sp_cuda_spec_greedy(SpEngine* target, SpEngine* draft, const uint32_t* prompt, size_t n_prompt, int32_t k, size_t max_new,
                            const uint32_t* eos_ids, int32_t n_eos, uint32_t* tokens_out, size_t* n_out, uint64_t* stats) {
    API_BEGIN
    if (!target || !draft) { set_error("null engine"); return SP_ERR_ARG; }
    if (n_eos < 0 || (n_eos > 0 && !eos_ids)) { set_error("spec_greedy: bad eos list"); return SP_ERR_ARG; }
    return sp::spec_greedy(target->e, draft->e, prompt, n_prompt, k, max_new, eos_ids, n_eos, tokens_out, n_out, stats);
    API_END
}

int32_t sp_cuda_engine_slot_page(const SpEngine* e, int32_t slot, int32_t index, int32_t* page) {
    API_BEGIN
    if (!e || !page) { set_error("null argument"); return SP_ERR_ARG; }
    const Engine& en = *e->e;
    if (!en.finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    if (slot < 0 || slot >= en.d.max_batch || index < 0 || index >= en.pages.held[slot]) { set_error("slot or page index out of range"); return SP_ERR_ARG; }
    *page = en.pages.page_of(slot, index);
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_adopt_prefix(SpEngine* e, int32_t slot, const int32_t* pages, int32_t n) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!e->e->finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    return e->e->adopt_prefix(slot, pages, n);
    API_END
}

// ── continuous batching ──
struct SpBatcher {
    sp::SeqBackend* be;
    sp::Batcher* b;
    int device;  // -1: host stand-in
};

int32_t sp_cuda_batcher_create(SpEngine* e, int32_t prefill_chunk, int32_t prefix_cache, SpBatcher** out) {
    API_BEGIN
    if (!e || !out) { set_error("null argument"); return SP_ERR_ARG; }
    if (!e->e->finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    if (prefill_chunk < 1) { set_error("batcher: prefill_chunk must be positive"); return SP_ERR_ARG; }
    for (int s = 0; s < e->e->d.max_batch; ++s)
        if (e->e->seq_len[s] != 0) { set_error("batcher: the engine's caches must be empty"); return SP_ERR_STATE; }
    SpBatcher* h = new SpBatcher{sp::make_engine_backend(e->e), nullptr, e->e->d.device};
    h->b = new sp::Batcher(h->be, prefill_chunk, prefix_cache != 0);
    *out = h;
    return SP_OK;
    API_END
}

int32_t sp_cuda_batcher_create_selftest(int32_t vocab, int32_t max_slots, int32_t max_ctx, int32_t n_pages, int32_t prefill_chunk,
                                        int32_t prefix_cache, SpBatcher** out) {
    API_BEGIN
    if (!out || vocab < 2 || max_slots < 1 || max_ctx < 2 || n_pages < 1 || prefill_chunk < 1) { set_error("bad argument"); return SP_ERR_ARG; }
    SpBatcher* h = new SpBatcher{sp::make_mock_backend(vocab, max_slots, max_ctx, n_pages), nullptr, -1};
    h->b = new sp::Batcher(h->be, prefill_chunk, prefix_cache != 0);
    *out = h;
    return SP_OK;
    API_END
}

void sp_cuda_batcher_destroy(SpBatcher* b) {
    if (!b) return;
    try {
        if (b->device >= 0) cudaSetDevice(b->device);
        delete b->b;
        delete b->be;
        delete b;
    } catch (...) {
    }
}

int32_t sp_cuda_batcher_submit(SpBatcher* b, const uint32_t* prompt, size_t n, size_t max_new, const uint32_t* eos_ids, int32_t n_eos,
                               uint64_t* id) {
    API_BEGIN
    if (!b) { set_error("null batcher"); return SP_ERR_ARG; }
    return b->b->submit(prompt, n, max_new, eos_ids, n_eos, id);
    API_END
}

int32_t sp_cuda_batcher_step(SpBatcher* b, int32_t* n_running, int32_t* n_waiting) {
    API_BEGIN
    if (!b) { set_error("null batcher"); return SP_ERR_ARG; }
    int r = 0, w = 0;
    const int st = b->b->step(&r, &w);
    if (n_running) *n_running = r;
    if (n_waiting) *n_waiting = w;
    return st;
    API_END
}

int32_t sp_cuda_batcher_poll(const SpBatcher* b, uint64_t id, uint32_t* tokens_out, size_t cap, size_t* n_tokens, int32_t* finished) {
    API_BEGIN
    if (!b) { set_error("null batcher"); return SP_ERR_ARG; }
    int fin = 0;
    const int st = b->b->poll(id, tokens_out, cap, n_tokens, &fin);
    if (finished) *finished = fin;
    return st;
    API_END
}

int32_t sp_cuda_batcher_cancel(SpBatcher* b, uint64_t id) {
    API_BEGIN
    if (!b) { set_error("null batcher"); return SP_ERR_ARG; }
    return b->b->cancel(id);
    API_END
}

int32_t sp_cuda_batcher_forget(SpBatcher* b, uint64_t id) {
    API_BEGIN
    if (!b) { set_error("null batcher"); return SP_ERR_ARG; }
    return b->b->forget(id);
    API_END
}

int32_t sp_cuda_batcher_stats(const SpBatcher* b, uint64_t* out, int32_t cap) {
    API_BEGIN
    if (!b || !out || cap < 1) { set_error("null argument"); return SP_ERR_ARG; }
    const sp::BatcherStats& s = b->b->stats();
    const uint64_t v[SP_BATCHER_STATS] = {s.submitted, s.finished, s.steps, s.prefill_tokens, s.shared_tokens, s.decode_tokens, s.evicted_pages,
                                          s.cached_pages, (uint64_t)b->be->pool().available()};
    for (int i = 0; i < cap && i < SP_BATCHER_STATS; ++i) out[i] = v[i];
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_synchronize(SpEngine* e) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(e->e->d.device));
    SP_CUDA_TRY(cudaStreamSynchronize(e->e->stream));
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_set_graphs(SpEngine* e, int32_t on) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    e->e->use_graphs = on != 0;
    return SP_OK;
}

int32_t sp_cuda_engine_load_stats(const SpEngine* e, double* seconds, uint64_t* bytes) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (seconds) *seconds = e->e->load_seconds;
    if (bytes) *bytes = e->e->load_bytes;
    return SP_OK;
}

int32_t sp_cuda_nccl_unique_id(const char* libnccl_path, void* out, size_t cap) {
    API_BEGIN
    return sp::nccl_unique_id(libnccl_path, out, cap);
    API_END
}

int32_t sp_cuda_engine_tp_nccl_init(SpEngine* e, const char* libnccl_path, const void* unique_id) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_nccl_init(libnccl_path, unique_id);
    API_END
}

int32_t sp_cuda_engine_tp_set_allreduce(SpEngine* e, int32_t mode) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_set_allreduce(mode);
    API_END
}

int32_t sp_cuda_engine_tp_set_wait_ms(SpEngine* e, int32_t ms) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_set_wait_ms(ms);
    API_END
}

int32_t sp_cuda_engine_tp_reset(SpEngine* e) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->tp_reset();
    API_END
}

int32_t sp_cuda_engine_set_large_m_gemm(SpEngine* e, int32_t on) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(e->e->d.device));
    if (on < 0 || on > 2) { set_error("large-M mode must be 0, 1 or 2"); return SP_ERR_ARG; }
    e->e->use_tc5 = on != 0;
    e->e->tc5_exact = on == 2;
    e->e->drop_graphs();
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_set_many_row_gemv(SpEngine* e, int32_t on) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if ((on != 0) != e->e->use_rows) e->e->drop_graphs();
    e->e->use_rows = on != 0;
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_set_ring(SpEngine* e, int32_t on) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    SP_CUDA_TRY(cudaSetDevice(e->e->d.device));
    e->e->use_ring = on != 0;
    e->e->drop_graphs();  // captured steps hold the old kernel sequence
    return SP_OK;
    API_END
}

int32_t sp_cuda_engine_set_profile(SpEngine* e, int32_t on) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    e->e->profile_on = on != 0;
    return SP_OK;
}

int32_t sp_cuda_engine_time_families(SpEngine* e, uint32_t family_mask, int32_t n_tokens, int32_t reps, float* ms_per_step) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    return e->e->time_families(family_mask, n_tokens, reps, ms_per_step);
    API_END
}

int32_t sp_cuda_engine_profile_read(SpEngine* e, double* ms, uint64_t* launches, int32_t cap, int32_t reset) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    const int n = e->e->profile_read(ms, launches, cap);
    if (reset) e->e->profile_reset();
    return n;
}

int32_t sp_cuda_reset_cache(SpEngine* e, int32_t slot) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!e->e->finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    return e->e->reset(slot);
    API_END
}

int32_t sp_cuda_truncate_cache(SpEngine* e, int32_t slot, size_t n, size_t* kept) {
    API_BEGIN
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (!e->e->finalized) { set_error("engine not finalised"); return SP_ERR_STATE; }
    return e->e->truncate(slot, n, kept);
    API_END
}

int32_t sp_cuda_seq_len(const SpEngine* e, int32_t slot, size_t* len) {
    if (!e || !len || slot < 0 || slot >= e->e->d.max_batch) { set_error("bad argument"); return SP_ERR_ARG; }
    *len = (size_t)e->e->seq_len[slot];
    return SP_OK;
}

int32_t sp_cuda_backend_label(const SpEngine* e, char* buf, size_t cap) {
    if (!e || !buf || cap == 0) { set_error("bad argument"); return SP_ERR_ARG; }
    std::string s = "cuda";
    if (e->e->d.tp_size > 1) s += " (tp" + std::to_string(e->e->d.tp_size) + ")";
    std::strncpy(buf, s.c_str(), cap - 1);
    buf[cap - 1] = 0;
    return SP_OK;
}

int32_t sp_cuda_debug_layer_out(SpEngine* e, int32_t layer, float* out, size_t cap_floats, int32_t* n_tokens) {
    API_BEGIN
    if (!e || !out) { set_error("null argument"); return SP_ERR_ARG; }
    return e->e->debug_layer_out(layer, out, cap_floats, n_tokens);
    API_END
}

int32_t sp_cuda_engine_resident_bytes(const SpEngine* e, uint64_t* weights, uint64_t* kv) {
    if (!e) { set_error("null engine"); return SP_ERR_ARG; }
    if (weights) *weights = e->e->weight_bytes;
    if (kv) *kv = e->e->kv_bytes;
    return SP_OK;
}

}  // extern "C"
