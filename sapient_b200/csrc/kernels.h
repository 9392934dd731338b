// Launch wrappers of the sm_100a kernels (definitions in kernels.cu). All pointers are
// device pointers; every launcher enqueues on `st` and returns cudaGetLastError().
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemv_imma.cuh"

namespace sp {

// One weight matrix of a grouped dequant-GEMV: rows [N, K] of raw ggml blocks.
struct GemvSeg {
    const uint8_t* w;   // raw blocks, row-major
    const float* bias;  // [n] or null
    float* y;           // output base; element (m, r) at y[m * ldy + r]
    int dtype;
    int n;
    int ldy;
    int pad_;
};

struct GemvArgs {
    GemvSeg seg[3];
    int nseg;
    int k;
    int m;
    int ldx;
    const float* x;     // [m, k], row stride ldx
    const float* res;   // optional residual added to segment 0's output (same indexing as y), may alias y
    int ldres;
    int pad_;
};

// Paged KV cache geometry: half pool[layer][page][2 (K,V)][n_kv][KV_PAGE][head_dim].
struct KvGeom {
    __half* pool;
    const int32_t* page_table;  // [n_slots, max_pages]
    int n_pages, n_kv, head_dim, max_pages;
};

// Kernels launched by this library since process start.
uint64_t launch_count();
// Graph replays launch kernels without passing through the launchers; they report their node count here.
void adjust_launch_count(int64_t delta);

// Tensor-core GEMV on tile-repacked weights (gemv_imma.cu).
bool imma_supported(int dtype, int64_t k);
size_t imma_tiled_bytes(int dtype, int64_t n, int64_t k);
int imma_q8_bpt(int64_t k);
cudaError_t launch_repack(int dtype, const uint8_t* raw, int64_t n, int64_t k, uint8_t* tiled, cudaStream_t st);
struct ActWorkspace;
// Fills digits / ncp / eb / kp and the table pointers of `a` from a.m, a.k and the workspace.
void imma_plan(ImmaArgs& a, const ActWorkspace& ws);
cudaError_t launch_act_quant(const float* x, int ldx, const ImmaArgs& a, cudaStream_t st);
cudaError_t launch_gemv_imma(const ImmaArgs& a, cudaStream_t st);
// 0: the one-CTA-per-tile-row kernel; 3: the persistent TMA-streaming kernel when k % 256 == 0 and the digits fit
// shared memory.
void imma_select_kernel(int which);
// Activation precision of the tensor-core GEMV passes (process-wide): 0 = 3 digits for 1-2 rows, 2 digits (16 rows per
// pass) above; 1 = 3 digits always (10 rows per pass). imma_rows_per_pass() is the pass size that follows.
void imma_set_digit_mode(int mode);
int imma_rows_per_pass();
// Bounded device-side waits (mbarrier waits of the streaming GEMV and of the tcgen05 GEMM) raise a per-device flag when
// they run out. These read and clear it on the current device: 1 = expired since the last call, 0 = none, -1 = CUDA error.
int imma_take_timeout();
int tc5_take_timeout();
// ── Persistent ring GEMV for steps of 1-5 rows (gemv_ring.cu) ──
// Where the activations of a launch come from: f32 rows as they are, or through the operation that precedes the matrix
// in the layer, applied by every CTA on its own copy.
enum RingSrc : int { RING_SRC_PLAIN = 0, RING_SRC_RMS = 1, RING_SRC_LN = 2, RING_SRC_SWIGLU = 3, RING_SRC_GELU = 4 };
constexpr int RING_MAX_STAGES = 6;
constexpr int RING_MAX_M = 5;  // activation rows per launch: three digit columns each, two 8-column n-tiles
// Scratch of tile rows shared between CTAs: two 16 x 5 partial blocks per CTA and one arrival counter per tile row of
// the largest launch. Launches that may overlap on the device must not share one (one per engine / op-level weight).
struct RingScratch {
    float* part = nullptr;
    unsigned* cnt = nullptr;   // zero between launches
    int rows_cap = 0, ctas_cap = 0;
    cudaError_t alloc(int max_rows);  // on the current device; not during stream capture
    void release();
};
struct RingArgs {
    ImmaSeg seg[3];       // wt, bias, y, dtype, n, ldy of up to three matrices sharing the activations (bpt unused: 8)
    int nseg;
    int k, m;             // k % 256 == 0, 1 <= m <= RING_MAX_M
    int src;              // RingSrc
    const float* x;       // [m][ldx] f32; SWIGLU: gate at column 0 and up at column k of each row; GELU: fc1 output
    int ldx;
    const float* nw;      // norm weight [k] (RMS, LN)
    const float* nb;      // LayerNorm bias [k] or null
    float eps;
    const float* res;     // residual added to segment 0 (may alias its y) or null
    int ldres;
    // filled by ring_plan:
    int digits, kt, total_tiles;
    int seg_tile0[4], seg_row0[4];
    int stage_bytes, stages, smem_total;
    int cw, fmt;          // consumer warps of the instance; its single weight format (0: mixed)
    int off_bar, off_flush, off_cs, off_rec32, off_rec16, off_xq, off_stage;
    float* fix_part;
    unsigned* fix_cnt;
    int* err;
};
// One-time per-device set-up of the ring kernel's error flag (host-mapped memory): call before the first launch on a
// device, outside stream capture (engine finalize and weight upload do).
cudaError_t ring_device_init();
// share_sm: size the ring so that two CTAs fit an SM (this kernel's and the next kernel's prologue under programmatic
// dependent launch). False when the launch cannot use this kernel (shape, formats, shared memory, scratch size).
bool ring_plan(RingArgs& a, const RingScratch& sc, bool share_sm = false);
cudaError_t launch_gemv_ring(RingArgs& a, cudaStream_t st);

// Producers that emit the digits of a GEMV input directly (a: planned ImmaArgs; a.m rows, a.k columns):
// RMSNorm / LayerNorm of x (y optional f32 copy), SwiGLU (act 0) / tanh-GELU (act 1) of gu, merged split-K attention.
// tp != null: x first receives the pending tensor-parallel sum (tp.cuh), in place.
cudaError_t launch_norm_quant(const float* x, int ldx, const float* w, const float* b, bool layer_norm, float eps, float* y, int ldy,
                              const ImmaArgs& a, cudaStream_t st, const struct TpDev* tp = nullptr);
cudaError_t launch_act_fn_quant(const float* gu, int ld, int ffn, int act, const ImmaArgs& a, cudaStream_t st);
cudaError_t launch_attn_merge_quant(const float* part, int n_heads, int n_splits, int hd, float* out, int ldo, const ImmaArgs& a,
                                    cudaStream_t st);
// Whether a decode-shaped launch with these sizes runs on the tensor-core grouped-query kernel (ctx_hint as for
// launch_attention): callers choose the split count accordingly — that kernel wants few, long key ranges.
bool attention_takes_mma(int n_tok, int ctx_hint, int n_heads, int n_kv, int head_dim);
// The split phase of launch_attention alone (partials to scratch); n_splits > 1.
cudaError_t launch_attention_split(const float* q, int ldq, int n_tok, int n_heads, const int32_t* tok_slot, const int32_t* tok_pos,
                                   KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st, int ctx_hint = 0);

// Prefill attention on tensor cores: n_tok tokens of one sequence at consecutive positions pos0.. (keys already cached).
bool attention_prefill_supported(int head_dim);
cudaError_t launch_attention_prefill(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, int slot, int pos0, KvGeom kv,
                                     int layer, float scale, cudaStream_t st, __half* out_h = nullptr);

// Scratch of the GEMM's split last wave: one 256 x 128 f32 partial tile per CTA of that wave (at most one per SM:
// 19 MB on a 148-SM device) and one arrival counter per shared work item. Owned by whoever owns the stream the launches
// go to (an engine, an op-level weight): launches that may overlap on the device must not share one. Without scratch the
// last wave is not split.
constexpr int TC5_SPLIT_MAX_ITEMS = 256;
struct Tc5Scratch {
    float* buf = nullptr;
    unsigned* cnt = nullptr;   // zero between launches
    size_t parts_cap = 0;      // partial tiles buf holds
    cudaError_t alloc();       // on the current device; not during stream capture
    void release();
};
// Workspace of the activation digits for up to 16 activation rows of k_max columns.
struct ActWorkspace {
    int8_t* xq = nullptr;
    float* colscale = nullptr;
    int8_t* xs32d = nullptr;
    int8_t* xs16d = nullptr;
    int k_max = 0;
    __half* xh = nullptr;      // fp16 copy of the activations for the large-M tensor-core GEMM (gemm_tc5.cu)
    size_t xh_elems = 0;
    float* xscale = nullptr;   // per-row power-of-two scales of the exact mode's activations (same allocation as xh)
    static constexpr int XSCALE_ROWS = 4096;
    Tc5Scratch tc5;            // allocated with xh
    cudaError_t ensure_xh(size_t elems);  // grows the buffer (allocates: not during stream capture)
    static constexpr int NCP_MAX = 96;  // digit columns: 32 rows x 3 digits (gemv_rows.cu); the tile-row kernel uses up to 32
    cudaError_t alloc(int k_max_);
    void release();
};
// Digits for x[m, k] (m <= 16) followed by the tensor-core GEMV over up to three weight segments sharing x.
// Fills a.digits/ncp/eb/xq/...; a.seg/nseg/k/m/res must be set by the caller.
cudaError_t launch_quant_gemv(const float* x, int ldx, ImmaArgs& a, const ActWorkspace& ws, bool requantize, cudaStream_t st);

// One-pass tensor-core GEMV for 11..32 activation rows (gemv_rows.cu): a CTA owns eight tile rows and shares the staged
// digits of each k-tile among its warps. `a` as for launch_gemv_imma with digits planned for a.m <= IMMA_ROWS_MAX rows
// (imma_plan_rows) and a.eb == 256; every segment Q4_K / Q6_K / Q8_0 with k % 256 == 0; not for tensor-parallel pushes.
constexpr int IMMA_ROWS_MAX = 32;
struct RowsScratch {
    float* part = nullptr;     // partial outputs of K-split launches
    unsigned* cnt = nullptr;   // arrival counters per 128-row group
    static constexpr int CNT_MAX = 2048;
    static size_t part_floats();
    cudaError_t alloc();
    void release();
};
bool rows_supported(int dtype, int64_t k);
void imma_plan_rows(ImmaArgs& a, const ActWorkspace& ws);  // three digits, 32-column groups (a.m <= IMMA_ROWS_MAX)
cudaError_t launch_gemv_rows(const ImmaArgs& a, const RowsScratch& sc, cudaStream_t st);

// Large-M dequant GEMM on tcgen05 / TMEM (gemm_tc5.cu): y[m, n] = x·Wᵀ (+ bias, + res) from the tiled weights and an
// fp16 copy of the activations; k % 256 == 0, Q4_K / Q6_K / Q8_0.
constexpr int TC5_MIN_M = 17;  // up to 16 rows one GEMV pass is faster; from 17 rows on (two passes) the tcgen05 GEMM wins (measured at 32 rows: 5.6 vs 7.1 ms per decode step of the 8B shape)
bool tc5_supported(int dtype, int64_t k);
cudaError_t launch_x_to_f16(const float* x, int ldx, int m, int k, __half* out, cudaStream_t st);
// For the GEMM's exact mode: every row is scaled by a power of two to (-1, 1) first (rowscale[m] receives the inverse), so
// that the remainders stay inside the fp16 range whatever the row's magnitude; out[2 m][k]: rows 0..m-1 the fp16 leading
// parts, rows m..2m-1 the fp16 of what that rounding dropped.
cudaError_t launch_x_to_f16_hilo(const float* x, int ldx, int m, int k, __half* out, float* rowscale, cudaStream_t st);
cudaError_t launch_gemm_tc5(const uint8_t* wt, int dtype, int n, int k, const __half* xh, int m, float* y, int ldy, const float* bias,
                            const float* res, int ldres, cudaStream_t st, const Tc5Scratch* scratch = nullptr, const float* xscale = nullptr);
struct Tc5Seg {
    const uint8_t* wt;  // tiled weights
    float* y;           // output base: element (m, r) at y[m * ldy + r]
    const float* bias;  // [n] or null
    int dtype, n;       // format, rows
};
// Up to three matrices sharing the activations in ONE launch (q|k|v, gate|up); res is added to segment 0.
cudaError_t launch_gemm_tc5_multi(const Tc5Seg* segs, int nseg, int k, const __half* xh, int m, int ldy, const float* res, int ldres,
                                  cudaStream_t st, const Tc5Scratch* scratch = nullptr, const float* xscale = nullptr);
// xscale != null selects the exact mode: xh holds [2 m][k] as launch_x_to_f16_hilo writes it, xscale its row scales.

cudaError_t launch_dequant(int dtype, const uint8_t* w, int64_t n, int64_t k, float* out, cudaStream_t st);
cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t st);
cudaError_t launch_embed(int dtype, const uint8_t* table, int64_t hidden, const uint32_t* ids, int n_tok, float* out,
                         cudaStream_t st);
cudaError_t launch_rms_norm(const float* x, const float* w, int rows, int dim, float eps, float* y, cudaStream_t st);
cudaError_t launch_rms_norm_f16(const float* x, const float* w, int rows, int dim, float eps, __half* yh, cudaStream_t st);
cudaError_t launch_layer_norm_f16(const float* x, const float* w, const float* b, int rows, int dim, float eps, __half* yh,
                                  cudaStream_t st);
cudaError_t launch_act_f16(const float* gu, int ld, int ffn, int rows, int kind, __half* out, cudaStream_t st);
cudaError_t launch_layer_norm(const float* x, const float* w, const float* b, int rows, int dim, float eps, float* y,
                              cudaStream_t st);
// In-place NEOX rotation of the q heads of qkv[T, (H+2Hkv)*hd]; rotated k and raw v are
// written as fp16 into the paged cache at (slot, pos) of each token.
cudaError_t launch_rope_kv_append(float* qkv, int n_tok, int n_heads, int n_kv, int head_dim, int rotary_dim,
                                  const float2* cos_sin, const int32_t* tok_slot, const int32_t* tok_pos, KvGeom kv,
                                  int layer, int kv_round, cudaStream_t st);
// Rotation only (no cache): x[T, n_heads*hd] in place. Used by the standalone RoPE op.
cudaError_t launch_rope(float* x, int n_tok, int n_heads, int head_dim, int rotary_dim, const float2* cos_sin,
                        const int32_t* tok_pos, int ld, cudaStream_t st);
// Causal GQA attention of each token against keys 0..pos of its slot, online softmax, keys split over
// n_splits blocks per (head, token). n_splits > 1 needs `scratch` of attention_scratch_floats() floats.
size_t attention_scratch_floats(int n_tok, int n_heads, int n_splits, int head_dim);
// ctx_hint: upper bound of the longest context among the tokens (0: unknown); picks the kernel variant, not the result's meaning.
cudaError_t launch_attention(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                             const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch,
                             cudaStream_t st, int ctx_hint = 0);
cudaError_t launch_swiglu(const float* gate_up, int ld, int ffn, int rows, float* out, cudaStream_t st);
cudaError_t launch_gelu(float* x, int64_t n, cudaStream_t st);
cudaError_t launch_silu(float* x, int64_t n, cudaStream_t st);
cudaError_t launch_add(const float* a, const float* b, float* y, int64_t n, cudaStream_t st);
cudaError_t launch_mul(const float* a, const float* b, float* y, int64_t n, cudaStream_t st);
// Row-wise argmax with the reference's tie rule (the LAST maximum wins).
// scratch (optional, argmax_scratch_bytes() of zeroed device memory owned by the caller's stream): rows of 8192 columns
// and more are then scanned by ARGMAX_PARTS blocks each instead of one.
constexpr int ARGMAX_PARTS = 64, ARGMAX_MAX_ROWS = 64;
inline size_t argmax_scratch_bytes() { return (size_t)ARGMAX_MAX_ROWS * ARGMAX_PARTS * 8 + ARGMAX_MAX_ROWS * 4; }
cudaError_t launch_argmax(const float* logits, int rows, int n, int ld, uint32_t* out, cudaStream_t st, void* scratch = nullptr);
cudaError_t launch_gather_rows(const float* src, int ld, const int32_t* rows, int n_rows, int dim, float* dst,
                               cudaStream_t st);

}  // namespace sp
