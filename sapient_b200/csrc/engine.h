// Host-side resident engine: device weights in raw ggml block layout, a paged fp16 KV
// cache with per-slot page tables, and the per-layer launch sequence for Llama/Qwen
// and Phi-2 shaped decoders. Mirrors the contract of the reference's resident GPU
// engine (crates/sapient-models/src/forward/wgpu_engine.rs:93-110,173-341,362-676)
// behind ForwardEngine (crates/sapient-models/src/forward/mod.rs:381-506).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/sapient_cuda.h"
#include "kernels.h"
#include "page_pool.h"
#include "tp.cuh"

namespace sp {

void set_error(const std::string& msg);
const char* get_error();

#define SP_CUDA_TRY(expr)                                                                          \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess) {                                                                   \
            ::sp::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));                   \
            return _e == cudaErrorMemoryAllocation ? SP_ERR_OOM : SP_ERR_CUDA;                     \
        }                                                                                          \
    } while (0)

// The slice of a full tensor that rank `rank` of `size` keeps (tp.cu); sharded == false: the tensor is replicated.
int tp_shard_tensor(const std::string& name, int dtype, const int64_t* dims, int ndim, const uint8_t* bytes, int rank, int size,
                    int64_t vocab, std::vector<uint8_t>& out, std::vector<int64_t>& out_dims, bool& sharded);

struct DevTensor {
    int dtype = 0;
    std::vector<int64_t> dims;
    uint8_t* d = nullptr;      // raw ggml blocks (freed after repacking unless rows are gathered from it)
    size_t nbytes = 0;
    uint8_t* tiled = nullptr;  // tile-repacked copy for the tensor-core GEMV
    size_t tiled_bytes = 0;
    int64_t numel() const { int64_t n = 1; for (auto v : dims) n *= v; return n; }
};

struct LayerW {
    const float *n1w = nullptr, *n1b = nullptr, *n2w = nullptr;  // norm weights / bias as f32
    const DevTensor *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
    const DevTensor *gate = nullptr, *up = nullptr, *down = nullptr;  // Phi-2: up = fc1, down = fc2
    const float *qb = nullptr, *kb = nullptr, *vb = nullptr, *ob = nullptr, *upb = nullptr, *downb = nullptr;
};

class Engine {
  public:
    explicit Engine(const SpModelDesc& d);
    ~Engine();
    int set_tensor(const char* name, int dtype, const int64_t* dims, int ndim, const void* bytes, size_t nbytes);
    // The same with the rows of each head still in the GGUF llama order (row h*D + 2b + a holds HF row h*D + a*D/2 + b,
    // crates/sapient-models/src/gguf_weights.rs:98-154): unpermute_heads > 0 names the head count of this (full) tensor;
    // the rows are put in place by a device-side gather after the upload.
    int set_tensor_ex(const char* name, int dtype, const int64_t* dims, int ndim, const void* bytes, size_t nbytes, int unpermute_heads);
    // Seconds spent in host->device transfers of weights (pinned double-buffered staging) and bytes moved.
    double load_seconds = 0.0;
    uint64_t load_bytes = 0;
    int finalize();
    // Appends n tokens (ids[i] to slot slots[i]; consecutive entries of one slot take consecutive
    // positions). want_all: logits for every token, else only for the last token. Either output may be null.
    int forward(const uint32_t* ids, const int32_t* slots, int64_t n, bool want_all, float* logits_out,
                uint32_t* argmax_out);
    int reset(int slot);
    int truncate(int slot, size_t n, size_t* kept);
    int debug_layer_out(int layer, float* out, size_t cap, int32_t* n_tokens);
    // `steps` greedy decode steps for b slots with no host work in between: step 0 consumes first_ids, every
    // later step consumes the device-side argmax of the previous one. tokens_out[steps * b] (host) may be null.
    int decode_greedy(const uint32_t* first_ids, const int32_t* slots, int b, int steps, uint32_t* tokens_out);
    // Per-kernel-family device time of profiled forwards (ms, accumulated) and launch counts.
    enum Family { F_GEMV = 0, F_ATTN, F_NORM, F_ROPE, F_ELEM, F_EMBED, F_ARGMAX, F_COUNT };
    // Device time of one decode step of T tokens restricted to the kernel families in fam_mask (bit i = family i):
    // the step is captured with the other launches left out and replayed `reps` times between two events.
    // Activations and the KV entries of the last staged positions are undefined afterwards.
    int time_families(unsigned fam_mask, int T, int reps, float* ms_per_step);
    unsigned fam_mask = 0xFFFFFFFFu;
    int profile_read(double* ms, uint64_t* launches, int cap);
    void profile_reset();

    // Tensor parallelism (tp.cuh): d holds this rank's LOCAL head / ffn counts, g the description as given.
    int tp_handle(void* out, size_t cap);           // CUDA IPC handle of this rank's communication block
    int tp_connect(const void* handles, int n);     // map every rank's block (handles in rank order)
    int tp_connect_ptrs(void* const* blocks, int n); // the same for engines of ONE process: device pointers, no IPC
    void* tp_block() const { return tp_block_; }
    int tp_check();                                 // SP_ERR_COMM if a wait on a peer gave up
    int tp_set_wait_ms(int ms);                     // bound of the device-side waits on peers
    int tp_reset();                                 // counters, marks and the sticky flag back to the initial state
    // Comparison arm (nccl_arm.cu): the sums of the column-split products through ncclAllReduce instead of the fused push.
    int tp_nccl_init(const char* libpath, const void* unique_id);  // collective over the group
    int tp_set_allreduce(int mode);                 // 0: fused peer push (default); 1: library all-reduce
    // After a stream synchronise: SP_ERR_CUDA if a bounded mbarrier wait of one of this device's kernels ran out since
    // the last check (the kernel's outputs are then stale), else tp_check().
    int device_check();
    void drop_graphs();                             // forget the captured step graphs (a launch parameter changed)
    int vocab_local() const { return vocab_l_; }
    // Page bookkeeping of the KV cache (page_pool.h). The batching scheduler reads it to share prompt prefixes between
    // slots: adopt_prefix makes an EMPTY slot a reader of pages that already hold its first 16 * n tokens.
    PagePool pages;
    int adopt_prefix(int slot, const int32_t* page_ids, int n);

    SpModelDesc d, g;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    bool finalized = false;
    bool trace_on = false;
    bool use_graphs = true;
    // Steps of 11 rows and more that do not take the tcgen05 GEMM (11-16 rows, or use_tc5 off) as passes of up to 32 rows on
    // the one-pass kernel (gemv_rows.cu) instead of passes of 10 on the tile-row kernel. Off by default: inside a step the
    // two cost the same (32-row step of the 8B shape: 15.97 vs 15.50 ms) — the one-pass kernel reads the weights once but
    // launches per segment and cannot take digits written by the fused producers; as a stand-alone matmul it is 1.3x
    // faster (the op-level choice for 11-16 rows).
    bool use_rows = false;
    bool use_ring = false;     // steps of 1-5 rows on the bulk-copy ring GEMV (opt-in: measured slower than the tile-row kernels)
    // Steps of TC5_MIN_M rows and more (prompts, batches) run on the tcgen05 GEMM. tc5_exact (the default): its exact-class
    // mode — weights and activations each as a leading fp16 part plus remainder, three products per chunk of K, ~1e-6 per
    // product; activations are converted from their f32 rows, attention stays on the f32-class kernels. Full-size models
    // keep the 2e-2 final-logit bar in this mode (8B shape, 128-token prompt: 6.7e-3).
    // tc5_exact == false: operands rounded once to fp16 (~3e-4 per product; 2x faster; the 8B shape's logits then move by up
    // to 4e-2), with the fused fp16 producers and the fp16 prefill attention. use_tc5 == false: integer-digit GEMV passes of
    // 10 rows at any row count (7x slower on a 512-token prompt). sp_cuda_engine_set_large_m_gemm chooses.
    bool use_tc5 = true;
    bool tc5_exact = true;
    bool graph_step_ = false;  // a step is being captured: its kernels may take positions only from device memory
    // 1 (default): new K / V rows get the reference's Q8_0 cache rounding before they are stored as fp16 (head_dim % 32
    // == 0, where the reference keeps a Q8_0 cache); 0: plain fp16 rounding. Change only while the caches are empty.
    int kv_round = 1;
    bool profile_on = false;
    std::vector<int> seq_len;
    uint64_t weight_bytes = 0, kv_bytes = 0;

  private:
    int run_chunk(const uint32_t* ids, const int32_t* slots, int T, int rows_from, float* logits_out, uint32_t* argmax_out);
    int enqueue_layers(int T);                       // embed + all layers for the staged token table
    // final norm is done by the caller; lm_head + argmax of rc rows (pre: digits of those rows already in the workspace)
    int enqueue_head(int rows_from, int r0, int rc, const ImmaArgs* pre = nullptr);
    int enqueue_decode_step(int T);                  // embed, layers, final norm, lm_head, argmax for T <= logit_rows_ rows
    int launch_decode_step(int T);                   // the same through a cached CUDA graph when allowed
    void prof_begin(int fam);
    void prof_end(int fam);
    int alloc_pages(int slot, int new_len);
    const DevTensor* find(const std::string& name) const;
    const float* find_f32(const std::string& name, int64_t n);
    int layer_llama(const LayerW& w, int l, int T);
    int layer_phi(const LayerW& w, int l, int T);
    // tp_sum: the matrix is column-split over the ranks; y0 (= res) receives res + the sum of all ranks' products
    int gemv(const float* x, int ldx, int m, int k, const DevTensor* w0, const float* b0, float* y0, int ldy0,
             const DevTensor* w1 = nullptr, const float* b1 = nullptr, float* y1 = nullptr, const DevTensor* w2 = nullptr,
             const float* b2 = nullptr, float* y2 = nullptr, const float* res = nullptr, const ImmaArgs* pre = nullptr,
             bool tp_sum = false);
    // Many-row steps on one GPU: the producers (norm, attention, activation) write fp16 rows straight into the GEMM's
    // input buffer; big_m says whether these matrices take that path, gemm_xh multiplies what the buffer holds.
    // Steps of 1-4 rows on one GPU: the persistent ring GEMV (gemv_ring.cu) with the preceding norm / activation applied
    // inside it. SP_OK with *done = true when it was launched, *done = false when the launch does not qualify (the
    // caller then takes the tile-row kernel and its separate producers).
    int try_ring(bool* done, int m, int k, int src, const float* x, int ldx, const float* nw, const float* nb, const DevTensor* w0,
                 const float* b0, float* y0, int ldy, const DevTensor* w1 = nullptr, const float* b1 = nullptr, float* y1 = nullptr,
                 const DevTensor* w2 = nullptr, const float* b2 = nullptr, float* y2 = nullptr, const float* res = nullptr);
    RingScratch ring_;
    RowsScratch rows_;         // K-split partials of the one-pass many-row GEMV
    bool big_m(int m, int k, const DevTensor* w0, const DevTensor* w1 = nullptr, const DevTensor* w2 = nullptr) const;
    int gemm_xh(int m, int k, const DevTensor* w0, const float* b0, float* y0, int ldy0, const DevTensor* w1 = nullptr,
                const float* b1 = nullptr, float* y1 = nullptr, const DevTensor* w2 = nullptr, const float* b2 = nullptr,
                float* y2 = nullptr, const float* res = nullptr);
    // The same for a column-split matrix (o_proj, down_proj) whose product is added into the residual stream x_: on one
    // GPU in place; under tensor parallelism the partial product goes to scratch and is pushed to every rank.
    int gemm_xh_sum(int m, int k, const DevTensor* w, const float* b);
    size_t tp_block_bytes() const;
    int tp_alloc();
    void tp_release();
    uint8_t* tp_block_ = nullptr;   // this rank's communication block
    uint8_t* tp_state_ = nullptr;   // sequence counters, block counter, timeout flag
    TpDev* d_tp_ = nullptr;         // device copy of the peer table
    uint8_t* tp_peer_[TP_MAX_RANKS] = {};
    bool tp_connected_ = false;
    void* nccl_comm_ = nullptr;
    bool tp_use_nccl_ = false;
    int nccl_all_reduce(float* buf, size_t count);
    void tp_nccl_release();
    uint64_t tp_wait_ns_ = TP_WAIT_NS_DEFAULT;
    bool tp_pending_ = false;       // partial rows have been pushed, x_ still lacks their sum
    // decode_greedy returned without waiting (tokens_out == null): copies out of the pinned staging buffers may still be
    // queued on the stream. Every call that rewrites those buffers drains the stream first.
    bool async_pending_ = false;
    int drain_async();
    const TpDev* tp_take() { const TpDev* t = tp_pending_ ? d_tp_ : nullptr; tp_pending_ = false; return t; }
    int tp_resolve(int T);          // stand-alone consumer when the next kernel is not the fused norm
    int vocab_l_ = 0, vocab_off_ = 0;
    DevTensor head_view_;           // lm_head restricted to the rows this engine computes
    bool plan_digits(int m, int k, ImmaArgs& ia);
    int attention_and_oproj(const LayerW& w, int l, int T);

    // Weight upload: two pinned staging buffers, copies enqueued on a dedicated stream; the host fills one buffer while the
    // other is in flight. Released at finalize.
    static constexpr size_t STAGE_BYTES = 32u << 20;
    uint8_t* stage_[2] = {nullptr, nullptr};
    cudaEvent_t stage_ev_[2] = {nullptr, nullptr};
    cudaStream_t load_stream_ = nullptr;
    int stage_next_ = 0;
    int upload_staged(uint8_t* dst, const uint8_t* src, size_t nbytes);
    void release_staging();
    std::map<std::string, DevTensor> tensors_;
    std::vector<void*> owned_;  // extra device allocations (converted biases, ...)
    std::vector<LayerW> layers_;
    const DevTensor *embed_ = nullptr, *lm_head_ = nullptr;
    const float *final_w_ = nullptr, *final_b_ = nullptr;
    const float* lm_bias_ = nullptr;

    ActWorkspace ws_;          // activation digits of the current GEMV input
    // split-K attention: steps of up to 16 rows split the keys over up to ATT_SPLITS blocks (scratch sized for ATT_SPLIT_TOKENS rows)
    static constexpr int ATT_SPLITS = 16, ATT_SPLIT_TOKENS = 32;
    float* att_scratch_ = nullptr;
    int repack_weights();

    // paged KV cache
    KvGeom kv_{};
    int32_t* d_page_table_ = nullptr;
    int sync_page_table();        // uploads the host page table when it changed
    int privatise_tail(int slot); // copy-on-write of a shared, partly filled last page before the slot appends

    // activations (sized for max_tokens)
    float *x_ = nullptr, *h_ = nullptr, *qkv_ = nullptr, *attn_ = nullptr, *gu_ = nullptr, *mid_ = nullptr, *sel_ = nullptr,
          *logits_ = nullptr, *trace_ = nullptr;
    uint32_t *d_ids_ = nullptr, *d_argmax_ = nullptr;
    void* argmax_scratch_ = nullptr;  // candidates and arrival counters of the multi-block arg-max
    int32_t *d_tok_slot_ = nullptr, *d_tok_pos_ = nullptr;
    float2* cos_sin_ = nullptr;
    int trace_tokens_ = 0;
    int logit_rows_ = 32;  // rows of the lm_head GEMV per pass
    // pinned staging
    uint32_t* p_ids_ = nullptr;
    int32_t *p_slot_ = nullptr, *p_pos_ = nullptr;
    float* p_logits_ = nullptr;
    uint32_t* p_argmax_ = nullptr;
    // device-resident greedy loop
    uint32_t* d_tokens_ = nullptr;
    size_t d_tokens_cap_ = 0;
    // CUDA graphs of one decode step, keyed by token count
    // keyed by (rows, attention split count): the split count follows the longest context of the step, see step_splits()
    std::map<int, cudaGraphExec_t> step_graphs_;
    std::map<int, int64_t> step_graph_kernels_;
    int step_ctx_ = 0;            // upper bound of the longest context among the staged tokens (host-side knowledge)
    int step_splits(int T) const; // key ranges per (token, head) of the decode-shaped attention
    // profiling: event pairs per launch, resolved after a synchronise
    struct ProfRec { int fam; cudaEvent_t a, b; };
    std::vector<ProfRec> prof_recs_;
    std::vector<cudaEvent_t> prof_pool_;
    double prof_ms_[F_COUNT] = {0};
    uint64_t prof_n_[F_COUNT] = {0};
    int prof_flush();
};

}  // namespace sp
