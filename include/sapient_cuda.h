/* sapient_cuda.h — C ABI of the B200 (sm_100a) CUDA backend for sapient's quantized
 * decoder-LLM path. Plain pointers and sizes only; no exception crosses the boundary
 * (the reference's release profile aborts on panic: Cargo.toml:147-152).
 *
 * Every entry point returns an int32 status (SP_OK == 0). On failure
 * sp_cuda_last_error() returns a message for the calling thread.
 *
 * The reference items each entry replaces are cited as file:line within the
 * reference repository (SkidGod4444/sapient v0.6.0).
 *
 * Threading: an engine is not re-entrant (the reference wraps its engine in a
 * Mutex: crates/sapient-generate/src/pipeline.rs:144); calls may arrive on different
 * OS threads. Several engines may coexist in one process.
 */
#ifndef SAPIENT_CUDA_H
#define SAPIENT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (crates/sapient-core/src/error.rs:10-96 collapses onto these) */
enum {
    SP_OK = 0,
    SP_ERR_SHAPE = 1,    /* ShapeMismatch / k not a multiple of the block size */
    SP_ERR_DTYPE = 2,    /* unsupported dtype */
    SP_ERR_OOM = 3,      /* device allocation failed */
    SP_ERR_CUDA = 4,     /* a CUDA call failed */
    SP_ERR_KV_FULL = 5,  /* context window or page pool exhausted (wgpu_engine.rs:372-374) */
    SP_ERR_COMM = 6,     /* tensor-parallel exchange timed out */
    SP_ERR_ARG = 7,      /* null / empty / out-of-range argument */
    SP_ERR_VOCAB = 8,    /* token id out of vocab range (forward/common.rs:184-186) */
    SP_ERR_STATE = 9,    /* engine not finalised / missing weight */
    SP_ERR_IO = 10       /* GGUF file unreadable or malformed */
};

/* ggml tensor type codes (crates/sapient-io/src/gguf.rs:88-129) */
enum { SP_F32 = 0, SP_F16 = 1, SP_Q4_0 = 2, SP_Q8_0 = 8, SP_Q4_K = 12, SP_Q5_K = 13, SP_Q6_K = 14, SP_BF16 = 30 };

const char* sp_cuda_last_error(void);
/* number of visible CUDA devices, or 0 */
int32_t sp_cuda_device_count(void);

/* ── op level: replaces WgpuContext::{upload_q8_0,upload_q4_k,upload_q6_k,matmul_nt*}
 *    (crates/sapient-backends/wgpu/src/quant.rs:94-480) and kernels::matmul::matmul_nt
 *    (crates/sapient-backends/cpu/src/kernels/matmul.rs:114-145) ───────────────── */
typedef struct SpWeight SpWeight;

/* Copies a [n, k] matrix of raw ggml blocks (Tensor::as_quant_blocks layout,
 * crates/sapient-core/src/tensor.rs:261-268) to the device. nbytes must equal the
 * dtype's byte_count(n*k) (crates/sapient-core/src/dtype.rs:136-145); K-quants need
 * k % 256 == 0 and Q8_0 k % 32 == 0 (kernels/matmul.rs:576,863,1112). */
int32_t sp_cuda_upload_weight(int32_t device, int32_t dtype, int64_t n, int64_t k, const void* host_blocks,
                              size_t nbytes, SpWeight** out);
void sp_cuda_free_weight(SpWeight* w);
/* Tensor::to_f32_vec (crates/sapient-core/src/tensor.rs:341-498): bit-exact f32 values, n*k floats to host. */
int32_t sp_cuda_dequant(const SpWeight* w, float* out_host);
/* Y[m,n] = X[m,k] · Wᵀ, host buffers (copies inside). */
int32_t sp_cuda_matmul_nt(const SpWeight* w, const float* x_host, int64_t m, float* y_host);
/* Same with device buffers on `stream` (a cudaStream_t, or NULL for the default stream); the launches are not waited
 * for. The weight carries a private workspace (activation digits, and an fp16 copy of x for calls of 17 rows and
 * more), so calls on one SpWeight must be ordered on ONE stream and never run from two threads at once; use one
 * SpWeight per stream otherwise. The fp16 buffer grows on demand: the first call with a given (larger) m of 17 rows or
 * more frees and allocates device memory, which waits for all work of the device — issue one such call per weight at
 * set-up, before any stream capture. A bounded wait inside the 17+-row kernel that runs out leaves y stale; the
 * condition is reported (SP_ERR_CUDA) by the next call of this library that synchronises: sp_cuda_matmul_nt,
 * sp_cuda_check_kernels, or an engine call that returns host data. */
int32_t sp_cuda_matmul_nt_dev(const SpWeight* w, const float* x_dev, int64_t m, float* y_dev, void* stream);
/* Waits for all work of `device`, then reports (SP_ERR_CUDA, message in sp_cuda_last_error) whether a bounded wait
 * inside one of this library's kernels ran out on that device since the last check; the flag is cleared by the report.
 * The reference's GPU backend has no such condition to report (its wgpu queue has no device-side waits,
 * crates/sapient-backends/wgpu/src/context.rs); this is the error channel of the asynchronous device-pointer calls. */
int32_t sp_cuda_check_kernels(int32_t device);
/* Precision of the activations in the tensor-core GEMV passes. The reference multiplies f32 activations
 * (kernels/matmul.rs:862-943); this backend splits each activation into int8 digits with one power-of-two scale per 256
 * (Q8_0: 32) columns, so that the products with the integer weights are exact. 1 (default): three digits (2^-23 of the
 * block maximum) at every row count, 10 rows per pass. 0: three digits for steps of 1-2 rows, two digits (2^-15) and 16
 * rows per pass above — fewer passes for batched steps at ~1e-4 relative error per product. Process-wide; engines drop
 * their captured step graphs when it changes (sp_cuda_engine_set_graphs off/on). */
int32_t sp_cuda_set_activation_digits(int32_t mode);
/* Which GEMV kernel runs (process-wide; op-level calls — engines have sp_cuda_engine_set_ring):
 *   0 (default): the tensor-core GEMV — one CTA per 16-row tile row for up to 10 activation rows, the one-pass many-row
 *      kernel (a CTA per eight tile rows, digits of a k-tile shared in shared memory) for passes of 11 to 32 rows;
 *   2: the tile-row kernel only (passes of 10 rows at any row count);
 *   1: the CUDA-core GEMV on the raw blocks (an independent second implementation for cross-checks);
 *   3: the per-warp streaming variant of the tile-row kernel where the shape qualifies;
 *   4: calls of 1-5 rows take the bulk-copy ring GEMV (persistent CTAs, shared-memory ring fed by cp.async.bulk,
 *      activation digits built inside the kernel) where the shape fits. */
int32_t sp_cuda_set_gemv_path(int32_t path);
/* Op-level matmuls with m >= 17 rows and k % 256 == 0 (Q8_0: k % 128 == 0):
 * 2 (default): the tcgen05 / TMEM dequant GEMM with exact-class operands — weights and activations each as an fp16
 *    leading part plus the fp16 of what that rounding dropped (rows scaled by a power of two first), three tensor-core
 *    products per chunk of K: ~1e-6 per product, the level of the integer-digit GEMV;
 * 1: the same GEMM with operands rounded once to fp16 (~3e-4 per product, 2x faster);
 * 0: exact integer products on the mma.sync kernels at every row count (passes of up to 32 rows).
 * Process-wide; engines have their own switch with the same values and default. */
int32_t sp_cuda_set_large_m_gemm(int32_t on);
/* Device address and byte size of the resident blocks (for benchmarks that rotate buffers). */
int32_t sp_cuda_weight_info(const SpWeight* w, int32_t* dtype, int64_t* n, int64_t* k, size_t* nbytes);

/* LlmBackend per-op contract (crates/sapient-models/src/forward/backend.rs:57-115), host buffers. */
int32_t sp_cuda_rms_norm(int32_t device, const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y);
int32_t sp_cuda_layer_norm(int32_t device, const float* x, const float* w, const float* b, int64_t rows, int64_t dim,
                           float eps, float* y);
/* x: [n_heads, seq, head_dim] like the reference's [1,H,seq,hd]; positions[seq]. */
int32_t sp_cuda_rope(int32_t device, const float* x, int64_t n_heads, int64_t seq, int64_t head_dim,
                     const int64_t* positions, float base, int64_t rotary_dim, float* y);
/* causal GQA attention: q [H, sq, hd], k/v [Hkv, sk, hd] (f32, stored as fp16 pages on the device), out [H, sq, hd] */
int32_t sp_cuda_attention(int32_t device, const float* q, const float* k, const float* v, int64_t n_heads,
                          int64_t n_kv_heads, int64_t sq, int64_t sk, int64_t head_dim, float* out);
/* No counterpart in the reference: the same split-K attention for callers that must not allocate device memory
 * (a serving loop whose memory pool owns the whole device, or code where an allocation's device-wide
 * synchronisation would stall other streams). Every pointer is a DEVICE pointer the caller owns:
 * d_q [n_tok, ldq] and d_out [n_tok, ldo] hold n_heads * head_dim floats per row; d_kv_pool is the fp16 page pool
 * [layer][page][K|V][n_kv_heads][16 tokens][head_dim]; d_page_table [slots, max_pages]; d_tok_slot / d_tok_pos give
 * each row's sequence slot and position (keys 0..pos are attended). The per-split partials live in a fixed array
 * inside the library, SP_ATTENTION_STATIC_MAX_FLOATS floats per device: a call needing more
 * (n_tok * n_heads * n_splits * (head_dim + 2) when n_splits > 1) fails with SP_ERR_SHAPE. The array is shared by
 * all calls on a device, so calls must not overlap in time; it needs no clearing between calls. The first call on
 * a device resolves the array's address and should be made before any stream capture. Launches on `stream`
 * (a cudaStream_t, NULL = default stream) and returns without synchronising. */
#define SP_ATTENTION_STATIC_MAX_FLOATS (1u << 20)
int32_t sp_cuda_attention_paged_static(int32_t device, const float* d_q, int32_t ldq, float* d_out, int32_t ldo, int32_t n_tok,
                                       int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, const int32_t* d_tok_slot,
                                       const int32_t* d_tok_pos, const void* d_kv_pool, const int32_t* d_page_table,
                                       int32_t n_pages, int32_t max_pages, int32_t layer, int32_t n_splits, void* stream);
int32_t sp_cuda_silu(int32_t device, const float* x, int64_t n, float* y);
int32_t sp_cuda_gelu(int32_t device, const float* x, int64_t n, float* y);
int32_t sp_cuda_add(int32_t device, const float* a, const float* b, int64_t n, float* y);
int32_t sp_cuda_mul(int32_t device, const float* a, const float* b, int64_t n, float* y);
/* embed_tokens (forward/common.rs:164-217): rows of a [vocab, hidden] table, dequantised per row. */
int32_t sp_cuda_embed(const SpWeight* table, const uint32_t* ids, int64_t n, float* out_host);
/* sampler::argmax (crates/sapient-generate/src/sampler.rs:161-168): last maximum wins. */
int32_t sp_cuda_argmax(int32_t device, const float* logits, int64_t rows, int64_t n, uint32_t* out);

/* ── engine level: replaces ForwardEngine (crates/sapient-models/src/forward/mod.rs:49-65,381-506)
 *    in the shape of the resident WgpuForwardEngine (forward/wgpu_engine.rs:93-110,173-341,362-676) ── */
typedef struct SpEngine SpEngine;

typedef struct SpModelDesc {
    int32_t arch;        /* 0: llama/qwen2 family (LlamaForward); 1: phi2 (PhiForward parallel block) */
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;
    int32_t max_ctx;     /* KV window per sequence (kv_cache_ctx, forward/common.rs:25-37) */
    int32_t rotary_dim;  /* head_dim for full RoPE */
    float norm_eps, rope_theta;
    int32_t max_batch;   /* sequence slots (1 = the reference's single-sequence engine) */
    int32_t max_tokens;  /* tokens per internal forward chunk (prefill is chunked; results do not depend on it) */
    int32_t device;      /* CUDA device ordinal */
    int32_t tp_rank, tp_size; /* tensor-parallel placement (1 = single GPU) */
    int64_t kv_pages;    /* pages of 16 tokens in the pool; 0 = max_batch * ceil(max_ctx/16) */
} SpModelDesc;

/* ModelInfo::from_gguf_metadata (crates/sapient-hub/src/model_info.rs:234-352) + ForwardEngine::from_weights */
int32_t sp_cuda_engine_create(const SpModelDesc* desc, SpEngine** out);
/* One entry of the HF-named weight map that from_weights consumes (forward/wgpu_engine.rs:173-186). dims are
 * [out, in] for matrices, [n] for vectors; bytes are raw ggml blocks / f32 / f16; the library copies. */
int32_t sp_cuda_engine_set_tensor(SpEngine* e, const char* hf_name, int32_t dtype, const int64_t* dims, int32_t ndim,
                                  const void* host_bytes, size_t nbytes);
/* Resolves weights (tied lm_head fallback: crates/sapient-models/src/weights.rs:88-109), allocates KV pages and
 * activations. */
int32_t sp_cuda_engine_finalize(SpEngine* e);
/* ForwardEngine::from_gguf (forward/mod.rs:223-316): parse a GGUF file (crates/sapient-io/src/gguf.rs:517-778), map
 * names (crates/sapient-models/src/gguf_weights.rs:61-96,360-455), un-permute llama q/k rows (:114-154), split Phi
 * qkv (:273-330), create + finalize. max_ctx/max_batch 0 = file's context_length (capped at 8192) / 1. */
int32_t sp_cuda_engine_from_gguf(const char* path, int32_t device, int32_t max_ctx, int32_t max_batch, SpEngine** out);
int32_t sp_cuda_engine_desc(const SpEngine* e, SpModelDesc* out);
void sp_cuda_engine_destroy(SpEngine* e);
/* Tensor parallelism (one process per GPU; Llama/Qwen block only). An engine created with tp_size > 1 keeps, of every
 * tensor handed to sp_cuda_engine_set_tensor in FULL, only its rank's slice: rows of q/k/v/gate/up and of lm_head
 * (vocab / tp_size rows), columns of o_proj / down_proj on block boundaries; norms and the embedding table are
 * replicated. After finalize every rank exports the CUDA IPC handle of its communication block (SP_TP_HANDLE_BYTES
 * bytes), the caller gathers the handles of all ranks in rank order (any transport) and passes them to
 * sp_cuda_engine_tp_connect on every rank. Column-split products are summed by pushing partial rows into every rank's
 * block over NVLink from the GEMV epilogue, with bounded waits (SP_ERR_COMM when a peer does not arrive). All ranks must
 * then make the same calls in the same order. Logit outputs hold this rank's vocabulary slice only
 * (sp_cuda_engine_vocab_local: its size and first token id); argmax outputs are global token ids on every rank. */
#define SP_TP_HANDLE_BYTES 64
int32_t sp_cuda_engine_tp_handle(SpEngine* e, void* out, size_t cap);
int32_t sp_cuda_engine_tp_connect(SpEngine* e, const void* handles, int32_t n_ranks);
int32_t sp_cuda_engine_vocab_local(const SpEngine* e, int32_t* rows, int32_t* first);
/* Engines of ONE process (one per GPU, or several on one GPU for tests): the device address of a rank's communication
 * block, and connecting with the blocks of all ranks in rank order instead of IPC handles. */
int32_t sp_cuda_engine_tp_block(SpEngine* e, void** block);
int32_t sp_cuda_engine_tp_connect_local(SpEngine* e, void* const* blocks, int32_t n_ranks);
/* How long a kernel waits for a peer's partial rows before it gives up (default 5000 ms; the step then ends with
 * SP_ERR_COMM). Long enough for a peer that is still capturing its first step graph or finishing a prefill; a
 * supervisor that detects failures on the host can lower it. Takes effect with the next launch. */
int32_t sp_cuda_engine_tp_set_wait_ms(SpEngine* e, int32_t ms);
/* Comparison arm for the sums of the column-split products (o_proj, down_proj): mode 1 sends them through ncclAllReduce
 * on the engine's stream (partial product to scratch, all-reduce, one add) instead of the default mode 0, the push from
 * the GEMV epilogue into every rank's memory. NCCL is not linked: libnccl_path names the shared object to open (the copy
 * the process already uses; NULL or "" = "libnccl.so.2" by the loader's search). Rank 0 makes a 128-byte id with
 * sp_cuda_nccl_unique_id, the caller hands it to every rank, every rank calls sp_cuda_engine_tp_nccl_init (a collective),
 * then sp_cuda_engine_tp_set_allreduce chooses the arm (all ranks the same). The arg-max exchange stays on peer stores. */
#define SP_NCCL_ID_BYTES 128
int32_t sp_cuda_nccl_unique_id(const char* libnccl_path, void* out, size_t cap);
int32_t sp_cuda_engine_tp_nccl_init(SpEngine* e, const char* libnccl_path, const void* unique_id);
int32_t sp_cuda_engine_tp_set_allreduce(SpEngine* e, int32_t mode);
/* After SP_ERR_COMM, or to restart a group: exchange counters, arrival marks and the sticky error flag back to their
 * initial state. EVERY rank calls it, with a host-side barrier before (no rank still inside a step) and after (no rank
 * starts a step before all have cleared). The KV caches are untouched: truncate or reset them as the caller sees fit. */
int32_t sp_cuda_engine_tp_reset(SpEngine* e);
/* The slice rank `rank` of `size` keeps of one full tensor (host only, no device needed): writes the slice to out
 * (may be NULL to query sizes), its dims to out_dims[ndim] and its byte size to *out_bytes. Replicated tensors come
 * back whole. vocab bounds the rows of lm_head.weight. */
int32_t sp_cuda_tp_shard(const char* hf_name, int32_t dtype, const int64_t* dims, int32_t ndim, const void* bytes, size_t nbytes,
                         int32_t rank, int32_t size, int64_t vocab, void* out, size_t out_cap, int64_t* out_dims,
                         size_t* out_bytes);
/* How new K / V rows are rounded into the fp16 page pool. 1 (default): through the reference's Q8_0 cache rounding first
 * (per 32 values: scale = amax / 127 held as f16, value = round(x / scale) * scale; forward/common.rs:336-348,449-538;
 * applies when head_dim % 32 == 0, where the reference keeps a Q8_0 cache), so attention reads what the reference's
 * cache yields; 0: plain fp16 rounding of the f32 values. Only while every sequence is empty. */
int32_t sp_cuda_engine_set_kv_rounding(SpEngine* e, int32_t mode);
/* Launch on this cudaStream_t instead of the engine's own stream (NULL restores it). */
int32_t sp_cuda_engine_set_stream(SpEngine* e, void* stream);

/* ForwardEngine::forward_logits (forward/mod.rs:416-426): appends ids to slot 0 (use_cache == 0 resets first, like
 * wgpu_engine.rs:639-641) and writes last-position logits[vocab] to host. */
int32_t sp_cuda_forward_logits(SpEngine* e, const uint32_t* ids, size_t n, int32_t use_cache, float* logits_out);
/* forward_all_logits (reset, all positions) and forward_all_logits_cached (append): out[n * vocab]. */
int32_t sp_cuda_forward_all_logits(SpEngine* e, const uint32_t* ids, size_t n, float* out);
int32_t sp_cuda_forward_all_logits_cached(SpEngine* e, const uint32_t* ids, size_t n, float* out);
/* Same for an explicit sequence slot (batched extension; the reference engine has exactly one sequence). */
int32_t sp_cuda_forward_slot(SpEngine* e, int32_t slot, const uint32_t* ids, size_t n, int32_t all_positions,
                             float* logits_out);
/* One decode step for b sequences: ids[i] is appended to slot slots[i]. Either output may be NULL:
 * logits_out[b * vocab] (host) and/or argmax_out[b] (host; last-maximum tie rule). */
int32_t sp_cuda_decode_batch(SpEngine* e, const uint32_t* ids, const int32_t* slots, int32_t b, float* logits_out,
                             uint32_t* argmax_out);
/* Greedy decode kept on the device: `steps` steps for b slots; step 0 consumes first_ids, each later step consumes the
 * argmax (last-maximum rule) of the previous one, with no host work in between. tokens_out[steps * b] (host, step-major)
 * may be NULL, in which case the call returns without synchronising (use sp_cuda_engine_synchronize). This is the loop
 * Pipeline::generate_* runs with SamplingStrategy::Greedy (crates/sapient-generate/src/pipeline.rs:540-659). */
int32_t sp_cuda_decode_greedy(SpEngine* e, const uint32_t* first_ids, const int32_t* slots, int32_t b, int32_t steps,
                              uint32_t* tokens_out);
/* Greedy speculative decoding of one sequence (slot 0 of both engines, which are reset first): the schedule of
 * SpeculativePipeline with greedy sampling (crates/sapient-generate/src/speculative.rs:499-631; draft length `k` as
 * crates/sapient-cli/src/server.rs:282-283) with both loops inside the library. Per round the draft runs k steps of the
 * device-resident greedy loop, the target verifies in ONE forward of k + 1 rows (the token committed last + the k
 * drafts), drafts are kept while they equal the target's arg-max (last maximum wins), the target's pick after them is
 * committed as well, and both caches are rolled back to the committed tokens. The committed stream equals the target's
 * own greedy decoding. tokens_out[max_new] receives the generated tokens (the prompt is not repeated), *n_out their
 * count (generation stops after an id listed in eos_ids); stats, when not NULL, receives {rounds, drafted, accepted}.
 * 1 <= k <= 15; both engines single-GPU with the same vocabulary. */
int32_t sp_cuda_spec_greedy(SpEngine* target, SpEngine* draft, const uint32_t* prompt, size_t n_prompt, int32_t k, size_t max_new,
                            const uint32_t* eos_ids, int32_t n_eos, uint32_t* tokens_out, size_t* n_out, uint64_t* stats);
int32_t sp_cuda_engine_synchronize(SpEngine* e);

/* Page sharing between sequence slots. The cache is a pool of 16-token pages with an owner count per page;
 * sp_cuda_engine_slot_page names the pool page that holds tokens [16 index, 16 index + 16) of a slot, and
 * sp_cuda_engine_adopt_prefix makes an EMPTY slot a reader of n such pages (its length becomes 16 n): the prefix is not
 * recomputed and not copied. Shared pages are never written — appending to a slot whose partly filled last page has
 * another owner (after a truncate into a shared page) first moves the slot to a private copy of that page. The
 * reference's single cache can only re-use the prefix of its own previous contents
 * (truncate_cache, crates/sapient-models/src/forward/llama.rs:307-313). */
int32_t sp_cuda_engine_slot_page(const SpEngine* e, int32_t slot, int32_t index, int32_t* page);
int32_t sp_cuda_engine_adopt_prefix(SpEngine* e, int32_t slot, const int32_t* pages, int32_t n);

/* ── Continuous batching over the paged KV cache ──
 * The reference serves one sequence per engine and re-uses a prompt prefix only against the previous turn of the same
 * conversation (crates/sapient-generate/src/pipeline.rs:818-830); batching is on its roadmap (docs/ROADMAP.md:312).
 * A batcher owns the sequence slots of one engine (max_batch of them; the engine's caches must be empty when it is
 * created and the engine must not be driven directly while the batcher lives). Requests are greedy generations
 * (last-maximum arg-max, sampler.rs:161-168): each request's tokens equal what the engine produces for that prompt
 * alone. sp_cuda_batcher_step runs ONE scheduler iteration:
 *   1. admit queued requests, first come first served, while a slot is free and the page pool can hold
 *      prompt + max_new tokens beside what running requests were promised; pages of an already computed prompt prefix
 *      (whole 16-token pages, found by content in the prefix index) are shared instead of recomputed, and index pages
 *      nobody reads are evicted, least recently used first, when the pool is short;
 *   2. at most prefill_chunk prompt tokens of the oldest prefilling requests;
 *   3. one decode step carrying one token of every decoding sequence.
 * A request leaves the batch after an id of its eos list or max_new tokens; its slot is free for the next iteration.
 * Single thread per batcher. Errors of the engine calls are returned by the step that made them. Destroy the batcher
 * before the engine it drives (its destructor returns the slots' pages to the engine's pool). */
typedef struct SpBatcher SpBatcher;
int32_t sp_cuda_batcher_create(SpEngine* e, int32_t prefill_chunk, int32_t prefix_cache, SpBatcher** out);
/* The same scheduler over a host stand-in instead of an engine (no GPU, no model: the "next token" is a hash of the
 * sequence as read back through the page tables). It exists so the scheduling logic — admission, page accounting,
 * sharing, eviction, copy-on-write — can be tested where there is no GPU; it computes nothing of the product. */
int32_t sp_cuda_batcher_create_selftest(int32_t vocab, int32_t max_slots, int32_t max_ctx, int32_t n_pages, int32_t prefill_chunk,
                                        int32_t prefix_cache, SpBatcher** out);
void sp_cuda_batcher_destroy(SpBatcher* b);
/* Queues a request; *id names it afterwards. SP_ERR_KV_FULL when prompt + max_new exceeds the window or the pool. */
int32_t sp_cuda_batcher_submit(SpBatcher* b, const uint32_t* prompt, size_t n, size_t max_new, const uint32_t* eos_ids, int32_t n_eos,
                               uint64_t* id);
int32_t sp_cuda_batcher_step(SpBatcher* b, int32_t* n_running, int32_t* n_waiting);
/* Tokens generated so far (at most cap are copied, *n_tokens is the full count); *finished = 1 once the request has left
 * the batch. Finished requests stay readable until sp_cuda_batcher_forget. */
int32_t sp_cuda_batcher_poll(const SpBatcher* b, uint64_t id, uint32_t* tokens_out, size_t cap, size_t* n_tokens, int32_t* finished);
int32_t sp_cuda_batcher_cancel(SpBatcher* b, uint64_t id);
int32_t sp_cuda_batcher_forget(SpBatcher* b, uint64_t id);
/* out[0..9): submitted, finished, steps, prompt tokens computed, prompt tokens shared, tokens decoded, index pages evicted,
 * index pages held, free pool pages. */
#define SP_BATCHER_STATS 9
int32_t sp_cuda_batcher_stats(const SpBatcher* b, uint64_t* out, int32_t cap);
/* Replay decode steps as CUDA graphs (default on). */
int32_t sp_cuda_engine_set_graphs(SpEngine* e, int32_t on);
/* Steps of 17 rows and more (prefill chunks, batched decode) run on the tcgen05 GEMM: each weight tile is dequantised
 * once and multiplied with all rows on the 5th-generation tensor cores.
 * on = 2 (default): exact-class operands (leading fp16 part + remainder for weights and activations, three products per
 *    chunk of K, ~1e-6 per product); activations are converted from their f32 rows, attention stays on the f32-class
 *    kernels. Full-size models keep the 2e-2 final-logit bar (8B shape, 128-token prompt: 6.7e-3).
 * on = 1: operands rounded once to fp16 (~3e-4 per product, inside the 1e-3 per-op bar, but the 8B shape's final logits
 *    then move by up to 4e-2), fused fp16 producers and the fp16 prefill attention: a 512-token prefill of the 8B shape
 *    takes 15 ms instead of 28 ms.
 * on = 0: integer-digit GEMV passes of 10 rows at any row count (201 ms for that prefill).
 * Drops the captured step graphs. */
int32_t sp_cuda_engine_set_large_m_gemm(SpEngine* e, int32_t on);
/* Steps of 1-5 rows on the bulk-copy ring GEMV with the preceding norm / activation fused into it (default off: it
 * measures slower than the default kernels). Drops the captured step graphs. */
int32_t sp_cuda_engine_set_ring(SpEngine* e, int32_t on);
/* For the steps that do not go to the tcgen05 GEMM (11-16 rows; every step of 11 rows and more when
 * sp_cuda_engine_set_large_m_gemm is 0): 1 = passes of up to 32 rows on the one-pass many-row GEMV, weights read once per
 * 32 rows; 0 (default) = passes of 10 rows on the tile-row kernel. The same exact integer products, another order of the
 * f32 additions over k. */
int32_t sp_cuda_engine_set_many_row_gemv(SpEngine* e, int32_t on);
/* Per-kernel-family device timing (CUDA events around every launch; disables graphs while on). Families, in order:
 * gemv, attention, norm, rope_kv, elementwise, embed, argmax. Returns the family count; ms/launches accumulate
 * until reset (reset != 0 clears after reading). */
int32_t sp_cuda_engine_set_profile(SpEngine* e, int32_t on);
/* Device time (ms) of one decode step of n_tokens rows restricted to the kernel families whose bits are set in
 * family_mask (bit i = family i of the list above; 0x7F = the whole step), measured by replaying that subset as a
 * CUDA graph `reps` times between two events. Activations and the newest KV entries are undefined afterwards. */
int32_t sp_cuda_engine_time_families(SpEngine* e, uint32_t family_mask, int32_t n_tokens, int32_t reps, float* ms_per_step);
int32_t sp_cuda_engine_profile_read(SpEngine* e, double* ms, uint64_t* launches, int32_t cap, int32_t reset);
/* reset_cache / truncate_cache (forward/mod.rs:381-414): kept = min(n, current). slot < 0 = all slots. */
int32_t sp_cuda_reset_cache(SpEngine* e, int32_t slot);
int32_t sp_cuda_truncate_cache(SpEngine* e, int32_t slot, size_t n, size_t* kept);
int32_t sp_cuda_seq_len(const SpEngine* e, int32_t slot, size_t* len);
/* backend_label (forward/mod.rs:482-494) -> "cuda"; is_hybrid is always false. */
int32_t sp_cuda_backend_label(const SpEngine* e, char* buf, size_t cap);
/* Keep the hidden state after every layer of each forward chunk (for per-layer parity checks); off by default. */
int32_t sp_cuda_engine_set_trace(SpEngine* e, int32_t on);
/* Weight upload accounting: seconds the engine spent moving tensor bytes to the device (host pages -> two pinned staging
 * buffers -> asynchronous copies on a dedicated stream, the host filling one buffer while the other is in flight) and the
 * bytes moved. sp_cuda_engine_from_gguf maps the file, so these are the only copies of the weights made on the host;
 * the llama q / k row un-permute runs as a device-side gather and the Phi qkv split as three row ranges of one mapping
 * (the reference does both on the host: crates/sapient-models/src/gguf_weights.rs:114-154,273-311). */
int32_t sp_cuda_engine_load_stats(const SpEngine* e, double* seconds, uint64_t* bytes);
/* Hidden state after `layer` of the most recent forward chunk, [n_tokens, hidden] to host; returns rows in *n_tokens. */
int32_t sp_cuda_debug_layer_out(SpEngine* e, int32_t layer, float* out, size_t cap_floats, int32_t* n_tokens);
/* Number of kernels this library has launched since process start (all engines and ops). */
uint64_t sp_cuda_launch_count(void);
/* Device bytes held by the weights and by the KV page pool (the reference logs the same at engine-ready time,
 * forward/wgpu_engine.rs:314-327). */
int32_t sp_cuda_engine_resident_bytes(const SpEngine* e, uint64_t* weights, uint64_t* kv);

#ifdef __cplusplus
}
#endif
#endif /* SAPIENT_CUDA_H */
