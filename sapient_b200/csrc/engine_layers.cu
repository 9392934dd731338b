// Per-layer launch sequences of the resident engine.
//   Llama/Qwen: crates/sapient-models/src/forward/llama.rs:400-539
//   Phi-2     : crates/sapient-models/src/forward/phi.rs:373-503
//
// Decode-shaped steps (T <= 16 rows) run fused: every kernel that produces a GEMV input (norm,
// SwiGLU / GELU, the split-K attention merge) emits the int8 digits the tensor-core GEMV consumes,
// so a layer is 10 launches: norm+digits, qkv, rope+kv, attention split, merge+digits, o,
// norm+digits, gate|up, swiglu+digits, down.
#include <cstdlib>
#include <algorithm>

#include "engine.h"
#include "sp_common.cuh"

namespace sp {

#define SP_TRY(expr)                  \
    do {                              \
        int _s = (expr);              \
        if (_s != SP_OK) return _s;   \
    } while (0)

#define SP_LAUNCH(fam, expr)              \
    do {                                  \
        if (fam_mask & (1u << (fam))) {   \
            prof_begin(fam);              \
            SP_CUDA_TRY(expr);            \
            prof_end(fam);                \
        }                                 \
    } while (0)

int Engine::tp_resolve(int T) {
    if (!tp_pending_) return SP_OK;
    tp_pending_ = false;
    SP_LAUNCH(F_NORM, launch_tp_reduce(x_, d.hidden, T, d.hidden, d_tp_, stream));
    return SP_OK;
}

// Plans the digit workspace for m rows of k columns; true when the fused producers may be used
// (all rows fit the workspace at once).
bool Engine::plan_digits(int m, int k, ImmaArgs& ia) {
    ia = ImmaArgs{};
    ia.m = m;
    ia.k = k;
    if (m > imma_rows_per_pass() || k > ws_.k_max) return false;
    imma_plan(ia, ws_);
    return true;
}

// y_i[m, n_i] = x[m, k] · W_iᵀ (+ bias_i) for up to three matrices sharing x; `res` is added to the first.
// pre != null: the digits of x are already in the workspace (planned as *pre).
int Engine::gemv(const float* x, int ldx, int m, int k, const DevTensor* w0, const float* b0, float* y0, int ldy0,
                 const DevTensor* w1, const float* b1, float* y1, const DevTensor* w2, const float* b2, float* y2,
                 const float* res, const ImmaArgs* pre, bool tp_sum) {
    tp_sum = tp_sum && d.tp_size > 1;
    if (tp_sum && !tp_connected_) { set_error("tensor-parallel engine used before tp_connect"); return SP_ERR_STATE; }
    const DevTensor* ws[3] = {w0, w1, w2};
    const float* bs[3] = {b0, b1, b2};
    float* ys[3] = {y0, y1, y2};
    bool tiled = true;
    for (int i = 0; i < 3 && ws[i]; ++i) tiled = tiled && ws[i]->tiled != nullptr;
    if (tiled && !pre && m >= TC5_MIN_M && use_tc5 && ws_.xh && (size_t)m * k * (tc5_exact ? 2 : 1) <= ws_.xh_elems &&
        (!tc5_exact || m <= ActWorkspace::XSCALE_ROWS) && (!tp_sum || (y0 == x_ && res == x_ && ldy0 == d.hidden && !w1 && x != h_))) {
        bool ok = true;
        for (int i = 0; i < 3 && ws[i]; ++i) ok = ok && tc5_supported(ws[i]->dtype, k);
        if (ok) {
            // many rows: dequantise each weight tile once and multiply on the 5th-generation tensor cores
            if (tc5_exact) SP_LAUNCH(F_ELEM, launch_x_to_f16_hilo(x, ldx, m, k, ws_.xh, ws_.xscale, stream));
            else SP_LAUNCH(F_ELEM, launch_x_to_f16(x, ldx, m, k, ws_.xh, stream));
            Tc5Seg segs[3];
            int ns = 0;
            if (tp_sum) {
                // column-split matrix: this rank's partial product to scratch (the bias once, on rank 0), then to every
                // rank's receive area (or through the library all-reduce of the comparison arm)
                segs[ns++] = Tc5Seg{w0->tiled, h_, d.tp_rank == 0 ? b0 : nullptr, w0->dtype, (int)w0->dims[0]};
                SP_LAUNCH(F_GEMV, launch_gemm_tc5_multi(segs, ns, k, ws_.xh, m, d.hidden, nullptr, 0, stream, &ws_.tc5, tc5_exact ? ws_.xscale : nullptr));
                if (tp_use_nccl_) {
                    SP_TRY(nccl_all_reduce(h_, (size_t)m * d.hidden));
                    SP_LAUNCH(F_ELEM, launch_add(x_, h_, x_, (int64_t)m * d.hidden, stream));
                    return SP_OK;
                }
                SP_LAUNCH(F_GEMV, launch_tp_push(h_, d.hidden, m, d.hidden, d_tp_, stream));
                tp_pending_ = true;
                return SP_OK;
            }
            for (int i = 0; i < 3 && ws[i]; ++i) segs[ns++] = Tc5Seg{ws[i]->tiled, ys[i], bs[i], ws[i]->dtype, (int)ws[i]->dims[0]};
            SP_LAUNCH(F_GEMV, launch_gemm_tc5_multi(segs, ns, k, ws_.xh, m, ldy0, res, ldy0, stream, &ws_.tc5, tc5_exact ? ws_.xscale : nullptr));
            return SP_OK;
        }
    }
    // 11 rows and more on one GPU: passes of up to 32 rows, each reading the weights once (gemv_rows.cu)
    if (tiled && !tp_sum && !pre && use_rows && m > imma_rows_per_pass() && k % 256 == 0 && k <= ws_.k_max) {
        bool ok = true;
        for (int i = 0; i < 3 && ws[i]; ++i) ok = ok && rows_supported(ws[i]->dtype, k);
        if (ok) {
            for (int m0 = 0; m0 < m; m0 += IMMA_ROWS_MAX) {
                ImmaArgs ia{};
                ia.k = k; ia.m = std::min(IMMA_ROWS_MAX, m - m0);
                ia.res = res ? res + (size_t)m0 * ldy0 : nullptr;
                ia.ldres = ldy0;
                for (int i = 0; i < 3 && ws[i]; ++i) {
                    ImmaSeg& sgm = ia.seg[ia.nseg++];
                    sgm.wt = ws[i]->tiled; sgm.bias = bs[i]; sgm.y = ys[i] + (size_t)m0 * ldy0; sgm.dtype = ws[i]->dtype;
                    sgm.n = (int)ws[i]->dims[0]; sgm.ldy = ldy0; sgm.bpt = imma_q8_bpt(k);
                }
                imma_plan_rows(ia, ws_);
                SP_LAUNCH(F_ELEM, launch_act_quant(x + (size_t)m0 * ldx, ldx, ia, stream));
                SP_LAUNCH(F_GEMV, launch_gemv_rows(ia, rows_, stream));
            }
            return SP_OK;
        }
    }
    // comparison arm: the partial product to scratch, a library all-reduce, one add into the residual stream
    const bool via_nccl = tp_sum && tp_use_nccl_ && tiled;
    if (via_nccl && (y0 != x_ || res != x_ || ldy0 != d.hidden || w1)) { set_error("internal: tensor-parallel sum outside the residual stream"); return SP_ERR_STATE; }
    if (tiled) {
        // tensor-core path: digits of up to 16 activation rows at a time, all segments share them
        const int pass = imma_rows_per_pass();
        for (int m0 = 0; m0 < m; m0 += pass) {
            ImmaArgs ia{};
            if (pre) ia = *pre;
            ia.k = k; ia.m = std::min(pass, m - m0);
            ia.res = (res && !tp_sum) ? res + (size_t)m0 * ldy0 : nullptr;
            ia.ldres = ldy0;
            ia.tp = (tp_sum && !via_nccl) ? d_tp_ : nullptr;
            ia.tp_row0 = m0;
            ia.nseg = 0;
            for (int i = 0; i < 3 && ws[i]; ++i) {
                ImmaSeg& sgm = ia.seg[i];
                sgm.wt = ws[i]->tiled; sgm.bias = (via_nccl && d.tp_rank != 0) ? nullptr : bs[i]; sgm.y = (via_nccl ? h_ : ys[i]) + (size_t)m0 * ldy0; sgm.dtype = ws[i]->dtype;
                sgm.n = (int)ws[i]->dims[0]; sgm.ldy = ldy0; sgm.bpt = imma_q8_bpt(k);
                ia.nseg++;
            }
            if (!pre) {
                imma_plan(ia, ws_);
                SP_LAUNCH(F_ELEM, launch_act_quant(x + (size_t)m0 * ldx, ldx, ia, stream));
            }
            SP_LAUNCH(F_GEMV, launch_gemv_imma(ia, stream));
        }
        if (via_nccl) {
            SP_TRY(nccl_all_reduce(h_, (size_t)m * d.hidden));
            SP_LAUNCH(F_ELEM, launch_add(x_, h_, x_, (int64_t)m * d.hidden, stream));
            return SP_OK;
        }
        // the partial rows are on their way to every rank; whoever reads y0 next adds their sum first
        if (tp_sum) {
            if (y0 != x_ || res != x_) { set_error("internal: tensor-parallel sum outside the residual stream"); return SP_ERR_STATE; }
            tp_pending_ = true;
        }
        return SP_OK;
    }
    if (tp_sum) { set_error("tensor parallel: column-split matrix without tiles"); return SP_ERR_STATE; }
    if (pre) { set_error("internal: pre-quantised input for a weight without tiles"); return SP_ERR_STATE; }
    if (w1 && (w0->tiled || w1->tiled || (w2 && w2->tiled))) {
        // mixed layouts: one launch per matrix
        SP_TRY(gemv(x, ldx, m, k, w0, b0, y0, ldy0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, res));
        SP_TRY(gemv(x, ldx, m, k, w1, b1, y1, ldy0));
        if (w2) SP_TRY(gemv(x, ldx, m, k, w2, b2, y2, ldy0));
        return SP_OK;
    }
    GemvArgs a{};
    a.x = x; a.ldx = ldx; a.m = m; a.k = k; a.res = res; a.ldres = ldy0;
    a.nseg = 0;
    for (int i = 0; i < 3; ++i) {
        if (!ws[i]) break;
        a.seg[i].w = ws[i]->d; a.seg[i].bias = bs[i]; a.seg[i].y = ys[i]; a.seg[i].dtype = ws[i]->dtype;
        a.seg[i].n = (int)ws[i]->dims[0]; a.seg[i].ldy = ldy0;
        a.nseg++;
    }
    SP_LAUNCH(F_GEMV, launch_gemv(a, stream));
    return SP_OK;
}

int Engine::try_ring(bool* done, int m, int k, int src, const float* x, int ldx, const float* nw, const float* nb, const DevTensor* w0,
                     const float* b0, float* y0, int ldy, const DevTensor* w1, const float* b1, float* y1, const DevTensor* w2,
                     const float* b2, float* y2, const float* res) {
    *done = false;
    if (!use_ring || d.tp_size > 1 || trace_on || m > RING_MAX_M) return SP_OK;
    const DevTensor* ws[3] = {w0, w1, w2};
    const float* bs[3] = {b0, b1, b2};
    float* ys[3] = {y0, y1, y2};
    RingArgs ra{};
    for (int i = 0; i < 3 && ws[i]; ++i) {
        if (!ws[i]->tiled) return SP_OK;
        ImmaSeg& sg = ra.seg[ra.nseg++];
        sg.wt = ws[i]->tiled; sg.bias = bs[i]; sg.y = ys[i]; sg.dtype = ws[i]->dtype; sg.n = (int)ws[i]->dims[0]; sg.ldy = ldy; sg.bpt = 8;
    }
    ra.k = k; ra.m = m; ra.src = src; ra.x = x; ra.ldx = ldx; ra.nw = nw; ra.nb = nb; ra.eps = d.norm_eps; ra.res = res; ra.ldres = ldy;
    if (!ring_plan(ra, ring_)) return SP_OK;
    SP_LAUNCH(F_GEMV, launch_gemv_ring(ra, stream));
    *done = true;
    return SP_OK;
}

bool Engine::big_m(int m, int k, const DevTensor* w0, const DevTensor* w1, const DevTensor* w2) const {
    if (m < TC5_MIN_M || !use_tc5 || tc5_exact || !ws_.xh || (size_t)m * k > ws_.xh_elems) return false;
    const DevTensor* ws[3] = {w0, w1, w2};
    for (int i = 0; i < 3 && ws[i]; ++i)
        if (!ws[i]->tiled || !tc5_supported(ws[i]->dtype, k)) return false;
    return true;
}

int Engine::gemm_xh(int m, int k, const DevTensor* w0, const float* b0, float* y0, int ldy0, const DevTensor* w1, const float* b1,
                    float* y1, const DevTensor* w2, const float* b2, float* y2, const float* res) {
    const DevTensor* ws[3] = {w0, w1, w2};
    const float* bs[3] = {b0, b1, b2};
    float* ys[3] = {y0, y1, y2};
    Tc5Seg segs[3];
    int ns = 0;
    for (int i = 0; i < 3 && ws[i]; ++i) segs[ns++] = Tc5Seg{ws[i]->tiled, ys[i], bs[i], ws[i]->dtype, (int)ws[i]->dims[0]};
    SP_LAUNCH(F_GEMV, launch_gemm_tc5_multi(segs, ns, k, ws_.xh, m, ldy0, res, ldy0, stream, &ws_.tc5));
    return SP_OK;
}

int Engine::gemm_xh_sum(int m, int k, const DevTensor* w, const float* b) {
    if (d.tp_size <= 1) return gemm_xh(m, k, w, b, x_, d.hidden, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_);
    if (!tp_connected_) { set_error("tensor-parallel engine used before tp_connect"); return SP_ERR_STATE; }
    // the partial product of this rank's columns (the bias once, on rank 0) to scratch, then to every rank's receive area
    SP_TRY(gemm_xh(m, k, w, d.tp_rank == 0 ? b : nullptr, h_, d.hidden));
    if (tp_use_nccl_) {
        SP_TRY(nccl_all_reduce(h_, (size_t)m * d.hidden));
        SP_LAUNCH(F_ELEM, launch_add(x_, h_, x_, (int64_t)m * d.hidden, stream));
        return SP_OK;
    }
    SP_LAUNCH(F_GEMV, launch_tp_push(h_, d.hidden, m, d.hidden, d_tp_, stream));
    tp_pending_ = true;
    return SP_OK;
}

static inline bool all_tiled(const DevTensor* a, const DevTensor* b = nullptr, const DevTensor* c = nullptr) {
    return a->tiled && (!b || b->tiled) && (!c || c->tiled);
}

// Keys are split over several blocks while (token, head) pairs alone leave SMs idle — 16 ways for one or two rows, fewer
// as the rows grow — and, whatever the row count, so that no block walks more than ~128 keys: at 32 sequences x 1024
// keys the unsplit kernel is a chain of 260 dependent iterations per block (measured 6 ms of attention per step of the
// 8B shape; the KV bytes need 0.7 ms). The count is a power of two up to 16 and part of the step graph's key.
int Engine::step_splits(int T) const {
    if (T <= ATT_SPLIT_TOKENS && attention_takes_mma(T, step_ctx_, d.n_heads, d.n_kv_heads, d.head_dim)) {
        // tensor-core kernel, a block per (KV head, token, split): enough blocks to fill the SMs three deep, but no range
        // shorter than 256 keys (4 pages per warp) — its fixed cost per block (query fragments, warp merge) is larger
        int want = 1, limit = 1;
        while (want < ATT_SPLITS && d.n_kv_heads * T * want < 444) want <<= 1;
        while (limit < ATT_SPLITS && limit * 2 * 256 <= step_ctx_) limit <<= 1;
        return std::min(want, limit);
    }
    int splits = 1;
    if (T <= imma_rows_per_pass()) splits = d.n_heads * T <= 64 ? ATT_SPLITS : d.n_heads * T <= 128 ? 8 : 4;
    if (T <= ATT_SPLIT_TOKENS) {
        int by_ctx = 1;
        while (by_ctx < ATT_SPLITS && by_ctx * 128 < step_ctx_) by_ctx <<= 1;
        splits = std::max(splits, by_ctx);
    }
    return splits;
}

// Attention of the T staged tokens, then the output projection added into x_ (x += W_o attn (+ b_o)).
int Engine::attention_and_oproj(const LayerW& w, int l, int T) {
    const int H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim, hid = d.hidden;
    const int qkv_ld = (H + 2 * Hkv) * hd;
    const float scale = 1.0f / sqrtf((float)hd);
    // Keys are split over several blocks only while (token, head) pairs alone leave SMs idle: 16 ways for one or two
    // rows, fewer as the rows grow, not at all from 17 rows on (measured on the 8B shape at context 300: 16 rows 0.89 ms
    // of attention per step with 4 splits against 1.37 with 16; 32 rows 0.54 ms unsplit against 2.34).
    const int splits = step_splits(T);
    ImmaArgs ia;
    if (splits > 1 && use_ring && d.tp_size == 1 && !trace_on && T <= RING_MAX_M && all_tiled(w.o)) {
        // split-K attention merged to f32 rows; the output projection quantises them itself
        SP_LAUNCH(F_ATTN, launch_attention(qkv_, qkv_ld, attn_, H * hd, T, H, d_tok_slot_, d_tok_pos_, kv_, l, scale, splits, att_scratch_, stream, step_ctx_));
        bool done = false;
        SP_TRY(try_ring(&done, T, H * hd, RING_SRC_PLAIN, attn_, H * hd, nullptr, nullptr, w.o, w.ob, x_, hid, nullptr, nullptr, nullptr, nullptr,
                        nullptr, nullptr, x_));
        if (done) return SP_OK;
        return gemv(attn_, H * hd, T, H * hd, w.o, w.ob, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, nullptr, true);
    }
    if (splits > 1 && !trace_on && all_tiled(w.o) && plan_digits(T, H * hd, ia)) {
        SP_LAUNCH(F_ATTN, launch_attention_split(qkv_, qkv_ld, T, H, d_tok_slot_, d_tok_pos_, kv_, l, scale, splits, att_scratch_, stream, step_ctx_));
        SP_LAUNCH(F_ATTN, launch_attn_merge_quant(att_scratch_, H, splits, hd, nullptr, 0, ia, stream));
        return gemv(attn_, H * hd, T, H * hd, w.o, w.ob, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, &ia, true);
    }
    // a prefill chunk (one sequence, consecutive positions): the tiled tensor-core kernel
    // (takes the sequence and its first position as launch arguments: not inside a captured step, which is replayed)
    bool one_seq = splits == 1 && !graph_step_ && use_tc5 && !tc5_exact && attention_prefill_supported(hd);
    for (int i = 1; one_seq && i < T; ++i) one_seq = p_slot_[i] == p_slot_[0] && p_pos_[i] == p_pos_[0] + i;
    if (one_seq && big_m(T, H * hd, w.o)) {
        SP_LAUNCH(F_ATTN, launch_attention_prefill(qkv_, qkv_ld, nullptr, H * hd, T, H, p_slot_[0], p_pos_[0], kv_, l, scale, stream, ws_.xh));
        return gemm_xh_sum(T, H * hd, w.o, w.ob);
    }
    if (one_seq) {
        SP_LAUNCH(F_ATTN, launch_attention_prefill(qkv_, qkv_ld, attn_, H * hd, T, H, p_slot_[0], p_pos_[0], kv_, l, scale, stream));
        return gemv(attn_, H * hd, T, H * hd, w.o, w.ob, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, nullptr, true);
    }
    SP_LAUNCH(F_ATTN, launch_attention(qkv_, qkv_ld, attn_, H * hd, T, H, d_tok_slot_, d_tok_pos_, kv_, l, scale, splits, att_scratch_,
                                       stream, step_ctx_));
    return gemv(attn_, H * hd, T, H * hd, w.o, w.ob, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, nullptr, true);
}

int Engine::layer_llama(const LayerW& w, int l, int T) {
    const int H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim, hid = d.hidden, ffn = d.ffn;
    const int qkv_ld = (H + 2 * Hkv) * hd;
    ImmaArgs ia;
    bool ringed = false;
    SP_TRY(try_ring(&ringed, T, hid, RING_SRC_RMS, x_, hid, w.n1w, nullptr, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd));
    if (ringed) {
    } else if (big_m(T, hid, w.q, w.k, w.v)) {
        SP_TRY(tp_resolve(T));
        SP_LAUNCH(F_NORM, launch_rms_norm_f16(x_, w.n1w, T, hid, d.norm_eps, ws_.xh, stream));
        SP_TRY(gemm_xh(T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb, qkv_ + (size_t)(H + Hkv) * hd));
    } else if (all_tiled(w.q, w.k, w.v) && plan_digits(T, hid, ia)) {
        SP_LAUNCH(F_NORM, launch_norm_quant(x_, hid, w.n1w, nullptr, false, d.norm_eps, nullptr, 0, ia, stream, tp_take()));
        SP_TRY(gemv(h_, hid, T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd, nullptr, &ia));
    } else {
        SP_TRY(tp_resolve(T));
        SP_LAUNCH(F_NORM, launch_rms_norm(x_, w.n1w, T, hid, d.norm_eps, h_, stream));
        SP_TRY(gemv(h_, hid, T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd));
    }
    SP_LAUNCH(F_ROPE, launch_rope_kv_append(qkv_, T, H, Hkv, hd, d.rotary_dim, cos_sin_, d_tok_slot_, d_tok_pos_, kv_, l, kv_round, stream));
    SP_TRY(attention_and_oproj(w, l, T));
    SP_TRY(try_ring(&ringed, T, hid, RING_SRC_RMS, x_, hid, w.n2w, nullptr, w.gate, nullptr, gu_, 2 * ffn, w.up, nullptr, gu_ + ffn));
    if (ringed) {
    } else if (big_m(T, hid, w.gate, w.up)) {
        SP_TRY(tp_resolve(T));
        SP_LAUNCH(F_NORM, launch_rms_norm_f16(x_, w.n2w, T, hid, d.norm_eps, ws_.xh, stream));
        SP_TRY(gemm_xh(T, hid, w.gate, nullptr, gu_, 2 * ffn, w.up, nullptr, gu_ + ffn));
    } else if (all_tiled(w.gate, w.up) && plan_digits(T, hid, ia)) {
        SP_LAUNCH(F_NORM, launch_norm_quant(x_, hid, w.n2w, nullptr, false, d.norm_eps, nullptr, 0, ia, stream, tp_take()));
        SP_TRY(gemv(h_, hid, T, hid, w.gate, nullptr, gu_, 2 * ffn, w.up, nullptr, gu_ + ffn, nullptr, nullptr, nullptr, nullptr, &ia));
    } else {
        SP_TRY(tp_resolve(T));
        SP_LAUNCH(F_NORM, launch_rms_norm(x_, w.n2w, T, hid, d.norm_eps, h_, stream));
        SP_TRY(gemv(h_, hid, T, hid, w.gate, nullptr, gu_, 2 * ffn, w.up, nullptr, gu_ + ffn));
    }
    SP_TRY(try_ring(&ringed, T, ffn, RING_SRC_SWIGLU, gu_, 2 * ffn, nullptr, nullptr, w.down, nullptr, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr,
                    nullptr, x_));
    if (ringed) {
    } else if (big_m(T, ffn, w.down)) {
        SP_LAUNCH(F_ELEM, launch_act_f16(gu_, 2 * ffn, ffn, T, 0, ws_.xh, stream));
        SP_TRY(gemm_xh_sum(T, ffn, w.down, nullptr));
    } else if (all_tiled(w.down) && plan_digits(T, ffn, ia)) {
        SP_LAUNCH(F_ELEM, launch_act_fn_quant(gu_, 2 * ffn, ffn, 0, ia, stream));
        SP_TRY(gemv(mid_, ffn, T, ffn, w.down, nullptr, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, &ia, true));
    } else {
        SP_LAUNCH(F_ELEM, launch_swiglu(gu_, 2 * ffn, ffn, T, mid_, stream));
        SP_TRY(gemv(mid_, ffn, T, ffn, w.down, nullptr, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, nullptr, true));
    }
    return SP_OK;
}

int Engine::layer_phi(const LayerW& w, int l, int T) {
    const int H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim, hid = d.hidden, ffn = d.ffn;
    const int qkv_ld = (H + 2 * Hkv) * hd;
    // parallel block: x + (attn_out + mlp(h)); both branches read the same normalised input h
    ImmaArgs ia;
    bool ringed = false, ringed2 = false;
    SP_TRY(try_ring(&ringed, T, hid, RING_SRC_LN, x_, hid, w.n1w, w.n1b, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd));
    if (ringed) SP_TRY(try_ring(&ringed2, T, hid, RING_SRC_LN, x_, hid, w.n1w, w.n1b, w.up, w.upb, gu_, ffn));
    if (ringed && !ringed2) {
        // fc1 does not fit the ring kernel: the separate norm feeds it
        SP_LAUNCH(F_NORM, launch_layer_norm(x_, w.n1w, w.n1b, T, hid, d.norm_eps, h_, stream));
        SP_TRY(gemv(h_, hid, T, hid, w.up, w.upb, gu_, ffn));
    }
    if (ringed) {
    } else if (big_m(T, hid, w.q, w.k, w.v) && big_m(T, hid, w.up)) {
        SP_LAUNCH(F_NORM, launch_layer_norm_f16(x_, w.n1w, w.n1b, T, hid, d.norm_eps, ws_.xh, stream));
        SP_TRY(gemm_xh(T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb, qkv_ + (size_t)(H + Hkv) * hd));
        SP_TRY(gemm_xh(T, hid, w.up, w.upb, gu_, ffn));
    } else if (all_tiled(w.q, w.k, w.v) && all_tiled(w.up) && plan_digits(T, hid, ia)) {
        SP_LAUNCH(F_NORM, launch_norm_quant(x_, hid, w.n1w, w.n1b, true, d.norm_eps, nullptr, 0, ia, stream));
        SP_TRY(gemv(h_, hid, T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd, nullptr, &ia));
        SP_TRY(gemv(h_, hid, T, hid, w.up, w.upb, gu_, ffn, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &ia));
    } else {
        SP_LAUNCH(F_NORM, launch_layer_norm(x_, w.n1w, w.n1b, T, hid, d.norm_eps, h_, stream));
        SP_TRY(gemv(h_, hid, T, hid, w.q, w.qb, qkv_, qkv_ld, w.k, w.kb, qkv_ + (size_t)H * hd, w.v, w.vb,
                    qkv_ + (size_t)(H + Hkv) * hd));
        SP_TRY(gemv(h_, hid, T, hid, w.up, w.upb, gu_, ffn));
    }
    SP_LAUNCH(F_ROPE, launch_rope_kv_append(qkv_, T, H, Hkv, hd, d.rotary_dim, cos_sin_, d_tok_slot_, d_tok_pos_, kv_, l, kv_round, stream));
    // the MLP's fc1 output waits in gu_ while the workspace serves the attention output projection
    SP_TRY(attention_and_oproj(w, l, T));
    SP_TRY(try_ring(&ringed, T, ffn, RING_SRC_GELU, gu_, ffn, nullptr, nullptr, w.down, w.downb, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr,
                    nullptr, x_));
    if (ringed) {
    } else if (big_m(T, ffn, w.down)) {
        SP_LAUNCH(F_ELEM, launch_act_f16(gu_, ffn, ffn, T, 1, ws_.xh, stream));
        SP_TRY(gemm_xh(T, ffn, w.down, w.downb, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_));
    } else if (all_tiled(w.down) && plan_digits(T, ffn, ia)) {
        SP_LAUNCH(F_ELEM, launch_act_fn_quant(gu_, ffn, ffn, 1, ia, stream));
        SP_TRY(gemv(mid_, ffn, T, ffn, w.down, w.downb, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_, &ia));
    } else {
        SP_CUDA_TRY(cudaMemcpyAsync(mid_, gu_, (size_t)T * ffn * 4, cudaMemcpyDeviceToDevice, stream));
        SP_LAUNCH(F_ELEM, launch_gelu(mid_, (int64_t)T * ffn, stream));
        SP_TRY(gemv(mid_, ffn, T, ffn, w.down, w.downb, x_, hid, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, x_));
    }
    return SP_OK;
}

}  // namespace sp
