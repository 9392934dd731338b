// Causal GQA attention over the paged fp16 KV cache, split over the keys (flash-decoding).
//
// Block (head h, token t, split s) runs the reference's online-softmax recurrence
// (crates/sapient-backends/cpu/src/kernels/attention.rs:98-165) over its share of the keys
// 0..pos of the token's sequence: warps stride over the keys four at a time, lanes split
// head_dim in (even, odd) pairs, scores come from warp shuffles, and every state (m, l, o) is
// merged with the log-sum-exp correction — first across the block's warps, then across the
// splits by a second small kernel. K and V are fp16 in the cache, all arithmetic is f32.
// With one split the block writes the output row directly.
#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_PAIRS = 4;  // head_dim <= 256
constexpr int ATT_KEYS = 4;       // keys per warp iteration

__device__ __forceinline__ int64_t kv_off(const KvGeom& kv, int layer, int page, int which, int head) {
    return ((((int64_t)layer * kv.n_pages + page) * 2 + which) * kv.n_kv + head) * (int64_t)(KV_PAGE * kv.head_dim);
}

// part: [n_tok][n_heads][n_splits][head_dim + 2] = (m, l, o[head_dim]); unused when n_splits == 1.
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_split_kernel(const float* __restrict__ q, int ldq, float* __restrict__ out, int ldo, int n_heads,
                       const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos, KvGeom kv, int layer,
                       float scale, int n_splits, float* __restrict__ part) {
    __shared__ float sh_m[ATT_WARPS], sh_l[ATT_WARPS];
    __shared__ float sh_o[ATT_WARPS][256];
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, t = blockIdx.y, sp = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = kv.head_dim, npairs = hd >> 1;
    const int slot = tok_slot[t], n_keys = tok_pos[t] + 1;
    // this split's key range
    const int per = (n_keys + n_splits - 1) / n_splits;
    const int k_begin = sp * per, k_end = min(n_keys, k_begin + per);
    const int kv_h = h / (n_heads / kv.n_kv);
    const float* qrow = q + (int64_t)t * ldq + (int64_t)h * hd;
    float2 qv[ATT_MAX_PAIRS], o[ATT_MAX_PAIRS];
#pragma unroll
    for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
        const int p = lane + 32 * i;
        qv[i] = (p < npairs) ? make_float2(qrow[2 * p], qrow[2 * p + 1]) : make_float2(0.f, 0.f);
        o[i] = make_float2(0.f, 0.f);
    }
    float m = -INFINITY, l = 0.f;
    const int32_t* pt = kv.page_table + (int64_t)slot * kv.max_pages;
    for (int key0 = k_begin + warp * ATT_KEYS; key0 < k_end; key0 += ATT_WARPS * ATT_KEYS) {
        // all K and V fragments of the four keys are requested before any arithmetic, so the V loads do not wait
        // for the scores
        __half2 kr[ATT_KEYS][ATT_MAX_PAIRS], vr[ATT_KEYS][ATT_MAX_PAIRS];
        float s[ATT_KEYS];
#pragma unroll
        for (int j = 0; j < ATT_KEYS; ++j) {
            const int key = min(key0 + j, k_end - 1);  // tail keys repeat the last one and get weight 0
            const int page = pt[key / KV_PAGE];
            const __half2* kp = reinterpret_cast<const __half2*>(kv.pool + kv_off(kv, layer, page, 0, kv_h) + (int64_t)(key % KV_PAGE) * hd);
            const __half2* vp = reinterpret_cast<const __half2*>(kv.pool + kv_off(kv, layer, page, 1, kv_h) + (int64_t)(key % KV_PAGE) * hd);
#pragma unroll
            for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
                const int p = lane + 32 * i;
                kr[j][i] = (p < npairs) ? kp[p] : __half2();
                vr[j][i] = (p < npairs) ? vp[p] : __half2();
            }
        }
#pragma unroll
        for (int j = 0; j < ATT_KEYS; ++j) {
            float part_dot = 0.f;
#pragma unroll
            for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
                if (lane + 32 * i < npairs) {
                    const float2 kf = __half22float2(kr[j][i]);
                    part_dot = fmaf(qv[i].x, kf.x, part_dot);
                    part_dot = fmaf(qv[i].y, kf.y, part_dot);
                }
            }
            s[j] = part_dot;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
            for (int j = 0; j < ATT_KEYS; ++j) s[j] += __shfl_xor_sync(0xFFFFFFFFu, s[j], off);
        float m_new = m;
#pragma unroll
        for (int j = 0; j < ATT_KEYS; ++j) {
            s[j] = (key0 + j < k_end) ? s[j] * scale : -INFINITY;
            m_new = fmaxf(m_new, s[j]);
        }
        const float corr = expf(m - m_new);  // the first key of the range is always live, so m_new is finite
        float pw[ATT_KEYS], psum = 0.f;
#pragma unroll
        for (int j = 0; j < ATT_KEYS; ++j) { pw[j] = expf(s[j] - m_new); psum += pw[j]; }
#pragma unroll
        for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
            if (lane + 32 * i < npairs) {
                float ox = corr * o[i].x, oy = corr * o[i].y;
#pragma unroll
                for (int j = 0; j < ATT_KEYS; ++j) {
                    const float2 vf = __half22float2(vr[j][i]);
                    ox = fmaf(pw[j], vf.x, ox);
                    oy = fmaf(pw[j], vf.y, oy);
                }
                o[i].x = ox; o[i].y = oy;
            }
        }
        l = fmaf(corr, l, psum);
        m = m_new;
    }
    if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
        const int p = lane + 32 * i;
        if (p < npairs) { sh_o[warp][2 * p] = o[i].x; sh_o[warp][2 * p + 1] = o[i].y; }
    }
    __syncthreads();
    float M = sh_m[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) M = fmaxf(M, sh_m[w]);
    float L = 0.f, cw[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        cw[w] = (sh_m[w] == -INFINITY) ? 0.f : expf(sh_m[w] - M);
        L = fmaf(cw[w], sh_l[w], L);
    }
    if (n_splits == 1) {
        const float inv = (L == 0.f) ? 0.f : 1.0f / L;
        for (int e = threadIdx.x; e < hd; e += blockDim.x) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) acc = fmaf(cw[w], sh_o[w][e], acc);
            out[(int64_t)t * ldo + (int64_t)h * hd + e] = acc * inv;
        }
    } else {
        float* dst = part + (((int64_t)t * n_heads + h) * n_splits + sp) * (hd + 2);
        if (threadIdx.x == 0) { dst[0] = M; dst[1] = L; }
        for (int e = threadIdx.x; e < hd; e += blockDim.x) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) acc = fmaf(cw[w], sh_o[w][e], acc);
            dst[2 + e] = acc;  // un-normalised, relative to M
        }
    }
}

bool attention_gqa_mma_supported(int n_heads, int n_kv, int head_dim);
bool attention_takes_mma(int n_tok, int ctx_hint, int n_heads, int n_kv, int head_dim) {
    return (int64_t)n_tok * ctx_hint >= 4096 && attention_gqa_mma_supported(n_heads, n_kv, head_dim);
}
cudaError_t launch_gqa_mma_phase(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                                 const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st);

// Which kernel a launch takes. ctx_hint: an upper bound of the longest context among the tokens (0: unknown). Short work
// is latency-bound and runs on the f32 kernel, a block per (head, token, split); from a few thousand (token, key) pairs
// on, grouped-query shapes take the tensor-core kernel, which reads the K / V rows once per group of query heads (the
// f32 kernel re-reads them once per query head, and at 32 sequences x 1024 keys spends 5.4 ms per step of the 8B shape
// on 4.4 GB of KV; the tensor-core kernel 1.5 ms).
static cudaError_t launch_split_phase(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                                      const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st,
                                      int ctx_hint) {
    if (attention_takes_mma(n_tok, ctx_hint, n_heads, kv.n_kv, kv.head_dim))
        return launch_gqa_mma_phase(q, ldq, out, ldo, n_tok, n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch, st);
    return launch_pdl(attention_split_kernel, dim3(n_heads, n_tok, n_splits), dim3(ATT_WARPS * 32), 0, st, q, ldq, out, ldo, n_heads, tok_slot,
                      tok_pos, kv, layer, scale, n_splits, scratch);
}

__global__ void attention_merge_kernel(const float* __restrict__ part, int n_heads, int n_splits, int hd, float* __restrict__ out,
                                       int ldo) {
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, t = blockIdx.y;
    const float* src = part + ((int64_t)t * n_heads + h) * n_splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, src[(int64_t)s * (hd + 2)]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = src[(int64_t)s * (hd + 2)];
        if (ms != -INFINITY) L = fmaf(expf(ms - M), src[(int64_t)s * (hd + 2) + 1], L);
    }
    const float inv = (L == 0.f) ? 0.f : 1.0f / L;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = src[(int64_t)s * (hd + 2)];
            if (ms != -INFINITY) acc = fmaf(expf(ms - M), src[(int64_t)s * (hd + 2) + 2 + e], acc);
        }
        out[(int64_t)t * ldo + (int64_t)h * hd + e] = acc * inv;
    }
}

size_t attention_scratch_floats(int n_tok, int n_heads, int n_splits, int head_dim) {
    return n_splits > 1 ? (size_t)n_tok * n_heads * n_splits * (head_dim + 2) : 0;
}

cudaError_t launch_attention_split(const float* q, int ldq, int n_tok, int n_heads, const int32_t* tok_slot, const int32_t* tok_pos,
                                   KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st, int ctx_hint) {
    if (n_tok == 0) return cudaSuccess;
    if (n_splits < 2 || !scratch) return cudaErrorInvalidValue;
    cudaError_t le = launch_split_phase(q, ldq, nullptr, 0, n_tok, n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch, st, ctx_hint);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_attention(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                             const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch,
                             cudaStream_t st, int ctx_hint) {
    if (n_tok == 0) return cudaSuccess;
    if (n_splits < 1 || (n_splits > 1 && !scratch)) return cudaErrorInvalidValue;
    cudaError_t le = launch_split_phase(q, ldq, out, ldo, n_tok, n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch, st, ctx_hint);
    if (le != cudaSuccess) return le;
    cudaError_t e = count_launch_and_check();
    if (e != cudaSuccess || n_splits == 1) return e;
    le = launch_pdl(attention_merge_kernel, dim3(n_heads, n_tok), dim3(128), 0, st, (const float*)scratch, n_heads, n_splits, kv.head_dim, out, ldo);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

}  // namespace sp

// ───────────────────────────── prefill: tiled attention on tensor cores ─────────────────────────────
// Many query tokens of ONE sequence with consecutive positions (a prefill chunk). The split kernel above re-reads the
// whole key range once per query token; here a block takes 64 query rows of one head (4 warps x 16 rows), walks the keys
// in tiles of 64 (4 pages) staged in shared memory, and does both contractions with mma.sync.m16n8k16 (fp16 operands —
// K and V are fp16 in the cache already, q and the softmax weights are rounded to fp16 — f32 accumulation), with the
// reference's online-softmax recurrence (kernels/attention.rs:98-165) applied per 64-key tile.
namespace sp {

constexpr int FA_ROWS = 64, FA_KEYS = 64, FA_WARPS = 4;

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// HD16 = head_dim / 16 (head_dim a multiple of 16, <= 128).
template <int HD16>
__global__ void __launch_bounds__(FA_WARPS * 32)
attention_prefill_kernel(const float* __restrict__ q, int ldq, float* __restrict__ out, __half* __restrict__ out_h, int ldo, int n_tok,
                         int n_heads, int slot, int pos0, KvGeom kv, int layer, float scale) {
    constexpr int HD = HD16 * 16, LD = HD + 8;  // padded row of the shared tiles (halves): conflict-free fragment loads
    extern __shared__ __align__(16) __half fa_smem[];
    // two (K, V) tile buffers: cp.async fills one while the tensor cores work on the other
    constexpr int TILE = FA_KEYS * LD;
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, t0 = blockIdx.y * FA_ROWS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kv_h = h / (n_heads / kv.n_kv);
    const int32_t* pt = kv.page_table + (int64_t)slot * kv.max_pages;
    // this thread's two query rows (rows past the chunk repeat the last one and are never written)
    const int r0 = t0 + warp * 16 + g, r1 = r0 + 8;
    const int q0 = min(r0, n_tok - 1), q1 = min(r1, n_tok - 1);
    const int p0 = pos0 + q0, p1 = pos0 + q1;
    uint32_t qa[HD16][4];
    {
        const float* a = q + (int64_t)q0 * ldq + (int64_t)h * HD;
        const float* b = q + (int64_t)q1 * ldq + (int64_t)h * HD;
#pragma unroll
        for (int kd = 0; kd < HD16; ++kd) {
            const float2 x0 = *reinterpret_cast<const float2*>(a + 16 * kd + 2 * t), x1 = *reinterpret_cast<const float2*>(b + 16 * kd + 2 * t);
            const float2 x2 = *reinterpret_cast<const float2*>(a + 16 * kd + 8 + 2 * t), x3 = *reinterpret_cast<const float2*>(b + 16 * kd + 8 + 2 * t);
            qa[kd][0] = pack_half2(x0.x * scale, x0.y * scale); qa[kd][1] = pack_half2(x1.x * scale, x1.y * scale);
            qa[kd][2] = pack_half2(x2.x * scale, x2.y * scale); qa[kd][3] = pack_half2(x3.x * scale, x3.y * scale);
        }
    }
    float o[2 * HD16][4];
#pragma unroll
    for (int i = 0; i < 2 * HD16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int last_pos = pos0 + min(t0 + FA_ROWS, n_tok) - 1;  // newest key any row of the block may see
    auto fetch_tile = [&](int k0, int buf) {  // asynchronous copy of keys k0 .. k0 + 63 (zeros past the newest visible key)
        __half* Kd = fa_smem + (2 * buf) * TILE;
        __half* Vd = Kd + TILE;
        for (int idx = threadIdx.x; idx < FA_KEYS * (HD / 8); idx += FA_WARPS * 32) {
            const int kr = idx / (HD / 8), pc = idx - kr * (HD / 8);
            const int key = k0 + kr;
            const bool live = key <= last_pos;
            const int page = live ? pt[key / KV_PAGE] : 0;
            const int64_t in_page = (int64_t)((live ? key : 0) % KV_PAGE) * HD + pc * 8;
            const __half* ksrc = kv.pool + kv_off(kv, layer, page, 0, kv_h) + in_page;
            const __half* vsrc = kv.pool + kv_off(kv, layer, page, 1, kv_h) + in_page;
            const uint32_t kd = (uint32_t)__cvta_generic_to_shared(Kd + kr * LD + pc * 8), vd = (uint32_t)__cvta_generic_to_shared(Vd + kr * LD + pc * 8);
            const int bytes = live ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(kd), "l"(ksrc), "r"(bytes) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vd), "l"(vsrc), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    fetch_tile(0, 0);
    for (int k0 = 0, buf = 0; k0 <= last_pos; k0 += FA_KEYS, buf ^= 1) {
        const __half* Ks = fa_smem + (2 * buf) * TILE;
        const __half* Vs = Ks + TILE;
        if (k0 + FA_KEYS <= last_pos) {
            fetch_tile(k0 + FA_KEYS, buf ^ 1);  // that buffer's previous tile was consumed before the barrier that ended the last iteration
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();  // everyone's copies of this tile have landed
        // S = (q * scale) K^T for 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kd = 0; kd < HD16; ++kd) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ks + (8 * j + g) * LD + 16 * kd + 2 * t);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ks + (8 * j + g) * LD + 16 * kd + 8 + 2 * t);
                mma_f16(s[j], qa[kd][0], qa[kd][1], qa[kd][2], qa[kd][3], b0, b1);
            }
        }
        // causal mask and the tile's row maxima (row g: s[j][0..1], row g+8: s[j][2..3]; keys 8j + 2t, +1)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int key = k0 + 8 * j + 2 * t;
            if (key > p0) s[j][0] = -INFINITY;
            if (key + 1 > p0) s[j][1] = -INFINITY;
            if (key > p1) s[j][2] = -INFINITY;
            if (key + 1 > p1) s[j][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        // a row whose keys of this tile are all masked keeps its state (n == m); key 0 is visible to every row, so
        // after the first tile every maximum is finite
        const float c0 = (n0 == -INFINITY) ? 1.f : expf(m0 - n0), c1 = (n1 == -INFINITY) ? 1.f : expf(m1 - n1);
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pa[4][4];  // softmax weights as fp16 A fragments: k-step kk covers keys 16 kk .. + 15
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float e0 = (s[j][0] == -INFINITY) ? 0.f : expf(s[j][0] - n0), e1 = (s[j][1] == -INFINITY) ? 0.f : expf(s[j][1] - n0);
            const float e2 = (s[j][2] == -INFINITY) ? 0.f : expf(s[j][2] - n1), e3 = (s[j][3] == -INFINITY) ? 0.f : expf(s[j][3] - n1);
            sum0 += e0 + e1;
            sum1 += e2 + e3;
            pa[j >> 1][(j & 1) * 2] = pack_half2(e0, e1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_half2(e2, e3);
        }
        sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 1); sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 2);
        sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 1); sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 2);
        l0 = fmaf(c0, l0, sum0); l1 = fmaf(c1, l1, sum1);
        m0 = n0; m1 = n1;
#pragma unroll
        for (int nd = 0; nd < 2 * HD16; ++nd) { o[nd][0] *= c0; o[nd][1] *= c0; o[nd][2] *= c1; o[nd][3] *= c1; }
        // O += P V: B fragments (keys x dims) come transposed out of the row-major V tile
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int nd = 0; nd < 2 * HD16; nd += 2) {
                uint32_t b0, b1, b2, b3;
                const __half* src = Vs + (16 * kk + (lane & 15)) * LD + 8 * (nd + (lane >> 4));
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(src);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                             : "r"(addr));
                mma_f16(o[nd], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                mma_f16(o[nd + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
        __syncthreads();  // this tile's buffer may be refilled from the next iteration on
    }
    const float i0 = (l0 == 0.f) ? 0.f : 1.0f / l0, i1 = (l1 == 0.f) ? 0.f : 1.0f / l1;
#pragma unroll
    for (int nd = 0; nd < 2 * HD16; ++nd) {
        const int64_t c = (int64_t)h * HD + 8 * nd + 2 * t;
        if (out_h) {  // fp16 rows for the tensor-core output projection
            if (r0 < n_tok) *reinterpret_cast<__half2*>(out_h + (int64_t)r0 * ldo + c) = __floats2half2_rn(o[nd][0] * i0, o[nd][1] * i0);
            if (r1 < n_tok) *reinterpret_cast<__half2*>(out_h + (int64_t)r1 * ldo + c) = __floats2half2_rn(o[nd][2] * i1, o[nd][3] * i1);
        } else {
            if (r0 < n_tok) *reinterpret_cast<float2*>(out + (int64_t)r0 * ldo + c) = make_float2(o[nd][0] * i0, o[nd][1] * i0);
            if (r1 < n_tok) *reinterpret_cast<float2*>(out + (int64_t)r1 * ldo + c) = make_float2(o[nd][2] * i1, o[nd][3] * i1);
        }
    }
}

// ───────────────── decode-shaped attention on tensor cores: the query heads of a GQA group as one tile ─────────────────
// Block (KV head, token, split), 4 warps. A warp walks 16-key pages of the split's range; a page of one KV head is
// a contiguous [16 keys][head_dim] fp16 run for K and one for V, copied asynchronously (double buffered per warp) into
// padded shared-memory rows. Both contractions run on mma.sync.m16n8k16 with the GROUP's query heads as the M rows, so
// K and V are read once for all heads of the group and no shuffle reduction or scalar FMA touches them.
// Precision stays that of the f32 kernels: the 16 M rows hold, for head g < 8, the fp16 leading part of its (f32) query
// row in row g and the fp16 remainder in row g + 8 (q = hi + lo to 2^-22); the two accumulator rows are added. The
// softmax weights are split the same way for the second contraction. K and V are fp16 in the cache, hence exact.
// Online softmax per page with the reference's recurrence (kernels/attention.rs:98-165); the warps' states are merged
// through shared memory, and the block writes either the output rows (one split) or the split partials.
constexpr int GM_WARPS = 4;
template <int HD16>
__global__ void __launch_bounds__(GM_WARPS * 32)
attention_gqa_mma_kernel(const float* __restrict__ q, int ldq, float* __restrict__ out, int ldo, int n_heads, const int32_t* __restrict__ tok_slot,
                         const int32_t* __restrict__ tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* __restrict__ part) {
    constexpr int HD = HD16 * 16, LD = HD + 8, TILE = KV_PAGE * LD;
    extern __shared__ __align__(16) __half gm_smem[];
    pdl_wait();
    pdl_trigger();
    const int kv_h = blockIdx.x, tok = blockIdx.y, sp = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = n_heads / kv.n_kv;
    const int slot = tok_slot[tok], n_keys = tok_pos[tok] + 1;
    const int n_pg = (n_keys + KV_PAGE - 1) / KV_PAGE;
    const int per = (n_pg + n_splits - 1) / n_splits;
    const int p_begin = sp * per, p_end = min(n_pg, p_begin + per);
    const int32_t* pt = kv.page_table + (int64_t)slot * kv.max_pages;
    __half* my = gm_smem + (size_t)warp * 4 * TILE;  // [buffer][K | V][16][LD]
    // query fragments: rows g (leading fp16 part) and g + 8 (remainder) of head kv_h * group + g
    uint32_t qa[HD16][4];
    {
        const bool live = g < group;
        const float* row = q + (int64_t)tok * ldq + (int64_t)(kv_h * group + (live ? g : 0)) * HD;
#pragma unroll
        for (int kd = 0; kd < HD16; ++kd) {
            float2 x0 = *reinterpret_cast<const float2*>(row + 16 * kd + 2 * t), x2 = *reinterpret_cast<const float2*>(row + 16 * kd + 8 + 2 * t);
            if (!live) { x0 = make_float2(0.f, 0.f); x2 = x0; }
            const __half2 h0 = __floats2half2_rn(x0.x, x0.y), h2 = __floats2half2_rn(x2.x, x2.y);
            const float2 f0 = __half22float2(h0), f2 = __half22float2(h2);
            qa[kd][0] = *reinterpret_cast<const uint32_t*>(&h0);
            qa[kd][1] = pack_half2(x0.x - f0.x, x0.y - f0.y);
            qa[kd][2] = *reinterpret_cast<const uint32_t*>(&h2);
            qa[kd][3] = pack_half2(x2.x - f2.x, x2.y - f2.y);
        }
    }
    auto fetch = [&](int pg, int buf) {  // keys 16 pg .. 16 pg + 15 of this KV head; keys past the sequence arrive as zeros
        const int page = pt[pg];
        const __half* ksrc = kv.pool + kv_off(kv, layer, page, 0, kv_h);
        const __half* vsrc = kv.pool + kv_off(kv, layer, page, 1, kv_h);
        __half* Kd = my + (size_t)buf * 2 * TILE;
        __half* Vd = Kd + TILE;
#pragma unroll
        for (int it = 0; it < (KV_PAGE * HD / 8) / 32; ++it) {
            const int idx = it * 32 + lane, kr = idx / (HD / 8), pc = idx - kr * (HD / 8);
            const int bytes = (pg * KV_PAGE + kr < n_keys) ? 16 : 0;
            const uint32_t kd = (uint32_t)__cvta_generic_to_shared(Kd + kr * LD + pc * 8), vd = (uint32_t)__cvta_generic_to_shared(Vd + kr * LD + pc * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(kd), "l"(ksrc + kr * HD + pc * 8), "r"(bytes) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vd), "l"(vsrc + kr * HD + pc * 8), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    float o[2 * HD16][4];
#pragma unroll
    for (int i = 0; i < 2 * HD16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m = -INFINITY, l = 0.f;  // head g's running maximum (the same in its four lanes) and this lane's share of the denominator
    int pg = p_begin + warp;
    if (pg < p_end) fetch(pg, 0);
    for (int buf = 0; pg < p_end; pg += GM_WARPS, buf ^= 1) {
        if (pg + GM_WARPS < p_end) {
            fetch(pg + GM_WARPS, buf ^ 1);  // that buffer was consumed before the __syncwarp that ended the last iteration
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncwarp();  // every lane's copies of this page have landed
        const __half* Ks = my + (size_t)buf * 2 * TILE;
        const __half* Vs = Ks + TILE;
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kd = 0; kd < HD16; ++kd) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ks + (8 * j + g) * LD + 16 * kd + 2 * t);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ks + (8 * j + g) * LD + 16 * kd + 8 + 2 * t);
                mma_f16(s[j], qa[kd][0], qa[kd][1], qa[kd][2], qa[kd][3], b0, b1);
            }
        }
        // scores of head g for keys 16 pg + 8 j + 2 t (+1): leading + remainder rows, then the scale
        float sc[2][2], mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int key = pg * KV_PAGE + 8 * j + 2 * t;
            sc[j][0] = (key < n_keys) ? (s[j][0] + s[j][2]) * scale : -INFINITY;
            sc[j][1] = (key + 1 < n_keys) ? (s[j][1] + s[j][3]) * scale : -INFINITY;
            mx = fmaxf(mx, fmaxf(sc[j][0], sc[j][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float mn = fmaxf(m, mx);  // finite: the first key of every page in range is live
        const float c = expf(m - mn);
        uint32_t pa[4];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float e0 = expf(sc[j][0] - mn), e1 = expf(sc[j][1] - mn);  // exp(-inf) = 0 for masked keys
            sum += e0 + e1;
            const __half2 hh = __floats2half2_rn(e0, e1);
            const float2 hf = __half22float2(hh);
            pa[2 * j] = *reinterpret_cast<const uint32_t*>(&hh);
            pa[2 * j + 1] = pack_half2(e0 - hf.x, e1 - hf.y);
        }
        l = fmaf(c, l, sum);
        m = mn;
        if (__any_sync(0xFFFFFFFFu, c != 1.0f)) {
#pragma unroll
            for (int nd = 0; nd < 2 * HD16; ++nd) { o[nd][0] *= c; o[nd][1] *= c; o[nd][2] *= c; o[nd][3] *= c; }
        }
#pragma unroll
        for (int nd = 0; nd < 2 * HD16; nd += 2) {
            uint32_t b0, b1, b2, b3;
            const __half* src = Vs + (lane & 15) * LD + 8 * (nd + (lane >> 4));
            const uint32_t addr = (uint32_t)__cvta_generic_to_shared(src);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
            mma_f16(o[nd], pa[0], pa[1], pa[2], pa[3], b0, b1);
            mma_f16(o[nd + 1], pa[0], pa[1], pa[2], pa[3], b2, b3);
        }
        __syncwarp();  // the page's buffer may be refilled from the next iteration on
    }
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);
    // merge of the warps' states (the tile buffers are free once every warp is out of its loop)
    __syncthreads();
    float* sh_m = reinterpret_cast<float*>(gm_smem);          // [warp][8]
    float* sh_l = sh_m + GM_WARPS * 8;                        // [warp][8]
    float* sh_o = sh_l + GM_WARPS * 8;                        // [warp][8][HD]
    if (t == 0) { sh_m[warp * 8 + g] = m; sh_l[warp * 8 + g] = l; }
#pragma unroll
    for (int nd = 0; nd < 2 * HD16; ++nd)
        *reinterpret_cast<float2*>(sh_o + ((size_t)warp * 8 + g) * HD + 8 * nd + 2 * t) = make_float2(o[nd][0] + o[nd][2], o[nd][1] + o[nd][3]);
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += GM_WARPS * 32) {
        const int hg = idx / HD, e = idx - hg * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < GM_WARPS; ++w) M = fmaxf(M, sh_m[w * 8 + hg]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < GM_WARPS; ++w) {
            const float cw = (sh_m[w * 8 + hg] == -INFINITY) ? 0.f : expf(sh_m[w * 8 + hg] - M);
            L = fmaf(cw, sh_l[w * 8 + hg], L);
            acc = fmaf(cw, sh_o[((size_t)w * 8 + hg) * HD + e], acc);
        }
        const int h = kv_h * group + hg;
        if (n_splits == 1) {
            out[(int64_t)tok * ldo + (int64_t)h * HD + e] = acc * ((L == 0.f) ? 0.f : 1.0f / L);
        } else {
            float* dst = part + (((int64_t)tok * n_heads + h) * n_splits + sp) * (HD + 2);
            if (e == 0) { dst[0] = M; dst[1] = L; }
            dst[2 + e] = acc;  // un-normalised, relative to M
        }
    }
}

bool attention_gqa_mma_supported(int n_heads, int n_kv, int head_dim) {
    if (n_kv <= 0 || n_heads % n_kv != 0) return false;
    const int group = n_heads / n_kv;
    return group >= 2 && group <= 8 && head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128;
}

cudaError_t launch_gqa_mma_phase(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                                 const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st) {
    const int hd16 = kv.head_dim / 16;
    const size_t smem = (size_t)GM_WARPS * 4 * KV_PAGE * (kv.head_dim + 8) * sizeof(__half);
    const dim3 grid(kv.n_kv, n_tok, n_splits), block(GM_WARPS * 32);
    cudaError_t le = cudaErrorInvalidValue;
#define SP_GM(N)                                                                                                        \
    if (hd16 == N) {                                                                                                    \
        static PerDeviceOnce big_smem;                                                                                  \
        if (smem > 48 * 1024) {                                                                                         \
            le = big_smem.run([] { return cudaFuncSetAttribute(attention_gqa_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024); }); \
            if (le != cudaSuccess) return le;                                                                           \
        }                                                                                                               \
        le = launch_pdl(attention_gqa_mma_kernel<N>, grid, block, smem, st, q, ldq, out, ldo, n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch); \
    }
    SP_GM(1) SP_GM(2) SP_GM(3) SP_GM(4) SP_GM(5) SP_GM(6) SP_GM(7) SP_GM(8)
#undef SP_GM
    return le;
}

bool attention_prefill_supported(int head_dim) { return head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128; }

// All n_tok tokens belong to sequence `slot` at positions pos0, pos0 + 1, ... (their keys are in the cache already).
// out_h != null: the rows go out as fp16 to out_h (same row stride) instead of f32 to out.
cudaError_t launch_attention_prefill(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, int slot, int pos0, KvGeom kv,
                                     int layer, float scale, cudaStream_t st, __half* out_h) {
    if (n_tok <= 0) return cudaSuccess;
    if (!attention_prefill_supported(kv.head_dim)) return cudaErrorInvalidValue;
    const int hd16 = kv.head_dim / 16;
    const size_t smem = (size_t)4 * FA_KEYS * (kv.head_dim + 8) * sizeof(__half);  // two (K, V) tile buffers
    const dim3 grid(n_heads, (n_tok + FA_ROWS - 1) / FA_ROWS), block(FA_WARPS * 32);
    cudaError_t le = cudaErrorInvalidValue;
#define SP_FA(N)                                                                                                        \
    if (hd16 == N) {                                                                                                    \
        static PerDeviceOnce big_smem;                                                                                  \
        if (smem > 48 * 1024) {                                                                                         \
            le = big_smem.run([] { return cudaFuncSetAttribute(attention_prefill_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024); }); \
            if (le != cudaSuccess) return le;                                                                           \
        }                                                                                                               \
    }                                                                                                                   \
    if (hd16 == N) le = launch_pdl(attention_prefill_kernel<N>, grid, block, smem, st, q, ldq, out, out_h, ldo, n_tok, n_heads, slot, pos0, kv, layer, scale)
    SP_FA(1); SP_FA(2); SP_FA(3); SP_FA(4); SP_FA(5); SP_FA(6); SP_FA(7); SP_FA(8);
#undef SP_FA
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

}  // namespace sp
