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

__global__ void attention_merge_kernel(const float* __restrict__ part, int n_heads, int n_splits, int hd, float* __restrict__ out,
                                       int ldo) {
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
                                   KvGeom kv, int layer, float scale, int n_splits, float* scratch, cudaStream_t st) {
    if (n_tok == 0) return cudaSuccess;
    if (n_splits < 2 || !scratch) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(attention_split_kernel, dim3(n_heads, n_tok, n_splits), dim3(ATT_WARPS * 32), 0, st, q, ldq,
                                (float*)nullptr, 0, n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_attention(const float* q, int ldq, float* out, int ldo, int n_tok, int n_heads, const int32_t* tok_slot,
                             const int32_t* tok_pos, KvGeom kv, int layer, float scale, int n_splits, float* scratch,
                             cudaStream_t st) {
    if (n_tok == 0) return cudaSuccess;
    if (n_splits < 1 || (n_splits > 1 && !scratch)) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(attention_split_kernel, dim3(n_heads, n_tok, n_splits), dim3(ATT_WARPS * 32), 0, st, q, ldq, out, ldo,
                                n_heads, tok_slot, tok_pos, kv, layer, scale, n_splits, scratch);
    if (le != cudaSuccess) return le;
    cudaError_t e = count_launch_and_check();
    if (e != cudaSuccess || n_splits == 1) return e;
    attention_merge_kernel<<<dim3(n_heads, n_tok), 128, 0, st>>>(scratch, n_heads, n_splits, kv.head_dim, out, ldo);
    return count_launch_and_check();
}

}  // namespace sp
