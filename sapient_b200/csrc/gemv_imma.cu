// Tensor-core dequant-GEMV / small-M GEMM on tile-repacked ggml blocks (layouts: gemv_imma.cuh).
//
// The products run on the integer tensor path (mma.sync m16n8k32 / m16n8k16, s8 x s8 -> s32):
// 4-bit / 6-bit / 8-bit weights are masked straight into s8 fragments (no float conversion per
// weight), activations arrive as 2-3 int8 digits per element, and the block scales are applied
// to the s32 sums:
//   Q4_K  per 256: y += cs * ( d * sum_s sc_s * C_s  -  dmin * sum_s m_s * X_s )      (s: 8 sub-blocks)
//   Q6_K  per 256: y += cs * d * sum_g sc_g * (C_g - 32 X_g)                            (g: 16 groups)
//   Q8_0  per  32: y += cs * d_b * C_b
// C = integer dot of weights and digits, X = digit sums, cs = the digit column's power-of-two scale.
// This is the arithmetic of the reference's matmul_nt (crates/sapient-backends/cpu/src/kernels/
// matmul.rs:575-689,862-943,1111-1167) with the activations held to 2^-23 (3 digits) or 2^-15
// (2 digits) of each block's maximum instead of f32.
#include "gemv_imma.cuh"
#include "gemv_imma_dev.cuh"

#include <atomic>

#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"
#include "tp.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

// 0: the one-CTA-per-tile-row kernel (default); 3: the persistent streaming kernel for launches that qualify (plan_stream).
static std::atomic<int> g_imma_kernel{0};

// ───────────────────────────── weight repack ────────────────────────────────
__device__ __forceinline__ uint32_t ld_word_2B(const uint8_t* p) {
    return (uint32_t)*reinterpret_cast<const uint16_t*>(p) | ((uint32_t)*reinterpret_cast<const uint16_t*>(p + 2) << 16);
}

__global__ void repack_q4_k_kernel(const uint8_t* __restrict__ raw, int64_t n, int64_t k_tiles, int64_t total_words,
                                   uint32_t* __restrict__ out) {
    const int64_t rb = k_tiles * Q4_K_BYTES;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tile = i / 576;
        const int w = (int)(i - tile * 576);
        const int64_t rt = tile / k_tiles, kt = tile - rt * k_tiles;
        int row, off;
        if (w < 512) {
            const int j = w >> 7, lane = (w >> 2) & 31, wi = w & 3;
            const int g = lane >> 2, t = lane & 3;
            row = g + ((wi & 2) ? 8 : 0);
            off = 16 + 32 * j + 16 * (wi & 1) + 4 * t;
        } else {
            row = (w - 512) >> 2;
            off = 4 * ((w - 512) & 3);
        }
        const int64_t r = rt * 16 + row;
        out[i] = r < n ? *reinterpret_cast<const uint32_t*>(raw + r * rb + kt * Q4_K_BYTES + off) : 0u;
    }
}

__global__ void repack_q6_k_kernel(const uint8_t* __restrict__ raw, int64_t n, int64_t k_tiles, int64_t total_words,
                                   uint32_t* __restrict__ out) {
    const int64_t rb = k_tiles * Q6_K_BYTES;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tile = i / 840;
        const int w = (int)(i - tile * 840);
        const int64_t rt = tile / k_tiles, kt = tile - rt * k_tiles;
        const uint8_t* blk0 = raw + kt * Q6_K_BYTES;
        uint32_t v = 0;
        if (w < 768) {
            const int ii = w >> 7, lane = (w >> 2) & 31, wi = w & 3;
            const int g = lane >> 2, t = lane & 3;
            const int s = 4 * ii + wi, c = s / 6, f = s - 6 * c;
            const int half = c >> 1, p = c & 1, kind = f % 3;
            const int64_t r = rt * 16 + g + (f >= 3 ? 8 : 0);
            const int off = kind == 0 ? 64 * half + 16 * p + 4 * t
                          : kind == 1 ? 64 * half + 32 + 16 * p + 4 * t
                                      : 128 + 32 * half + 16 * p + 4 * t;
            if (r < n) v = ld_word_2B(blk0 + r * rb + off);
        } else if (w < 832) {
            const int64_t r = rt * 16 + ((w - 768) >> 2);
            if (r < n) v = ld_word_2B(blk0 + r * rb + 192 + 4 * ((w - 768) & 3));
        } else {
            const int64_t r0 = rt * 16 + 2 * (w - 832);
            const uint32_t lo = r0 < n ? *reinterpret_cast<const uint16_t*>(blk0 + r0 * rb + 208) : 0u;
            const uint32_t hi = r0 + 1 < n ? *reinterpret_cast<const uint16_t*>(blk0 + (r0 + 1) * rb + 208) : 0u;
            v = lo | (hi << 16);
        }
        out[i] = v;
    }
}

// Q8_0: tile = bpt blocks; words per tile = bpt * 128 (values) + bpt * 8 (16 rows x bpt halfs).
__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ raw, int64_t n, int64_t k_tiles, int bpt, int64_t total_words,
                                   uint32_t* __restrict__ out) {
    const int64_t rb = k_tiles * bpt * Q8_0_BYTES;
    const int wpt = bpt * 136;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_words; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tile = i / wpt;
        const int w = (int)(i - tile * wpt);
        const int64_t rt = tile / k_tiles, kt = tile - rt * k_tiles;
        uint32_t v = 0;
        if (w < bpt * 128) {
            const int b = w >> 7, lane = (w >> 2) & 31, wi = w & 3;
            const int g = lane >> 2, t = lane & 3;
            const int64_t r = rt * 16 + g + ((wi & 2) ? 8 : 0);
            if (r < n) v = ld_word_2B(raw + r * rb + (kt * bpt + b) * Q8_0_BYTES + 2 + 16 * (wi & 1) + 4 * t);
        } else {
            // half index h = row * bpt + b; this word holds halfs 2*hw and 2*hw+1
            const int hw = w - bpt * 128;
            uint32_t parts[2];
            for (int q = 0; q < 2; ++q) {
                const int h = 2 * hw + q, row = h / bpt, b = h - row * bpt;
                const int64_t r = rt * 16 + row;
                parts[q] = r < n ? *reinterpret_cast<const uint16_t*>(raw + r * rb + (kt * bpt + b) * Q8_0_BYTES) : 0u;
            }
            v = parts[0] | (parts[1] << 16);
        }
        out[i] = v;
    }
}

int imma_q8_bpt(int64_t k) { return (k % 256 == 0) ? 8 : (k % 128 == 0) ? 4 : 1; }

size_t imma_tiled_bytes(int dtype, int64_t n, int64_t k) {
    const int64_t rt = (n + 15) / 16;
    if (dtype == T_Q4_K) return (size_t)(rt * (k / 256) * Q4_K_TILE_BYTES);
    if (dtype == T_Q6_K) return (size_t)(rt * (k / 256) * Q6_K_TILE_BYTES);
    if (dtype == T_Q8_0) return (size_t)(rt * (k / 32) * 544);
    return 0;
}

bool imma_supported(int dtype, int64_t k) {
    if (dtype == T_Q4_K || dtype == T_Q6_K) return k % 256 == 0;
    if (dtype == T_Q8_0) return k % 32 == 0;
    return false;
}

cudaError_t launch_repack(int dtype, const uint8_t* raw, int64_t n, int64_t k, uint8_t* tiled, cudaStream_t st) {
    const int64_t rt = (n + 15) / 16;
    const int64_t words = (int64_t)(imma_tiled_bytes(dtype, n, k) / 4);
    if (words == 0) return cudaSuccess;
    const int blocks = (int)((words + 255) / 256 < 148 * 32 ? (words + 255) / 256 : 148 * 32);
    (void)rt;
    if (dtype == T_Q4_K) repack_q4_k_kernel<<<blocks, 256, 0, st>>>(raw, n, k / 256, words, (uint32_t*)tiled);
    else if (dtype == T_Q6_K) repack_q6_k_kernel<<<blocks, 256, 0, st>>>(raw, n, k / 256, words, (uint32_t*)tiled);
    else if (dtype == T_Q8_0) {
        const int bpt = imma_q8_bpt(k);
        repack_q8_0_kernel<<<blocks, 256, 0, st>>>(raw, n, (k / 32) / bpt, bpt, words, (uint32_t*)tiled);
    } else return cudaErrorInvalidValue;
    return count_launch_and_check();
}

// ─────────────────────────── activation digits ───────────────────────────────
// Where the digits of one GEMV input go (see gemv_imma.cuh for the layouts).
struct QuantOut {
    int k, kp, digits, eb, ncp;
    int8_t* xq;
    float* colscale;
    int8_t* xs32d;
    int8_t* xs16d;
};
__host__ inline QuantOut quant_out(const ImmaArgs& a) {
    QuantOut q;
    q.k = a.k; q.kp = a.kp; q.digits = a.digits; q.eb = a.eb; q.ncp = a.ncp;
    q.xq = const_cast<int8_t*>(a.xq); q.colscale = const_cast<float*>(a.colscale);
    q.xs32d = const_cast<int8_t*>(a.xs32d); q.xs16d = const_cast<int8_t*>(a.xs16d);
    return q;
}

// One warp converts 256 columns (tile) of activation row m: lane holds the 8 consecutive columns
// tile * 256 + lane * 8 .. +7 in v (zeros when !live). All 32 lanes must call.
__device__ __forceinline__ void quantize_chunk(const float (&v)[8], bool live, int lane, int tile, int m, const QuantOut& qo) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // exponent block: the 4 lanes of a 32-column block, or the whole warp
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    if (qo.eb == 256) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 8));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 16));
    }
    const int digits = qo.digits, P = 8 * digits - 2;
    float up = 0.f, down = 0.f;  // x * up -> fixed point; digit 0 scale = down
    if (amax > 0.f && amax < INFINITY) {
        int e = ilogbf(amax) + 1;          // amax < 2^e
        e = max(e, -100);                  // keep 2^(P-e) finite
        up = scalbnf(1.0f, P - e);         // exact powers of two
        down = scalbnf(1.0f, e - P);
    }
    // balanced base-256 digits, least significant first
    uint32_t w0[3] = {0u, 0u, 0u}, w1[3] = {0u, 0u, 0u};
    int sum[3] = {0, 0, 0};
    const int lim = 1 << P;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int X = max(-lim, min(lim, __float2int_rn(v[i] * up)));
        const int q0 = ((X + 128) & 255) - 128;
        X = (X - q0) >> 8;
        int q1, q2;
        if (digits == 3) { q1 = ((X + 128) & 255) - 128; q2 = (X - q1) >> 8; }
        else { q1 = X; q2 = 0; }
        sum[0] += q0; sum[1] += q1; sum[2] += q2;
        const int sh = 8 * (i & 3);
        if (i < 4) { w0[0] |= (uint32_t)(q0 & 255) << sh; w0[1] |= (uint32_t)(q1 & 255) << sh; w0[2] |= (uint32_t)(q2 & 255) << sh; }
        else { w1[0] |= (uint32_t)(q0 & 255) << sh; w1[1] |= (uint32_t)(q1 & 255) << sh; w1[2] |= (uint32_t)(q2 & 255) << sh; }
    }
    const int a4 = lane & 3, blk = lane >> 2;       // 32-block of the tile
    const int h = a4 >> 1, t0 = 2 * (a4 & 1);       // lane's columns are 16h + 4t0 .. and 16h + 4(t0+1) .. of the block
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        const int s16 = sum[d] + __shfl_xor_sync(0xFFFFFFFFu, sum[d], 1);
        const int s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
        if (d < digits && live) {
            const int col = m * digits + d;
            int8_t* dst = qo.xq + (int64_t)col * qo.kp + (int64_t)tile * 256 + blk * 8 + 4 * h;
            *reinterpret_cast<uint32_t*>(dst + t0 * 64) = w0[d];
            *reinterpret_cast<uint32_t*>(dst + (t0 + 1) * 64) = w1[d];
            int8_t* r32 = qo.xs32d + ((int64_t)tile * qo.ncp + col) * 32;
            int8_t* r16 = qo.xs16d + ((int64_t)tile * qo.ncp + col) * 32;
            if ((lane & 1) == 0) {
                const int a = ((s16 + 32) & 63) - 32;
                r16[lane >> 1] = (int8_t)a;
                r16[16 + (lane >> 1)] = (int8_t)((s16 - a) >> 6);
            }
            if (a4 == 0) {
                const int a = ((s32 + 32) & 63) - 32;
                r32[blk] = (int8_t)a;
                r32[16 + blk] = (int8_t)((s32 - a) >> 6);
            }
        }
    }
    const bool writer = (qo.eb == 256) ? (lane == 0) : (a4 == 0);
    if (writer && live) {
        const int k0 = tile * 256 + lane * 8;
        float s = down;
        for (int d = 0; d < digits; ++d) {
            qo.colscale[(int64_t)(k0 / qo.eb) * qo.ncp + m * digits + d] = s;
            s *= 256.f;
        }
    }
}

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// Plain conversion: one warp per (256 columns, activation row).
__global__ void __launch_bounds__(32) act_quant_kernel(const float* __restrict__ x, int ldx, QuantOut qo) {
    const int lane = threadIdx.x, m = blockIdx.y, tile = blockIdx.x;
    const int k0 = tile * 256 + lane * 8;
    const bool live = k0 < qo.k;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) load8(x + (int64_t)m * ldx + k0, v);
    quantize_chunk(v, live, lane, tile, m, qo);
}

// RMSNorm / LayerNorm of one activation row per block, emitting the digits of the normalised row (and, when
// y != null, its f32 values). Arithmetic of the norm as in crates/sapient-backends/cpu/src/kernels/layernorm.rs:17-105.
constexpr int NORM_WARPS = 16;
template <bool LAYER_NORM>
__global__ void __launch_bounds__(NORM_WARPS * 32) norm_quant_kernel(float* x, int ldx, const float* __restrict__ w,
                                                                     const float* __restrict__ b, float eps, float* __restrict__ y, int ldy,
                                                                     QuantOut qo, const TpDev* tp) {
    __shared__ float sh[NORM_WARPS];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tensor parallel: the row still lacks the sum of the ranks' partial products (o_proj / down_proj); add it first
    uint32_t tp_epoch = 0;
    if (tp) tp_epoch = tp_consume_row(*tp, x, (int64_t)m * ldx, m, qo.k);
    const float* row = x + (int64_t)m * ldx;
    const int k = qo.k, tiles = (k + 255) / 256;
    auto block_sum = [&](float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        __syncthreads();
        if (lane == 0) sh[warp] = v;
        __syncthreads();
        float t = lane < NORM_WARPS ? sh[lane] : 0.f;
#pragma unroll
        for (int o = NORM_WARPS / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        return __shfl_sync(0xFFFFFFFFu, t, 0);
    };
    // Each warp owns the 256-column tiles warp, warp + 16, ...; a lane's 8 columns of the warp's first tile stay in
    // registers across the passes (rows of up to 4096 columns are read once).
    const int kf = warp * 256 + lane * 8;
    const bool have_first = kf < k;
    float xf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (have_first) load8(row + kf, xf);
    float mean = 0.f;
    if (LAYER_NORM) {
        float s = 0.f;
        if (have_first) s = ((xf[0] + xf[1]) + (xf[2] + xf[3])) + ((xf[4] + xf[5]) + (xf[6] + xf[7]));
        for (int tile = warp + NORM_WARPS; tile < tiles; tile += NORM_WARPS) {
            const int k0 = tile * 256 + lane * 8;
            if (k0 < k) {
                float xv[8];
                load8(row + k0, xv);
                s += ((xv[0] + xv[1]) + (xv[2] + xv[3])) + ((xv[4] + xv[5]) + (xv[6] + xv[7]));
            }
        }
        mean = block_sum(s) / (float)k;
    }
    float ss = 0.f;
    if (have_first) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float c = xf[i] - mean; ss = fmaf(c, c, ss); }
    }
    for (int tile = warp + NORM_WARPS; tile < tiles; tile += NORM_WARPS) {
        const int k0 = tile * 256 + lane * 8;
        if (k0 < k) {
            float xv[8];
            load8(row + k0, xv);
#pragma unroll
            for (int i = 0; i < 8; ++i) { const float c = xv[i] - mean; ss = fmaf(c, c, ss); }
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss) / (float)k + eps);
    for (int tile = warp; tile < tiles; tile += NORM_WARPS) {
        const int k0 = tile * 256 + lane * 8;
        const bool live = k0 < k;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (live) {
            float xv[8], wv[8];
            if (tile == warp) {
#pragma unroll
                for (int i = 0; i < 8; ++i) xv[i] = xf[i];
            } else {
                load8(row + k0, xv);
            }
            load8(w + k0, wv);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(xv[i] - mean, inv), wv[i]);
            if (LAYER_NORM && b) {
                float bv[8];
                load8(b + k0, bv);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(v[i], bv[i]);
            }
            if (y) store8(y + (int64_t)m * ldy + k0, v);
        }
        quantize_chunk(v, live, lane, tile, m, qo);
    }
    if (tp) tp_consume_done(*tp, tp_epoch, gridDim.x);
}

// SwiGLU (act == 0: silu(gate) * up from gu[m][0..ffn) and gu[m][ffn..2ffn)) or tanh-GELU (act == 1: of gu[m][0..ffn))
// emitting the digits of the result; one warp per (256 columns, row). Formulas: kernels/elementwise.rs:120-143.
__global__ void __launch_bounds__(32) act_fn_quant_kernel(const float* __restrict__ gu, int ld, int ffn, int act, QuantOut qo) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x, m = blockIdx.y, tile = blockIdx.x;
    const int k0 = tile * 256 + lane * 8;
    const bool live = k0 < ffn;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
        float g[8];
        load8(gu + (int64_t)m * ld + k0, g);
        if (act == 0) {
            float u[8];
            load8(gu + (int64_t)m * ld + ffn + k0, u);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(g[i] / (1.0f + expf(-g[i])), u[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float t = g[i];
                const float inner = __fmul_rn(0.79788456f, __fadd_rn(t, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, t), t), t)));
                v[i] = __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, tanhf(inner)));
            }
        }
    }
    quantize_chunk(v, live, lane, tile, m, qo);
}

// Merge of the split-K attention partials (see attention.cu) emitting the digits of the attention output row;
// one block per (256 columns of the [n_heads * hd] row, token), one thread per column, warp 0 converts the
// merged 256 values to digits. part: [tok][head][split][hd + 2]. Splits without keys carry m = -inf, l = 0, o = 0.
constexpr int MERGE_MAX_SPLITS = 32;
__global__ void __launch_bounds__(256) attn_merge_quant_kernel(const float* __restrict__ part, int n_heads, int n_splits, int hd,
                                                               float* __restrict__ out, int ldo, QuantOut qo) {
    __shared__ __align__(16) float sv[256];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.y, tile = blockIdx.x;
    const int col = tile * 256 + threadIdx.x;
    float v = 0.f;
    if (col < qo.k) {
        const int h = col / hd, e = col - h * hd;
        const float* src = part + ((int64_t)m * n_heads + h) * n_splits * (hd + 2);
        float ms[MERGE_MAX_SPLITS];
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < MERGE_MAX_SPLITS; ++s) {
            ms[s] = s < n_splits ? src[(int64_t)s * (hd + 2)] : -INFINITY;
            M = fmaxf(M, ms[s]);
        }
        float L = 0.f;
#pragma unroll
        for (int s = 0; s < MERGE_MAX_SPLITS; ++s) {
            if (s < n_splits) {
                const float c = (ms[s] == -INFINITY) ? 0.f : expf(ms[s] - M);
                L = fmaf(c, src[(int64_t)s * (hd + 2) + 1], L);
                v = fmaf(c, src[(int64_t)s * (hd + 2) + 2 + e], v);
            }
        }
        v *= (L == 0.f) ? 0.f : 1.0f / L;
        if (out) out[(int64_t)m * ldo + col] = v;
    }
    sv[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float w[8];
        load8(sv + lane * 8, w);
        quantize_chunk(w, tile * 256 + lane * 8 < qo.k, lane, tile, m, qo);
    }
}

// 1 (default): 3 digits for every pass (10 rows per pass): activations held to 2^-23 of each block's maximum at any row
//    count — the setting under which full-size models stay within the final-logit bar of the reference's f32 path.
// 0: 3 digits while they fit one 8-column n-tile (m <= 2), else 2 digits (2^-15) and 16 rows per pass: fewer passes for
//    batched steps, at ~1e-4 relative error per product.
static std::atomic<int> g_digit_mode{1};
void imma_set_digit_mode(int mode) { g_digit_mode.store(mode ? 1 : 0); }
int imma_rows_per_pass() { return g_digit_mode.load() ? 10 : 16; }

void imma_plan(ImmaArgs& a, const ActWorkspace& ws) {
    a.digits = (a.m <= 2 || (g_digit_mode.load() && a.m <= 10)) ? 3 : 2;
    const int cols = a.m * a.digits;
    a.ncp = cols <= 8 ? 8 : cols <= 16 ? 16 : 32;
    a.eb = (a.k % 256 == 0) ? 256 : 32;
    a.kp = (a.k + 255) / 256 * 256;
    a.xq = ws.xq; a.colscale = ws.colscale; a.xs32d = ws.xs32d; a.xs16d = ws.xs16d;
}

void imma_plan_rows(ImmaArgs& a, const ActWorkspace& ws) {
    a.digits = 3;
    a.ncp = (a.m * 3 + 31) / 32 * 32;
    a.eb = (a.k % 256 == 0) ? 256 : 32;
    a.kp = (a.k + 255) / 256 * 256;
    a.xq = ws.xq; a.colscale = ws.colscale; a.xs32d = ws.xs32d; a.xs16d = ws.xs16d;
}

cudaError_t launch_act_quant(const float* x, int ldx, const ImmaArgs& a, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    act_quant_kernel<<<dim3(a.kp / 256, a.m), 32, 0, st>>>(x, ldx, quant_out(a));
    return count_launch_and_check();
}

cudaError_t launch_norm_quant(const float* x, int ldx, const float* w, const float* b, bool layer_norm, float eps, float* y, int ldy,
                              const ImmaArgs& a, cudaStream_t st, const TpDev* tp) {
    if (a.m <= 0) return cudaSuccess;
    float* xm = const_cast<float*>(x);  // written only when tp != null (the pending sum is added in place)
    cudaError_t le = layer_norm ? launch_pdl(norm_quant_kernel<true>, dim3(a.m), dim3(NORM_WARPS * 32), 0, st, xm, ldx, w, b, eps, y,
                                             ldy, quant_out(a), tp)
                                : launch_pdl(norm_quant_kernel<false>, dim3(a.m), dim3(NORM_WARPS * 32), 0, st, xm, ldx, w,
                                             (const float*)nullptr, eps, y, ldy, quant_out(a), tp);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_act_fn_quant(const float* gu, int ld, int ffn, int act, const ImmaArgs& a, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    cudaError_t le = launch_pdl(act_fn_quant_kernel, dim3(a.kp / 256, a.m), dim3(32), 0, st, gu, ld, ffn, act, quant_out(a));
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_attn_merge_quant(const float* part, int n_heads, int n_splits, int hd, float* out, int ldo, const ImmaArgs& a,
                                    cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    if (n_splits > MERGE_MAX_SPLITS) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(attn_merge_quant_kernel, dim3(a.kp / 256, a.m), dim3(256), 0, st, part, n_heads, n_splits, hd, out, ldo,
                                quant_out(a));
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t ActWorkspace::alloc(int k_max_) {
    release();
    k_max = (k_max_ + 255) / 256 * 256;
    const size_t tiles = (size_t)k_max / 256;
    cudaError_t e;
    if ((e = cudaMalloc((void**)&xq, (size_t)NCP_MAX * k_max)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&colscale, (size_t)(k_max / 32) * NCP_MAX * 4)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&xs32d, tiles * NCP_MAX * 32)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&xs16d, tiles * NCP_MAX * 32)) != cudaSuccess) return e;
    // unused digit columns are read (and meet zero digits): keep them finite; bytes 8..15 / 24..31 of the
    // xs32d records are never written and must stay zero
    cudaMemset(xq, 0, (size_t)NCP_MAX * k_max);
    cudaMemset(colscale, 0, (size_t)(k_max / 32) * NCP_MAX * 4);
    cudaMemset(xs32d, 0, tiles * NCP_MAX * 32);
    cudaMemset(xs16d, 0, tiles * NCP_MAX * 32);
    return cudaDeviceSynchronize();
}

cudaError_t ActWorkspace::ensure_xh(size_t elems) {
    if (elems <= xh_elems) return cudaSuccess;
    if (xh) cudaFree(xh);
    xh = nullptr;
    xscale = nullptr;
    xh_elems = 0;
    const size_t bytes = (elems * sizeof(__half) + 255) / 256 * 256;
    cudaError_t e = cudaMalloc((void**)&xh, bytes + XSCALE_ROWS * sizeof(float));
    if (e == cudaSuccess) { xh_elems = elems; xscale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xh) + bytes); }
    if (e == cudaSuccess && !tc5.buf) e = tc5.alloc();
    return e;
}

void ActWorkspace::release() {
    if (xh) cudaFree(xh);
    xh = nullptr; xh_elems = 0; xscale = nullptr;
    tc5.release();
    if (xq) cudaFree(xq);
    if (colscale) cudaFree(colscale);
    if (xs32d) cudaFree(xs32d);
    if (xs16d) cudaFree(xs16d);
    xq = nullptr; colscale = nullptr; xs32d = nullptr; xs16d = nullptr; k_max = 0;
}

// ─────────────────────────────── the GEMV ────────────────────────────────────
// (mma wrappers, tile register images and per-tile arithmetic: gemv_imma_dev.cuh)
// ── Q8_0 with any number of blocks per tile (K not a multiple of 256) ──
template <int NT>
__device__ __forceinline__ void tile_q8_0(const ImmaArgs& a, const uint8_t* tile, int kt, int bpt, int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    const uint16_t* dh = reinterpret_cast<const uint16_t*>(tile + bpt * 512);
    for (int bb = 0; bb < bpt; ++bb) {
        const uint4 q = ldg_u4(tile + bb * 512 + lane * 16);
        const float d0 = half_bits_to_float(__ldg(dh + g * bpt + bb)), d1 = half_bits_to_float(__ldg(dh + (g + 8) * bpt + bb));
        const int blk32 = kt * bpt + bb;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = nt * 8 + g;
            uint2 b = make_uint2(0u, 0u);
            if (col < a.m * a.digits)
                b = __ldg(reinterpret_cast<const uint2*>(a.xq + (int64_t)col * a.kp + (int64_t)(blk32 >> 3) * 256 + t * 64 + (blk32 & 7) * 8));
            int c[4];
            imma_k32(c, q.x, q.z, q.y, q.w, b.x, b.y, 0, 0, 0, 0);
            const float2 cs = __ldg(reinterpret_cast<const float2*>(a.colscale + (int64_t)(blk32 * 32 / a.eb) * a.ncp + nt * 8 + 2 * t));
            acc[nt][0] = fmaf(cs.x * d0, (float)c[0], acc[nt][0]);
            acc[nt][1] = fmaf(cs.y * d0, (float)c[1], acc[nt][1]);
            acc[nt][2] = fmaf(cs.x * d1, (float)c[2], acc[nt][2]);
            acc[nt][3] = fmaf(cs.y * d1, (float)c[3], acc[nt][3]);
        }
    }
}

// Writes y for the 16 rows of tile row rt from the per-warp partial sums in red[warp][nt][e][lane].
template <int NT, int WARPS>
__device__ __forceinline__ void reduce_store(const ImmaArgs& a, const ImmaSeg& sg, bool first_seg, int rt, const float* red) {
    for (int idx = threadIdx.x; idx < 16 * a.m; idx += blockDim.x) {
        const int r = idx & 15, m = idx >> 4;
        const int64_t row = (int64_t)rt * 16 + r;
        if (row >= sg.n) continue;
        float v = 0.f;
        for (int d = 0; d < a.digits; ++d) {
            const int col = m * a.digits + d, nt = col >> 3, cc = col & 7;
            const int e = (r < 8 ? 0 : 2) + (cc & 1), ln = (r & 7) * 4 + (cc >> 1);
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += red[((w * NT + nt) * 4 + e) * 32 + ln];
        }
        if (sg.bias) v += sg.bias[row];
        if (a.tp) {
            // partial sum of a column-split matrix: straight into every rank's receive area (peer stores)
            const TpDev& tp = *a.tp;
            const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tp.ar_seq) + 1u;
            const int64_t off = (int64_t)(a.tp_row0 + m) * sg.ldy + row;
            const unsigned long long word = tp_word(v, epoch);  // value and arrival mark in one 64-bit store
            for (int p = 0; p < tp.size; ++p) tp_recv(tp, p, (int)(epoch & 1u), tp.rank)[off] = word;
            continue;
        }
        if (first_seg && a.res) v += a.res[(int64_t)m * a.ldres + row];
        sg.y[(int64_t)m * sg.ldy + row] = v;
    }
}

// Kernel A (any shape): one CTA per tile row; its 8 warps split the k-tiles, operands straight from global memory.
// FMT: 0 = segments of any format; T_Q4_K / T_Q6_K = every segment of the launch has that format — the code for the
// other formats is left out, which lets the M <= 2 instance fit 80 registers and run three CTAs (24 warps) per SM
// instead of two.
template <int NT, int FMT>
__global__ void __launch_bounds__(IMMA_WARPS * 32, (NT == 1 && FMT != 0) ? 3 : 2) gemv_imma_kernel(const ImmaArgs a) {
    __shared__ float red[IMMA_WARPS * NT * 4 * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    int rt = blockIdx.x, s = 0;
    while (s < a.nseg - 1 && rt >= (a.seg[s].n + 15) / 16) { rt -= (a.seg[s].n + 15) / 16; ++s; }
    const ImmaSeg& sg = a.seg[s];
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    if (FMT == T_Q4_K || (FMT == 0 && sg.dtype == T_Q4_K)) {
        const int kts = a.k >> 8;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * Q4_K_TILE_BYTES;
        Q4Regs ra, rb;
        BFrag<NT> b;
        int kt = warp;
        if (kt < kts) load_q4_k<true>(base + (int64_t)kt * Q4_K_TILE_BYTES, lane, ra);
        if (kt + IMMA_WARPS < kts) load_q4_k<true>(base + (int64_t)(kt + IMMA_WARPS) * Q4_K_TILE_BYTES, lane, rb);
        pdl_wait();  // the weight tiles above are in flight while the producer of the activations finishes
        pdl_trigger();
        bool first = true;
        while (kt < kts) {
            const int k1 = kt + IMMA_WARPS, k2 = kt + 2 * IMMA_WARPS;
            if (!first && k1 < kts) load_q4_k<true>(base + (int64_t)k1 * Q4_K_TILE_BYTES, lane, rb);
            first = false;
            load_b_global<NT>(a, kt, g, t, true, false, b);
            compute_q4_k<NT>(ra, b, lane, acc);
            if (k1 >= kts) break;
            if (k2 < kts) load_q4_k<true>(base + (int64_t)k2 * Q4_K_TILE_BYTES, lane, ra);
            load_b_global<NT>(a, k1, g, t, true, false, b);
            compute_q4_k<NT>(rb, b, lane, acc);
            kt = k2;
        }
    } else if (FMT == T_Q6_K || (FMT == 0 && sg.dtype == T_Q6_K)) {
        const int kts = a.k >> 8;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * Q6_K_TILE_BYTES;
        Q6Regs ra;
        BFrag<NT> b;
        if (warp < kts) load_q6_k<true>(base + (int64_t)warp * Q6_K_TILE_BYTES, lane, ra);
        pdl_wait();
        pdl_trigger();
        for (int kt = warp; kt < kts; kt += IMMA_WARPS) {
            if (kt != warp) load_q6_k<true>(base + (int64_t)kt * Q6_K_TILE_BYTES, lane, ra);
            load_b_global<NT>(a, kt, g, t, false, true, b);
            compute_q6_k<NT>(ra, b, lane, acc);
        }
    } else if (FMT == 0) {
        const int bpt = sg.bpt, kts = (a.k >> 5) / bpt, tb = bpt * 544;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * tb;
        pdl_wait();
        pdl_trigger();
        for (int kt = warp; kt < kts; kt += IMMA_WARPS) tile_q8_0<NT>(a, base + (int64_t)kt * tb, kt, bpt, lane, acc);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((warp * NT + nt) * 4 + e) * 32 + lane] = acc[nt][e];
    __syncthreads();
    reduce_store<NT, IMMA_WARPS>(a, sg, s == 0, rt, red);
}

// ── Kernel B (k % 256 == 0, digits fit shared memory): persistent streaming kernel ──
// One CTA per SM with 16 warps. Warp w owns k-tiles w, w+16, ... of every tile row the CTA visits
// (rows blockIdx.x, +gridDim.x, ...), so consecutive tiles of a warp are weight data only: each is one
// contiguous 2.3-4.3 KB tile fetched by a single TMA bulk copy (cp.async.bulk, mbarrier completion) into a
// per-warp ring of STREAM_STAGES slots, while the activation digits, digit-sum records and column scales of
// the whole row sit in shared memory, loaded once per CTA. The weight prefetch is issued before the
// grid-dependency wait, so under programmatic dependent launch it overlaps the kernel that produces the
// activations.
constexpr int STREAM_WARPS = 16;
constexpr int STREAM_MAX_STAGES = 4;
constexpr int STREAM_SMEM_LIMIT = 220 * 1024;
constexpr int STREAM_SPIN_LIMIT = 1 << 16;  // polls of up to ~20 us each (the try_wait time hint) before a wait gives up: about a second

// Set when a bounded wait in a kernel of this file ran out; host code reads and clears it.
__device__ int g_imma_timeout = 0;

struct StreamPlan {
    int stage_bytes;   // ring slot size: largest tile among the segments, multiple of 128
    int stages;        // ring depth per warp (2..4, as many as fit)
    int bar_off, xq_off, rec32_off, rec16_off, cs_off, red_off, total;  // byte offsets in dynamic shared memory
    int total_tiles;   // tile rows over all segments
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, int bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Bounded wait for phase `parity` of the barrier; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (int spin = 0; spin < STREAM_SPIN_LIMIT; ++spin) {
        uint32_t ok;
        // the hint lets the hardware park the warp (up to ~20 us) instead of spinning through issue slots
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok)
                     : "r"(addr), "r"(parity), "r"(20000)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

template <int NT>
__global__ void __launch_bounds__(STREAM_WARPS * 32, 1) gemv_imma_stream_kernel(const ImmaArgs a, const StreamPlan p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kts = a.k >> 8;
    const int nk = kts > warp ? (kts - warp + STREAM_WARPS - 1) / STREAM_WARPS : 0;     // my k-tiles per tile row
    const int n_rows = p.total_tiles > (int)blockIdx.x ? (p.total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    uint8_t* ring = smem + (size_t)warp * p.stages * p.stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.bar_off) + warp * STREAM_MAX_STAGES;
    auto tile_bytes = [&](int dtype) { return dtype == T_Q4_K ? Q4_K_TILE_BYTES : dtype == T_Q6_K ? Q6_K_TILE_BYTES : 4352; };
    auto seg_tiles = [&](int s) { return (a.seg[s].n + 15) / 16; };

    if (lane == 0)
        for (int s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    __syncwarp();

    // producer cursor: the next tile to fetch = (segment ps, tile row pr of it, k-tile index pj of this warp)
    int ps = 0, pr = blockIdx.x, pj = 0, p_left = n_rows * nk, p_slot = 0;
    while (ps < a.nseg - 1 && pr >= seg_tiles(ps)) { pr -= seg_tiles(ps); ++ps; }
    auto issue = [&]() {
        if (p_left > 0 && lane == 0) {
            const int tb = tile_bytes(a.seg[ps].dtype);
            const uint8_t* src = a.seg[ps].wt + ((int64_t)pr * kts + warp + STREAM_WARPS * pj) * tb;
            mbar_expect_tx(&bars[p_slot], tb);
            bulk_copy_g2s(ring + (size_t)p_slot * p.stage_bytes, src, tb, &bars[p_slot]);
        }
        if (p_left > 0) {
            --p_left;
            p_slot = p_slot + 1 == p.stages ? 0 : p_slot + 1;
            if (++pj == nk) {
                pj = 0;
                pr += gridDim.x;
                while (ps < a.nseg - 1 && pr >= seg_tiles(ps)) { pr -= seg_tiles(ps); ++ps; }
            }
        }
    };
    for (int i = 0; i < p.stages - 1; ++i) issue();

    // everything below depends on the kernel that produced the activations
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    const int ncols = a.m * a.digits;
    {
        int8_t* xs = reinterpret_cast<int8_t*>(smem + p.xq_off);
        const int vec_per_col = a.kp / 16;
        for (int i = threadIdx.x; i < ncols * vec_per_col; i += blockDim.x) {
            const int c = i / vec_per_col, v = i - c * vec_per_col;
            reinterpret_cast<uint4*>(xs)[i] = ldg_u4(a.xq + (int64_t)c * a.kp + (int64_t)v * 16);
        }
        // records [kt][col][32 B] -> shared [kt][ncols][32 B]; scales [kt][ncp] -> shared [kt][ncp]
        uint4* r32 = reinterpret_cast<uint4*>(smem + p.rec32_off);
        uint4* r16 = reinterpret_cast<uint4*>(smem + p.rec16_off);
        for (int i = threadIdx.x; i < kts * ncols * 2; i += blockDim.x) {
            const int kt = i / (ncols * 2), rem = i - kt * ncols * 2;
            const int64_t src = ((int64_t)kt * a.ncp) * 32 + (int64_t)rem * 16;
            r32[i] = ldg_u4(a.xs32d + src);
            r16[i] = ldg_u4(a.xs16d + src);
        }
        float* cs = reinterpret_cast<float*>(smem + p.cs_off);
        for (int i = threadIdx.x; i < kts * a.ncp; i += blockDim.x) cs[i] = __ldg(a.colscale + i);
    }
    __syncthreads();

    const int8_t* xs = reinterpret_cast<const int8_t*>(smem + p.xq_off);
    const uint8_t* r32 = smem + p.rec32_off;
    const uint8_t* r16 = smem + p.rec16_off;
    const float* css = reinterpret_cast<const float*>(smem + p.cs_off);
    float* red = reinterpret_cast<float*>(smem + p.red_off);
    float acc[NT][4];
    int c_slot = 0;
    uint32_t c_parity = 0;
    bool ok = true;
    int s = 0, rt = blockIdx.x;
    while (s < a.nseg - 1 && rt >= seg_tiles(s)) { rt -= seg_tiles(s); ++s; }
    for (int it = 0; it < n_rows; ++it) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
        const int dtype = a.seg[s].dtype;
        for (int j = 0; j < nk; ++j) {
            issue();
            ok = ok && mbar_wait(&bars[c_slot], c_parity);
            const int kt = warp + STREAM_WARPS * j;
            const uint8_t* tile = ring + (size_t)c_slot * p.stage_bytes;
            BFrag<NT> b;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int col = nt * 8 + g;
                if (col < ncols) {
                    const int8_t* base = xs + (size_t)col * a.kp + (size_t)kt * 256 + t * 64;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 v = ld_u4(base + 16 * q);
                        b.w[nt][4 * q] = v.x; b.w[nt][4 * q + 1] = v.y; b.w[nt][4 * q + 2] = v.z; b.w[nt][4 * q + 3] = v.w;
                    }
                    const size_t rec = ((size_t)kt * ncols + col) * 32 + 4 * t;
                    b.ra32[nt] = *reinterpret_cast<const uint32_t*>(r32 + rec);
                    b.rb32[nt] = *reinterpret_cast<const uint32_t*>(r32 + rec + 16);
                    b.ra16[nt] = *reinterpret_cast<const uint32_t*>(r16 + rec);
                    b.rb16[nt] = *reinterpret_cast<const uint32_t*>(r16 + rec + 16);
                } else {
#pragma unroll
                    for (int q = 0; q < 16; ++q) b.w[nt][q] = 0u;
                    b.ra32[nt] = b.rb32[nt] = b.ra16[nt] = b.rb16[nt] = 0u;
                }
                b.cs[nt] = *reinterpret_cast<const float2*>(css + (size_t)kt * a.ncp + nt * 8 + 2 * t);
            }
            if (dtype == T_Q4_K) {
                Q4Regs r;
                load_q4_k<false>(tile, lane, r);
                compute_q4_k<NT>(r, b, lane, acc);
            } else if (dtype == T_Q6_K) {
                Q6Regs r;
                load_q6_k<false>(tile, lane, r);
                compute_q6_k<NT>(r, b, lane, acc);
            } else {
                Q8Regs r;
                load_q8_0<false>(tile, lane, r);
                compute_q8_0<NT>(r, b, acc);
            }
            __syncwarp();  // all lanes are done reading the slot before lane 0 refills it
            if (++c_slot == p.stages) { c_slot = 0; c_parity ^= 1u; }
        }
        float* rbuf = red + (size_t)(it & 1) * STREAM_WARPS * NT * 128;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) rbuf[((warp * NT + nt) * 4 + e) * 32 + lane] = acc[nt][e];
        __syncthreads();
        // 16 rows x m outputs, each the sum of STREAM_WARPS x digits partials: `grp` threads per output
        {
            int mp = 1;
            while (mp < a.m) mp <<= 1;
            const int grp = 32 / mp > 0 ? 32 / mp : 1;
            const int out = threadIdx.x / grp, sub = threadIdx.x - out * grp;
            const int r = out & 15, m = out >> 4;
            float v = 0.f;
            if (m < a.m) {
                for (int q = sub; q < STREAM_WARPS * a.digits; q += grp) {
                    const int w = q / a.digits, col = m * a.digits + (q - w * a.digits), nt = col >> 3, cc = col & 7;
                    v += rbuf[((w * NT + nt) * 4 + (r < 8 ? 0 : 2) + (cc & 1)) * 32 + (r & 7) * 4 + (cc >> 1)];
                }
            }
            for (int o = grp >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            const int64_t row = (int64_t)rt * 16 + r;
            if (sub == 0 && m < a.m && row < a.seg[s].n) {
                const ImmaSeg& sg = a.seg[s];
                if (sg.bias) v += sg.bias[row];
                if (s == 0 && a.res) v += a.res[(int64_t)m * a.ldres + row];
                sg.y[(int64_t)m * sg.ldy + row] = v;
            }
        }
        rt += gridDim.x;
        while (s < a.nseg - 1 && rt >= seg_tiles(s)) { rt -= seg_tiles(s); ++s; }
    }
    if (!ok && lane == 0) atomicExch(&g_imma_timeout, 1);
}

// Reads and clears g_imma_timeout (device the calling thread has current; call after a stream synchronise).
// 1 = a bounded wait of the streaming kernel expired since the last call, 0 = none, -1 = CUDA error.
// The ring GEMV (gemv_ring.cu) reports through a host-mapped flag per device, so that checking it costs no CUDA call.
static std::atomic<int*> g_ring_flag_host[SP_MAX_DEVICES];
static std::atomic<int*> g_ring_flag_dev[SP_MAX_DEVICES];
cudaError_t ring_device_init() {
    const int di = current_device_index();
    if (g_ring_flag_host[di].load()) return cudaSuccess;
    int* h = nullptr;
    cudaError_t e = cudaHostAlloc((void**)&h, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return e;
    *h = 0;
    int* d = nullptr;
    e = cudaHostGetDevicePointer((void**)&d, h, 0);
    if (e != cudaSuccess) { cudaFreeHost(h); return e; }
    int* expected = nullptr;
    if (g_ring_flag_host[di].compare_exchange_strong(expected, h)) g_ring_flag_dev[di].store(d);
    else cudaFreeHost(h);  // another thread was first
    return cudaSuccess;
}
int* imma_timeout_flag() {
    const int di = current_device_index();
    while (g_ring_flag_host[di].load() && !g_ring_flag_dev[di].load()) {}  // the winner of the race publishes the device pointer last
    return g_ring_flag_dev[di].load();
}
void imma_note_ring_launch() {}

static std::atomic<int> g_stream_launched[SP_MAX_DEVICES];  // per device: the streaming kernel has been launched since the flag was last read
int imma_take_timeout() {
    if (int* h = g_ring_flag_host[current_device_index()].load()) {
        volatile int* vh = h;
        if (*vh) { *vh = 0; return 1; }
    }
    if (g_stream_launched[current_device_index()].exchange(0) == 0) return 0;
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_imma_timeout, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_imma_timeout, &zero, sizeof(int));
    }
    return flag ? 1 : 0;
}

static PerDeviceOnce g_stream_attr[3];

// Shared-memory layout of the streaming kernel, or total == 0 when the launch does not qualify.
static StreamPlan plan_stream(const ImmaArgs& a) {
    StreamPlan p{};
    if (a.k % 256 != 0 || a.ncp > 16) return p;
    const int kts = a.k / 256, ncols = a.m * a.digits, nt = a.ncp / 8;
    int stage = 0, tiles = 0;
    for (int s = 0; s < a.nseg; ++s) {
        const int dt = a.seg[s].dtype;
        if (dt != T_Q4_K && dt != T_Q6_K && dt != T_Q8_0) return p;
        stage = stage > (dt == T_Q4_K ? Q4_K_TILE_BYTES : dt == T_Q6_K ? Q6_K_TILE_BYTES : 4352)
                    ? stage : (dt == T_Q4_K ? Q4_K_TILE_BYTES : dt == T_Q6_K ? Q6_K_TILE_BYTES : 4352);
        tiles += (a.seg[s].n + 15) / 16;
    }
    stage = (stage + 127) / 128 * 128;
    p.stage_bytes = stage;
    for (int stages = STREAM_MAX_STAGES; stages >= 2; --stages) {
        int off = STREAM_WARPS * stages * stage;
        p.stages = stages;
        p.bar_off = off; off += STREAM_WARPS * STREAM_MAX_STAGES * 8;
        p.xq_off = off; off += ncols * a.kp;
        p.rec32_off = off; off += kts * ncols * 32;
        p.rec16_off = off; off += kts * ncols * 32;
        p.cs_off = off; off += kts * a.ncp * 4;
        off = (off + 15) / 16 * 16;
        p.red_off = off; off += 2 * STREAM_WARPS * nt * 128 * 4;
        p.total = off;
        if (off <= STREAM_SMEM_LIMIT) break;
        p.total = 0;
    }
    p.total_tiles = tiles;
    return p;
}

cudaError_t launch_gemv_imma(const ImmaArgs& a, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) tiles += (a.seg[s].n + 15) / 16;
    if (tiles == 0) return cudaSuccess;
    const int nt = a.ncp / 8;
    // The persistent TMA-streaming kernel is opt-in: measured on B200 it trails the per-tile-row kernel
    // (132 vs 81 us on a 128256 x 4096 Q4_K matrix), so the default is the latter.
    const StreamPlan p = (g_imma_kernel.load() == 3 && !a.tp) ? plan_stream(a) : StreamPlan{};
    if (p.total > 0) {
        const int sms = device_sm_count();
        const int grid = tiles < sms ? tiles : sms;
        {
            const cudaError_t e = g_stream_attr[nt].run([nt] {
                return nt == 1 ? cudaFuncSetAttribute(gemv_imma_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, STREAM_SMEM_LIMIT)
                               : cudaFuncSetAttribute(gemv_imma_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, STREAM_SMEM_LIMIT);
            });
            if (e != cudaSuccess) return e;
        }
        g_stream_launched[current_device_index()].store(1);
        if (nt == 1) gemv_imma_stream_kernel<1><<<grid, STREAM_WARPS * 32, p.total, st>>>(a, p);
        else gemv_imma_stream_kernel<2><<<grid, STREAM_WARPS * 32, p.total, st>>>(a, p);
        return count_launch_and_check();
    }
    cudaError_t le;
    bool q4_only = true, q6_only = true;
    for (int s = 0; s < a.nseg; ++s) {
        q4_only = q4_only && a.seg[s].dtype == T_Q4_K;
        q6_only = q6_only && a.seg[s].dtype == T_Q6_K;
    }
    // The 80-register single-format instances trade per-CTA speed for occupancy: they win once the grid is several
    // waves deep (gate|up, lm_head) and lose on grids that fit the SMs at once (o_proj, down_proj), where one CTA's
    // latency is the kernel's.
    const bool deep = tiles >= 1024;
    if (nt == 1 && q4_only && deep) le = launch_pdl(gemv_imma_kernel<1, T_Q4_K>, dim3(tiles), dim3(IMMA_WARPS * 32), 0, st, a);
    else if (nt == 1 && q6_only && deep) le = launch_pdl(gemv_imma_kernel<1, T_Q6_K>, dim3(tiles), dim3(IMMA_WARPS * 32), 0, st, a);
    else if (nt == 1) le = launch_pdl(gemv_imma_kernel<1, 0>, dim3(tiles), dim3(IMMA_WARPS * 32), 0, st, a);
    else if (nt == 2) le = launch_pdl(gemv_imma_kernel<2, 0>, dim3(tiles), dim3(IMMA_WARPS * 32), 0, st, a);
    else if (nt == 4) le = launch_pdl(gemv_imma_kernel<4, 0>, dim3(tiles), dim3(IMMA_WARPS * 32), 0, st, a);
    else return cudaErrorInvalidValue;
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

void imma_select_kernel(int which) { g_imma_kernel.store(which); }

cudaError_t launch_quant_gemv(const float* x, int ldx, ImmaArgs& a, const ActWorkspace& ws, bool requantize, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    if (a.m > imma_rows_per_pass() || a.k > ws.k_max) return cudaErrorInvalidValue;
    imma_plan(a, ws);
    if (requantize) {
        cudaError_t e = launch_act_quant(x, ldx, a, st);
        if (e != cudaSuccess) return e;
    }
    return launch_gemv_imma(a, st);
}

}  // namespace sp
