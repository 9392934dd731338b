// sm_100a kernels for quantized-GGUF decoder inference: block dequantisation,
// dequant-fused GEMV / small-M GEMM on raw ggml blocks, embedding gather, norms,
// RoPE + paged-KV append, causal GQA attention over the paged fp16 cache, SwiGLU /
// GELU / residual elementwise ops and the tie-aware argmax.
//
// Arithmetic contract (what each kernel mirrors in the reference's CPU path):
//   dequant      crates/sapient-core/src/tensor.rs:378-389,504-565   bit-exact
//   gemv         crates/sapient-backends/cpu/src/kernels/matmul.rs:575-689,862-943,1111-1167
//                (f32 activations, f32 accumulate; summation order differs → ~1e-6 rel)
//   norms        crates/sapient-backends/cpu/src/kernels/layernorm.rs:17-105
//   rope         crates/sapient-backends/cpu/src/kernels/rope.rs:18-136 (cos/sin from a host table)
//   attention    crates/sapient-backends/cpu/src/kernels/attention.rs:98-284 (online softmax)
//   elementwise  crates/sapient-backends/cpu/src/kernels/elementwise.rs:61-69,120-143
//   argmax       crates/sapient-generate/src/sampler.rs:161-168 (last maximum wins)
#include "kernels.h"
#include "sp_common.cuh"

#include <atomic>
#include <cstdlib>

#include "pdl.cuh"

namespace sp {

static std::atomic<int> g_pdl{-1};
bool pdl_enabled() {
    int v = g_pdl.load();
    if (v < 0) {
        const char* e = std::getenv("SAPIENT_CUDA_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
        g_pdl.store(v);
    }
    return v != 0;
}
void pdl_set_enabled(bool on) { g_pdl.store(on ? 1 : 0); }

static std::atomic<uint64_t> g_launches{0};
uint64_t launch_count() { return g_launches.load(); }
void adjust_launch_count(int64_t delta) { g_launches.fetch_add((uint64_t)delta, std::memory_order_relaxed); }
cudaError_t count_launch_and_check() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}
static inline cudaError_t finish_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

// ─────────────────────────────── dequant ────────────────────────────────────
__global__ void dequant_kernel(int dtype, const uint8_t* __restrict__ w, int64_t n, int64_t k, int64_t rb,
                               float* __restrict__ out) {
    const int64_t total = n * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / k, c = i - r * k;
        out[i] = dequant_elem(dtype, w + r * rb, c);
    }
}

cudaError_t launch_dequant(int dtype, const uint8_t* w, int64_t n, int64_t k, float* out, cudaStream_t st) {
    const int64_t total = n * k;
    if (total == 0) return cudaSuccess;
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    dequant_kernel<<<blocks, 256, 0, st>>>(dtype, w, n, k, row_bytes(dtype, k), out);
    return finish_launch();
}

// ─────────────────────────────── embedding ──────────────────────────────────
__global__ void embed_kernel(int dtype, const uint8_t* __restrict__ table, int64_t hidden, int64_t rb,
                             const uint32_t* __restrict__ ids, float* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const uint8_t* row = table + (int64_t)ids[t] * rb;
    for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) out[(int64_t)t * hidden + c] = dequant_elem(dtype, row, c);
}

cudaError_t launch_embed(int dtype, const uint8_t* table, int64_t hidden, const uint32_t* ids, int n_tok, float* out,
                         cudaStream_t st) {
    if (n_tok == 0) return cudaSuccess;
    cudaError_t le = launch_pdl(embed_kernel, dim3(n_tok), dim3(256), 0, st, dtype, table, hidden, row_bytes(dtype, hidden), ids, out);
    if (le != cudaSuccess) return le;
    return finish_launch();
}

// ─────────────────────────── dequant-fused GEMV ──────────────────────────────
// One warp per weight row; lanes split the row's blocks into 16-byte (Q4_K),
// 4-element-column (Q6_K) or 8-element (Q8_0) units so that neighbouring lanes read
// neighbouring bytes. Each unit is unpacked once into registers and multiplied
// against up to MB activation rows; products use the factored form
//   Q4_K: d·sc·Σ q·x − dmin·m·Σ x     Q6_K: d·sc·Σ (q−32)·x     Q8_0: d·Σ q·x
// with f32 accumulation, then a shuffle reduction.

__device__ __forceinline__ float4 ldg_f4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

template <int MB>
__device__ __forceinline__ void dot_q4_k(const uint8_t* __restrict__ row, const float* __restrict__ x, int ldx, int k,
                                         int mcount, int lane, float (&acc)[MB]) {
    const int nunits = (k >> 8) * 8;
    for (int u = lane; u < nunits; u += 32) {
        const int sb = u >> 3, c = u & 7, g = c >> 1, h = c & 1;
        const uint8_t* blk = row + (int64_t)sb * Q4_K_BYTES;
        const uint4 qv = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 16 * c));
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));  // d, dmin, scales[12]
        const float d = half_bits_to_float((uint16_t)(hdr.x & 0xFFFFu));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        uint32_t sc0, mn0, sc1, mn1;
        k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g, &sc0, &mn0);
        k4_scale_min(hdr.y, hdr.z, hdr.w, 2 * g + 1, &sc1, &mn1);
        const float d0 = d * (float)sc0, m0 = dmin * (float)mn0;
        const float d1 = d * (float)sc1, m1 = dmin * (float)mn1;
        float qlo[16], qhi[16];
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const uint32_t b = (qw[e >> 2] >> (8 * (e & 3))) & 0xFFu;
            qlo[e] = (float)(b & 0xFu);
            qhi[e] = (float)(b >> 4);
        }
        const int xb = sb * 256 + g * 64 + h * 16;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const float* xm = x + (int64_t)(m < mcount ? m : mcount - 1) * ldx + xb;
            float sq0 = 0.f, sx0 = 0.f, sq1 = 0.f, sx1 = 0.f;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const float4 a = ldg_f4(xm + 4 * v);
                const float4 b = ldg_f4(xm + 32 + 4 * v);
                sq0 = fmaf(qlo[4 * v + 0], a.x, sq0); sq0 = fmaf(qlo[4 * v + 1], a.y, sq0);
                sq0 = fmaf(qlo[4 * v + 2], a.z, sq0); sq0 = fmaf(qlo[4 * v + 3], a.w, sq0);
                sx0 += (a.x + a.y) + (a.z + a.w);
                sq1 = fmaf(qhi[4 * v + 0], b.x, sq1); sq1 = fmaf(qhi[4 * v + 1], b.y, sq1);
                sq1 = fmaf(qhi[4 * v + 2], b.z, sq1); sq1 = fmaf(qhi[4 * v + 3], b.w, sq1);
                sx1 += (b.x + b.y) + (b.z + b.w);
            }
            acc[m] += (d0 * sq0 - m0 * sx0) + (d1 * sq1 - m1 * sx1);
        }
    }
}

__device__ __forceinline__ uint32_t ld_u32_2B(const uint8_t* p) {  // 4 bytes from a 2-byte-aligned address
    return (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p)) |
           ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p + 2)) << 16);
}

template <int MB>
__device__ __forceinline__ void dot_q6_k(const uint8_t* __restrict__ row, const float* __restrict__ x, int ldx, int k,
                                         int mcount, int lane, float (&acc)[MB]) {
    const int nunits = (k >> 8) * 16;
    for (int u = lane; u < nunits; u += 32) {
        const int sb = u >> 4, half = (u >> 3) & 1, j = u & 7, l0 = 4 * j;
        const uint8_t* blk = row + (int64_t)sb * Q6_K_BYTES;
        const uint32_t qla = ld_u32_2B(blk + 64 * half + l0);
        const uint32_t qlb = ld_u32_2B(blk + 64 * half + 32 + l0);
        const uint32_t qh = ld_u32_2B(blk + 128 + 32 * half + l0);
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + 8 * half + (j >> 2));
        const float d = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(blk + 208)));
        const float s1 = d * (float)sc[0], s2 = d * (float)sc[2], s3 = d * (float)sc[4], s4 = d * (float)sc[6];
        float q1[4], q2[4], q3[4], q4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t a = (qla >> (8 * e)) & 0xFFu, b = (qlb >> (8 * e)) & 0xFFu, hb = (qh >> (8 * e)) & 0xFFu;
            q1[e] = (float)((int)((a & 0xFu) | ((hb & 3u) << 4)) - 32);
            q2[e] = (float)((int)((b & 0xFu) | (((hb >> 2) & 3u) << 4)) - 32);
            q3[e] = (float)((int)((a >> 4) | (((hb >> 4) & 3u) << 4)) - 32);
            q4[e] = (float)((int)((b >> 4) | (((hb >> 6) & 3u) << 4)) - 32);
        }
        const int xb = sb * 256 + half * 128 + l0;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const float* xm = x + (int64_t)(m < mcount ? m : mcount - 1) * ldx + xb;
            const float4 x1 = ldg_f4(xm), x2 = ldg_f4(xm + 32), x3 = ldg_f4(xm + 64), x4 = ldg_f4(xm + 96);
            const float t1 = fmaf(q1[0], x1.x, fmaf(q1[1], x1.y, fmaf(q1[2], x1.z, q1[3] * x1.w)));
            const float t2 = fmaf(q2[0], x2.x, fmaf(q2[1], x2.y, fmaf(q2[2], x2.z, q2[3] * x2.w)));
            const float t3 = fmaf(q3[0], x3.x, fmaf(q3[1], x3.y, fmaf(q3[2], x3.z, q3[3] * x3.w)));
            const float t4 = fmaf(q4[0], x4.x, fmaf(q4[1], x4.y, fmaf(q4[2], x4.z, q4[3] * x4.w)));
            acc[m] += (s1 * t1 + s2 * t2) + (s3 * t3 + s4 * t4);
        }
    }
}

template <int MB>
__device__ __forceinline__ void dot_q8_0(const uint8_t* __restrict__ row, const float* __restrict__ x, int ldx, int k,
                                         int mcount, int lane, float (&acc)[MB]) {
    const int nunits = (k >> 5) * 4;
    for (int u = lane; u < nunits; u += 32) {
        const int b = u >> 2, qtr = u & 3;
        const uint8_t* blk = row + (int64_t)b * Q8_0_BYTES;
        const float d = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(blk)));
        const uint32_t w0 = ld_u32_2B(blk + 2 + 8 * qtr), w1 = ld_u32_2B(blk + 6 + 8 * qtr);
        float q[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            q[e] = (float)(int8_t)((w0 >> (8 * e)) & 0xFFu);
            q[4 + e] = (float)(int8_t)((w1 >> (8 * e)) & 0xFFu);
        }
        const int xb = b * 32 + qtr * 8;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const float* xm = x + (int64_t)(m < mcount ? m : mcount - 1) * ldx + xb;
            const float4 a = ldg_f4(xm), c = ldg_f4(xm + 4);
            float t = q[0] * a.x;
            t = fmaf(q[1], a.y, t); t = fmaf(q[2], a.z, t); t = fmaf(q[3], a.w, t);
            t = fmaf(q[4], c.x, t); t = fmaf(q[5], c.y, t); t = fmaf(q[6], c.z, t); t = fmaf(q[7], c.w, t);
            acc[m] = fmaf(d, t, acc[m]);
        }
    }
}

// f32 / f16 / bf16 weights (norm-free float matrices are rare on this path; kept for completeness).
template <int MB>
__device__ __forceinline__ void dot_float(int dtype, const uint8_t* __restrict__ row, const float* __restrict__ x, int ldx,
                                          int k, int mcount, int lane, float (&acc)[MB]) {
    for (int i = lane; i < k; i += 32) {
        const float w = dequant_elem(dtype, row, i);
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = fmaf(w, __ldg(x + (int64_t)(m < mcount ? m : mcount - 1) * ldx + i), acc[m]);
    }
}

constexpr int GEMV_WARPS = 8;

template <int MB>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_kernel(const GemvArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int r = blockIdx.x * GEMV_WARPS + warp;
    int s = 0;
    while (s < a.nseg && r >= a.seg[s].n) { r -= a.seg[s].n; ++s; }
    if (s >= a.nseg) return;
    const int m0 = blockIdx.y * MB;
    const int mcount = min(MB, a.m - m0);
    const int dtype = a.seg[s].dtype;
    const uint8_t* row = a.seg[s].w + (int64_t)r * row_bytes(dtype, a.k);
    const float* x = a.x + (int64_t)m0 * a.ldx;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f;
    if (dtype == T_Q4_K) dot_q4_k<MB>(row, x, a.ldx, a.k, mcount, lane, acc);
    else if (dtype == T_Q6_K) dot_q6_k<MB>(row, x, a.ldx, a.k, mcount, lane, acc);
    else if (dtype == T_Q8_0) dot_q8_0<MB>(row, x, a.ldx, a.k, mcount, lane, acc);
    else dot_float<MB>(dtype, row, x, a.ldx, a.k, mcount, lane, acc);
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
        const float bias = a.seg[s].bias ? a.seg[s].bias[r] : 0.f;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            if (m < mcount) {
                float v = acc[m] + bias;
                if (s == 0 && a.res) v += a.res[(int64_t)(m0 + m) * a.ldres + r];
                a.seg[s].y[(int64_t)(m0 + m) * a.seg[s].ldy + r] = v;
            }
        }
    }
}

cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    int total = 0;
    for (int s = 0; s < a.nseg; ++s) total += a.seg[s].n;
    if (total == 0) return cudaSuccess;
    const int bx = (total + GEMV_WARPS - 1) / GEMV_WARPS;
    if (a.m == 1) gemv_kernel<1><<<dim3(bx, 1), GEMV_WARPS * 32, 0, st>>>(a);
    else if (a.m == 2) gemv_kernel<2><<<dim3(bx, 1), GEMV_WARPS * 32, 0, st>>>(a);
    else if (a.m <= 4) gemv_kernel<4><<<dim3(bx, 1), GEMV_WARPS * 32, 0, st>>>(a);
    else gemv_kernel<8><<<dim3(bx, (a.m + 7) / 8), GEMV_WARPS * 32, 0, st>>>(a);
    return finish_launch();
}

// ─────────────────────────────── norms ──────────────────────────────────────
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();  // protect sh from a previous use
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? sh[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

// yh != null: the row goes out as fp16 (input of the tensor-core GEMM) instead of f32.
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, int dim, float eps,
                                float* __restrict__ y, __half* __restrict__ yh) {
    __shared__ float sh[32];
    const float* s = x + (int64_t)blockIdx.x * dim;
    float acc = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) acc = fmaf(s[i], s[i], acc);
    const float sum = block_sum(acc, sh);
    const float inv = 1.0f / sqrtf(sum / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __fmul_rn(__fmul_rn(s[i], inv), w ? w[i] : 1.0f);
        if (yh) yh[(int64_t)blockIdx.x * dim + i] = __float2half_rn(v);
        else y[(int64_t)blockIdx.x * dim + i] = v;
    }
}

__global__ void layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                  int dim, float eps, float* __restrict__ y, __half* __restrict__ yh) {
    __shared__ float sh[32];
    const float* s = x + (int64_t)blockIdx.x * dim;
    float acc = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) acc += s[i];
    const float mean = block_sum(acc, sh) / (float)dim;
    float va = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float t = s[i] - mean; va = fmaf(t, t, va); }
    const float var = block_sum(va, sh) / (float)dim;
    const float inv = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = __fmul_rn(s[i] - mean, inv);
        if (w) v = __fmul_rn(v, w[i]);
        if (b) v = __fadd_rn(v, b[i]);
        if (yh) yh[(int64_t)blockIdx.x * dim + i] = __float2half_rn(v);
        else y[(int64_t)blockIdx.x * dim + i] = v;
    }
}

cudaError_t launch_rms_norm(const float* x, const float* w, int rows, int dim, float eps, float* y, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    rms_norm_kernel<<<rows, 256, 0, st>>>(x, w, dim, eps, y, nullptr);
    return finish_launch();
}
// Row norm to fp16 for many rows: the row is read once with 16-byte loads and stays in registers (up to eight float4 per
// thread, blockDim.x >= dim / 32), the result goes out as four halves per store. dim % 4 == 0.
template <bool LAYER_NORM>
__global__ void __launch_bounds__(1024) norm_rows_f16_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                                             int dim, float eps, __half* __restrict__ yh) {
    __shared__ float sh[32];
    pdl_wait();
    pdl_trigger();
    const float4* s = reinterpret_cast<const float4*>(x + (int64_t)blockIdx.x * dim);
    const int n4 = dim >> 2;
    float4 v[8];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        v[i] = c < n4 ? s[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        acc += LAYER_NORM ? (v[i].x + v[i].y) + (v[i].z + v[i].w) : fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, v[i].w * v[i].w)));
    }
    float mean = 0.f, inv;
    if (LAYER_NORM) {
        mean = block_sum(acc, sh) / (float)dim;
        float va = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (threadIdx.x + i * blockDim.x < n4) {
                const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
                va += fmaf(d0, d0, fmaf(d1, d1, fmaf(d2, d2, d3 * d3)));
            }
        }
        inv = 1.0f / sqrtf(block_sum(va, sh) / (float)dim + eps);
    } else {
        inv = 1.0f / sqrtf(block_sum(acc, sh) / (float)dim + eps);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
            const float4 ww = w ? reinterpret_cast<const float4*>(w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
            float o0, o1, o2, o3;
            if (LAYER_NORM) {
                const float4 bb = b ? reinterpret_cast<const float4*>(b)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
                o0 = __fmul_rn(v[i].x - mean, inv); o1 = __fmul_rn(v[i].y - mean, inv);
                o2 = __fmul_rn(v[i].z - mean, inv); o3 = __fmul_rn(v[i].w - mean, inv);
                if (w) { o0 = __fmul_rn(o0, ww.x); o1 = __fmul_rn(o1, ww.y); o2 = __fmul_rn(o2, ww.z); o3 = __fmul_rn(o3, ww.w); }
                o0 = __fadd_rn(o0, bb.x); o1 = __fadd_rn(o1, bb.y); o2 = __fadd_rn(o2, bb.z); o3 = __fadd_rn(o3, bb.w);
            } else {
                o0 = __fmul_rn(__fmul_rn(v[i].x, inv), ww.x); o1 = __fmul_rn(__fmul_rn(v[i].y, inv), ww.y);
                o2 = __fmul_rn(__fmul_rn(v[i].z, inv), ww.z); o3 = __fmul_rn(__fmul_rn(v[i].w, inv), ww.w);
            }
            const __half2 h01 = __floats2half2_rn(o0, o1), h23 = __floats2half2_rn(o2, o3);
            reinterpret_cast<uint2*>(yh + (int64_t)blockIdx.x * dim)[c] =
                make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        }
    }
}

static inline int norm_rows_threads(int dim) {  // 0: the shape does not fit the register-resident kernel
    if (dim % 4 != 0 || dim > 32768) return 0;
    const int t = ((dim / 32 + 31) / 32) * 32;
    return t < 32 ? 32 : t;
}

cudaError_t launch_rms_norm_f16(const float* x, const float* w, int rows, int dim, float eps, __half* yh, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (const int t = norm_rows_threads(dim)) {
        cudaError_t le = launch_pdl(norm_rows_f16_kernel<false>, dim3(rows), dim3(t), 0, st, x, w, (const float*)nullptr, dim, eps, yh);
        if (le != cudaSuccess) return le;
    } else {
        rms_norm_kernel<<<rows, 256, 0, st>>>(x, w, dim, eps, nullptr, yh);
    }
    return finish_launch();
}
cudaError_t launch_layer_norm_f16(const float* x, const float* w, const float* b, int rows, int dim, float eps, __half* yh,
                                  cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (const int t = norm_rows_threads(dim)) {
        cudaError_t le = launch_pdl(norm_rows_f16_kernel<true>, dim3(rows), dim3(t), 0, st, x, w, b, dim, eps, yh);
        if (le != cudaSuccess) return le;
    } else {
        layer_norm_kernel<<<rows, 256, 0, st>>>(x, w, b, dim, eps, nullptr, yh);
    }
    return finish_launch();
}
cudaError_t launch_layer_norm(const float* x, const float* w, const float* b, int rows, int dim, float eps, float* y,
                              cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    layer_norm_kernel<<<rows, 256, 0, st>>>(x, w, b, dim, eps, y, nullptr);
    return finish_launch();
}

// ───────────────────────── RoPE + paged-KV append ────────────────────────────
// NEOX rotate-half over the first rotary_dim channels; the pair (i, i+half) becomes
// (x0·c − x1·s, x1·c + x0·s) with each product rounded separately, as the reference's
// scalar code does. cos_sin[pos * half + i] = (cos θ, sin θ) with θ computed on the
// host exactly as the reference does (pos / base^(2i/rotary_dim) in f32).
__device__ __forceinline__ void rope_pair(float x0, float x1, float2 cs, float* o0, float* o1) {
    *o0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
    *o1 = __fadd_rn(__fmul_rn(x1, cs.x), __fmul_rn(x0, cs.y));
}

__device__ __forceinline__ int64_t kv_offset(const KvGeom& kv, int layer, int page, int which, int head) {
    return ((((int64_t)layer * kv.n_pages + page) * 2 + which) * kv.n_kv + head) * (int64_t)(KV_PAGE * kv.head_dim);
}

// kv_round != 0 (head_dim % 32 == 0): before the fp16 store every 32-element block of the new K / V row goes through
// the reference's Q8_0 cache rounding (scale = amax / 127 kept as f16, value = round(x / scale) * scale;
// crates/sapient-models/src/forward/common.rs:336-348,449-538), so attention sees the values the reference's
// quantised cache yields (to one extra fp16 rounding, 2^-12 relative).
__global__ void rope_kv_append_kernel(float* __restrict__ qkv, int n_heads, int n_kv, int head_dim, int rotary_dim,
                                      const float2* __restrict__ cos_sin, const int32_t* __restrict__ tok_slot,
                                      const int32_t* __restrict__ tok_pos, KvGeom kv, int layer, int kv_round) {
    __shared__ float sh_row[256];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, j = blockIdx.y;
    const int pos = tok_pos[t], slot = tok_slot[t];
    const int half = rotary_dim >> 1;
    const int ld = (n_heads + 2 * n_kv) * head_dim;
    float* v = qkv + (int64_t)t * ld + (int64_t)j * head_dim;
    __half* dst = nullptr;
    bool rotate = true;
    if (j >= n_heads) {
        const int which = (j >= n_heads + n_kv) ? 1 : 0;
        const int head = j - n_heads - which * n_kv;
        const int page = kv.page_table[(int64_t)slot * kv.max_pages + pos / KV_PAGE];
        dst = kv.pool + kv_offset(kv, layer, page, which, head) + (int64_t)(pos % KV_PAGE) * head_dim;
        rotate = (which == 0);
    }
    for (int p = threadIdx.x; p < head_dim / 2; p += blockDim.x) {
        int i0, i1;
        float o0, o1;
        if (p < half) {
            i0 = p; i1 = p + half;
            if (rotate) rope_pair(v[i0], v[i1], cos_sin[(int64_t)pos * half + p], &o0, &o1);
            else { o0 = v[i0]; o1 = v[i1]; }
        } else {
            i0 = rotary_dim + 2 * (p - half); i1 = i0 + 1;
            o0 = v[i0]; o1 = v[i1];
        }
        if (dst && kv_round) { sh_row[i0] = o0; sh_row[i1] = o1; }
        else if (dst) { dst[i0] = __float2half_rn(o0); dst[i1] = __float2half_rn(o1); }
        else { v[i0] = o0; v[i1] = o1; }
    }
    if (dst && kv_round) {  // block-uniform
        __syncthreads();
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
        for (int b = warp; b < head_dim / 32; b += n_warps) {
            const float x = sh_row[b * 32 + lane];
            const float amax = warp_max(fabsf(x));
            const float scale = amax / 127.0f;
            const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
            float r = roundf(x * inv);  // half away from zero, like f32::round
            r = fminf(fmaxf(r, -127.0f), 127.0f);
            const float d = __half2float(__float2half_rn(scale));
            dst[b * 32 + lane] = __float2half_rn(__fmul_rn(r, d));
        }
    }
}

// The same for many tokens: one warp per (token, head), eight heads per block.
__global__ void __launch_bounds__(256) rope_kv_append_rows_kernel(float* __restrict__ qkv, int n_heads, int n_kv, int head_dim, int rotary_dim,
                                                                  const float2* __restrict__ cos_sin, const int32_t* __restrict__ tok_slot,
                                                                  const int32_t* __restrict__ tok_pos, KvGeom kv, int layer, int kv_round) {
    __shared__ float sh_rows[8][256];
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, j = blockIdx.y * 8 + warp;
    if (j >= n_heads + 2 * n_kv) return;
    float* sh_row = sh_rows[warp];
    const int pos = tok_pos[t], slot = tok_slot[t];
    const int half = rotary_dim >> 1;
    const int ld = (n_heads + 2 * n_kv) * head_dim;
    float* v = qkv + (int64_t)t * ld + (int64_t)j * head_dim;
    __half* dst = nullptr;
    bool rotate = true;
    if (j >= n_heads) {
        const int which = (j >= n_heads + n_kv) ? 1 : 0;
        const int head = j - n_heads - which * n_kv;
        const int page = kv.page_table[(int64_t)slot * kv.max_pages + pos / KV_PAGE];
        dst = kv.pool + kv_offset(kv, layer, page, which, head) + (int64_t)(pos % KV_PAGE) * head_dim;
        rotate = (which == 0);
    }
    for (int p = lane; p < head_dim / 2; p += 32) {
        int i0, i1;
        float o0, o1;
        if (p < half) {
            i0 = p; i1 = p + half;
            if (rotate) rope_pair(v[i0], v[i1], cos_sin[(int64_t)pos * half + p], &o0, &o1);
            else { o0 = v[i0]; o1 = v[i1]; }
        } else {
            i0 = rotary_dim + 2 * (p - half); i1 = i0 + 1;
            o0 = v[i0]; o1 = v[i1];
        }
        if (dst && kv_round) { sh_row[i0] = o0; sh_row[i1] = o1; }
        else if (dst) { dst[i0] = __float2half_rn(o0); dst[i1] = __float2half_rn(o1); }
        else { v[i0] = o0; v[i1] = o1; }
    }
    if (dst && kv_round) {  // warp-uniform
        __syncwarp();
        for (int b = 0; b < head_dim / 32; ++b) {
            const float x = sh_row[b * 32 + lane];
            const float amax = warp_max(fabsf(x));
            const float scale = amax / 127.0f;
            const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
            float r = roundf(x * inv);  // half away from zero, like f32::round
            r = fminf(fmaxf(r, -127.0f), 127.0f);
            const float d = __half2float(__float2half_rn(scale));
            dst[b * 32 + lane] = __float2half_rn(__fmul_rn(r, d));
        }
    }
}

cudaError_t launch_rope_kv_append(float* qkv, int n_tok, int n_heads, int n_kv, int head_dim, int rotary_dim,
                                  const float2* cos_sin, const int32_t* tok_slot, const int32_t* tok_pos, KvGeom kv,
                                  int layer, int kv_round, cudaStream_t st) {
    if (n_tok == 0) return cudaSuccess;
    if (head_dim % 32 != 0 || head_dim > 256) kv_round = 0;
    if (n_tok >= 32) {
        cudaError_t le = launch_pdl(rope_kv_append_rows_kernel, dim3(n_tok, (n_heads + 2 * n_kv + 7) / 8), dim3(256), 0, st, qkv, n_heads, n_kv,
                                    head_dim, rotary_dim, cos_sin, tok_slot, tok_pos, kv, layer, kv_round);
        if (le != cudaSuccess) return le;
        return finish_launch();
    }
    cudaError_t le = launch_pdl(rope_kv_append_kernel, dim3(n_tok, n_heads + 2 * n_kv), dim3(64), 0, st, qkv, n_heads, n_kv, head_dim,
                                rotary_dim, cos_sin, tok_slot, tok_pos, kv, layer, kv_round);
    if (le != cudaSuccess) return le;
    return finish_launch();
}

__global__ void rope_kernel(float* __restrict__ x, int head_dim, int rotary_dim, const float2* __restrict__ cos_sin,
                            const int32_t* __restrict__ tok_pos, int ld) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int half = rotary_dim >> 1;
    float* v = x + (int64_t)t * ld + (int64_t)h * head_dim;
    const int pos = tok_pos[t];
    for (int p = threadIdx.x; p < half; p += blockDim.x) {
        float o0, o1;
        rope_pair(v[p], v[p + half], cos_sin[(int64_t)pos * half + p], &o0, &o1);
        v[p] = o0; v[p + half] = o1;
    }
}

cudaError_t launch_rope(float* x, int n_tok, int n_heads, int head_dim, int rotary_dim, const float2* cos_sin,
                        const int32_t* tok_pos, int ld, cudaStream_t st) {
    if (n_tok == 0) return cudaSuccess;
    rope_kernel<<<dim3(n_tok, n_heads), 64, 0, st>>>(x, head_dim, rotary_dim, cos_sin, tok_pos, ld);
    return finish_launch();
}

// ─────────────────────────────── elementwise ─────────────────────────────────
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_f(float v) {
    const float inner = __fmul_rn(0.79788456f, __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v)));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
}

__global__ void swiglu_kernel(const float* __restrict__ gu, int ld, int ffn, int64_t total, float* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / ffn, c = i - r * ffn;
        const float g = gu[r * ld + c], u = gu[r * ld + ffn + c];
        out[i] = __fmul_rn(silu_f(g), u);
    }
}
// The MLP activation straight to fp16 [rows][ffn]: kind 0 = silu(gate) * up with gate | up side by side in a row of gu,
// kind 1 = gelu. One row per blockIdx.y, four columns per thread (ffn % 4 == 0, ld % 4 == 0).
__global__ void act_f16_kernel(const float* __restrict__ gu, int ld, int ffn, int kind, __half* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= ffn) return;
    const float* row = gu + (int64_t)blockIdx.y * ld;
    const float4 g = *reinterpret_cast<const float4*>(row + c);
    float a0, a1, a2, a3;
    if (kind == 0) {
        const float4 u = *reinterpret_cast<const float4*>(row + ffn + c);
        a0 = __fmul_rn(silu_f(g.x), u.x); a1 = __fmul_rn(silu_f(g.y), u.y);
        a2 = __fmul_rn(silu_f(g.z), u.z); a3 = __fmul_rn(silu_f(g.w), u.w);
    } else {
        a0 = gelu_f(g.x); a1 = gelu_f(g.y); a2 = gelu_f(g.z); a3 = gelu_f(g.w);
    }
    const __half2 h01 = __floats2half2_rn(a0, a1), h23 = __floats2half2_rn(a2, a3);
    *reinterpret_cast<uint2*>(out + (int64_t)blockIdx.y * ffn + c) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
}
__global__ void gelu_kernel(float* x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] = gelu_f(x[i]);
}
__global__ void silu_kernel(float* x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] = silu_f(x[i]);
}
__global__ void add_kernel(const float* a, const float* b, float* y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = a[i] + b[i];
}
__global__ void mul_kernel(const float* a, const float* b, float* y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = a[i] * b[i];
}

static inline int ew_blocks(int64_t n) {
    int64_t b = (n + 255) / 256;
    return (int)(b < 148 * 8 ? (b < 1 ? 1 : b) : 148 * 8);
}

cudaError_t launch_swiglu(const float* gate_up, int ld, int ffn, int rows, float* out, cudaStream_t st) {
    const int64_t total = (int64_t)rows * ffn;
    if (total == 0) return cudaSuccess;
    swiglu_kernel<<<ew_blocks(total), 256, 0, st>>>(gate_up, ld, ffn, total, out);
    return finish_launch();
}
cudaError_t launch_act_f16(const float* gu, int ld, int ffn, int rows, int kind, __half* out, cudaStream_t st) {
    if (rows == 0 || ffn == 0) return cudaSuccess;
    if ((ffn & 3) || (ld & 3)) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(act_f16_kernel, dim3((ffn / 4 + 255) / 256, rows), dim3(256), 0, st, gu, ld, ffn, kind, out);
    if (le != cudaSuccess) return le;
    return finish_launch();
}
cudaError_t launch_gelu(float* x, int64_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    gelu_kernel<<<ew_blocks(n), 256, 0, st>>>(x, n);
    return finish_launch();
}
cudaError_t launch_silu(float* x, int64_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    silu_kernel<<<ew_blocks(n), 256, 0, st>>>(x, n);
    return finish_launch();
}
cudaError_t launch_add(const float* a, const float* b, float* y, int64_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    add_kernel<<<ew_blocks(n), 256, 0, st>>>(a, b, y, n);
    return finish_launch();
}
cudaError_t launch_mul(const float* a, const float* b, float* y, int64_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    mul_kernel<<<ew_blocks(n), 256, 0, st>>>(a, b, y, n);
    return finish_launch();
}

// ─────────────────────────────── argmax ─────────────────────────────────────
// Ties resolve to the LAST index holding the maximum, like Iterator::max_by.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int n, int ld, uint32_t* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (int64_t)blockIdx.x * ld;
    float best = -INFINITY;
    int bi = -1;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (bi < 0 || v >= best) { best = v; bi = i; }
    }
    auto better = [](float v, int i, float bv, int b) { return i >= 0 && (b < 0 || v > bv || (v == bv && i > b)); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (uint32_t)(bi < 0 ? 0 : bi);
    }
}

// The same over ARGMAX_PARTS blocks per row: each block scans one slice, leaves its (value, index) candidate in scratch
// and counts its arrival; the last block of the row picks among the candidates. "Greatest value, among equals the
// greatest index" is associative and commutative, so the result does not depend on the order of arrival.
// scratch: [rows][ARGMAX_PARTS] float2 (value, index bits) followed by [rows] arrival counters (zero between launches).
__global__ void __launch_bounds__(256) argmax_parts_kernel(const float* __restrict__ logits, int n, int ld, uint32_t* __restrict__ out,
                                                          float2* __restrict__ cand, unsigned* __restrict__ cnt) {
    pdl_wait();
    pdl_trigger();
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool last;
    const int row_i = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
    const float* row = logits + (int64_t)row_i * ld;
    const int per = (n + parts - 1) / parts, lo = part * per, hi = min(n, lo + per);
    auto better = [](float v, int i, float bv, int b) { return i >= 0 && (b < 0 || v > bv || (v == bv && i > b)); };
    float best = -INFINITY;
    int bi = -1;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (bi < 0 || v >= best) { best = v; bi = i; }
    }
    auto warp_reduce = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
    };
    warp_reduce();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < 8 ? sv[lane] : -INFINITY;
        bi = lane < 8 ? si[lane] : -1;
        warp_reduce();
        if (lane == 0) {
            cand[(int64_t)row_i * parts + part] = make_float2(best, __int_as_float(bi));
            __threadfence();
            last = atomicAdd(&cnt[row_i], 1u) == (unsigned)(parts - 1);
        }
    }
    __syncthreads();
    if (!last || warp != 0) return;
    __threadfence();
    best = -INFINITY;
    bi = -1;
    for (int p = lane; p < parts; p += 32) {
        const float2 c = __ldcg(&cand[(int64_t)row_i * parts + p]);
        const int ci = __float_as_int(c.y);
        if (better(c.x, ci, best, bi)) { best = c.x; bi = ci; }
    }
    warp_reduce();
    if (lane == 0) {
        out[row_i] = (uint32_t)(bi < 0 ? 0 : bi);
        cnt[row_i] = 0u;
    }
}

cudaError_t launch_argmax(const float* logits, int rows, int n, int ld, uint32_t* out, cudaStream_t st, void* scratch) {
    if (rows == 0) return cudaSuccess;
    cudaError_t le;
    if (scratch && n >= 8192) {
        float2* cand = reinterpret_cast<float2*>(scratch);
        unsigned* cnt = reinterpret_cast<unsigned*>(cand + (size_t)ARGMAX_MAX_ROWS * ARGMAX_PARTS);
        if (rows > ARGMAX_MAX_ROWS) return cudaErrorInvalidValue;
        le = launch_pdl(argmax_parts_kernel, dim3(ARGMAX_PARTS, rows), dim3(256), 0, st, logits, n, ld, out, cand, cnt);
    } else {
        le = launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, st, logits, n, ld, out);
    }
    if (le != cudaSuccess) return le;
    return finish_launch();
}

__global__ void gather_rows_kernel(const float* __restrict__ src, int ld, const int32_t* __restrict__ rows, int dim,
                                   float* __restrict__ dst) {
    const float* s = src + (int64_t)rows[blockIdx.x] * ld;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[(int64_t)blockIdx.x * dim + i] = s[i];
}
cudaError_t launch_gather_rows(const float* src, int ld, const int32_t* rows, int n_rows, int dim, float* dst,
                               cudaStream_t st) {
    if (n_rows == 0) return cudaSuccess;
    gather_rows_kernel<<<n_rows, 256, 0, st>>>(src, ld, rows, dim, dst);
    return finish_launch();
}

}  // namespace sp
