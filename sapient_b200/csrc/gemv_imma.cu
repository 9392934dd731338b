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

#include "kernels.h"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

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
// One warp per (256 columns, activation row); lane handles 8 consecutive columns.
__global__ void __launch_bounds__(32) act_quant_kernel(const float* __restrict__ x, int ldx, int k, int digits, int eb, int ncp,
                                                       int8_t* __restrict__ xq, float* __restrict__ colscale,
                                                       int32_t* __restrict__ xsum, int32_t* __restrict__ cinit16) {
    const int lane = threadIdx.x, m = blockIdx.y;
    const int k0 = blockIdx.x * 256 + lane * 8;
    const bool live = k0 < k;
    float v[8];
    float amax = 0.f;
    if (live) {
        const float4 a = *reinterpret_cast<const float4*>(x + (int64_t)m * ldx + k0);
        const float4 b = *reinterpret_cast<const float4*>(x + (int64_t)m * ldx + k0 + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    // exponent block: the 4 lanes of a 32-column block, or the whole warp
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    if (eb == 256) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 8));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 16));
    }
    const int P = 8 * digits - 2;
    int e = 0;
    float up = 0.f, down = 0.f;  // x * up -> fixed point; digit 0 scale = down
    if (amax > 0.f && amax < INFINITY) {
        e = ilogbf(amax) + 1;              // amax < 2^e
        e = max(e, -100);                  // keep 2^(P-e) finite
        up = scalbnf(1.0f, P - e);         // exact powers of two
        down = scalbnf(1.0f, e - P);
    }
    int dg[3][8];
    int sum[3] = {0, 0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int X = __float2int_rn(v[i] * up);
        const int lim = 1 << P;
        X = max(-lim, min(lim, X));
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            int q;
            if (d == digits - 1) { q = X; }
            else { q = ((X + 128) & 255) - 128; X = (X - q) >> 8; }
            if (d >= digits) q = 0;
            dg[d][i] = q;
            sum[d] += q;
        }
    }
    const int blk32 = k0 >> 5, a4 = lane & 3;
    // fragment order inside a 32-block: byte p = 8 t' + 4 h + i  <->  column 16 h + 4 t' + i
    const int h = a4 >> 1, t0 = 2 * (a4 & 1);
    for (int d = 0; d < digits && live; ++d) {
        const int col = m * digits + d;
        int8_t* dst = xq + (int64_t)col * k + (int64_t)blk32 * 32;
        const uint32_t w0 = (uint32_t)(dg[d][0] & 255) | ((uint32_t)(dg[d][1] & 255) << 8) | ((uint32_t)(dg[d][2] & 255) << 16) |
                            ((uint32_t)(dg[d][3] & 255) << 24);
        const uint32_t w1 = (uint32_t)(dg[d][4] & 255) | ((uint32_t)(dg[d][5] & 255) << 8) | ((uint32_t)(dg[d][6] & 255) << 16) |
                            ((uint32_t)(dg[d][7] & 255) << 24);
        *reinterpret_cast<uint32_t*>(dst + 8 * t0 + 4 * h) = w0;
        *reinterpret_cast<uint32_t*>(dst + 8 * (t0 + 1) + 4 * h) = w1;
    }
    // per-16 and per-32 digit sums
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        const int s16 = sum[d] + __shfl_xor_sync(0xFFFFFFFFu, sum[d], 1);
        const int s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
        if (d < digits && live) {
            const int col = m * digits + d;
            if ((lane & 1) == 0) cinit16[(int64_t)(k0 >> 4) * ncp + col] = -32 * s16;
            if (a4 == 0) xsum[(int64_t)blk32 * ncp + col] = s32;
        }
    }
    const bool writer = (eb == 256) ? (lane == 0) : (a4 == 0);
    if (writer && live) {
        float s = down;
        for (int d = 0; d < digits; ++d) {
            colscale[(int64_t)(k0 / eb) * ncp + m * digits + d] = s;
            s *= 256.f;
        }
    }
}

cudaError_t launch_act_quant(const float* x, int ldx, int m, int k, int digits, int eb, int ncp, int8_t* xq, float* colscale,
                             int32_t* xsum, int32_t* cinit16, cudaStream_t st) {
    if (m <= 0) return cudaSuccess;
    act_quant_kernel<<<dim3((k + 255) / 256, m), 32, 0, st>>>(x, ldx, k, digits, eb, ncp, xq, colscale, xsum, cinit16);
    return count_launch_and_check();
}

// ─────────────────────────────── the GEMV ────────────────────────────────────
__device__ __forceinline__ void imma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

__device__ __forceinline__ uint4 ldg_u4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ int byte_u(uint32_t w, int i) { return (int)((w >> (8 * i)) & 0xFFu); }
__device__ __forceinline__ int byte_s(uint32_t w, int i) { return (int)(int8_t)((w >> (8 * i)) & 0xFFu); }

constexpr int IMMA_WARPS = 8;

// B fragments (digit words) of the eight 32-blocks of one 256-column tile for n-tile nt.
template <int NT>
__device__ __forceinline__ void load_b256(const ImmaArgs& a, int kt, int g, int t, uint2 (&b)[NT][8]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
        const bool on = col < a.m * a.digits;
        const int8_t* base = a.xq + (int64_t)col * a.k + (int64_t)kt * 256 + 8 * t;
#pragma unroll
        for (int s = 0; s < 8; ++s) b[nt][s] = on ? __ldg(reinterpret_cast<const uint2*>(base + 32 * s)) : make_uint2(0u, 0u);
    }
}

template <int NT>
__device__ __forceinline__ void tile_q4_k(const ImmaArgs& a, const uint8_t* tile, int kt, int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    uint4 q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = ldg_u4(tile + j * 512 + lane * 16);
    const uint4 h0 = ldg_u4(tile + 2048 + g * 16), h1 = ldg_u4(tile + 2048 + (g + 8) * 16);
    uint2 b[NT][8];
    load_b256<NT>(a, kt, g, t, b);
    // 6-bit scales / mins of the two rows -> one byte each
    uint32_t sc[2][2], mn[2][2];
    {
        const uint4 hh[2] = {h0, h1};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t u0 = hh[r].y, u1 = hh[r].z, u2 = hh[r].w;
            sc[r][0] = u0 & 0x3f3f3f3fu;
            sc[r][1] = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
            mn[r][0] = u1 & 0x3f3f3f3fu;
            mn[r][1] = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
        }
    }
    int D[NT][4], Dm[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) { D[nt][e] = 0; Dm[nt][e] = 0; }
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int j = s >> 1, sh = (s & 1) * 4;
        const uint32_t a0 = (q[j].x >> sh) & 0x0F0F0F0Fu, a2 = (q[j].y >> sh) & 0x0F0F0F0Fu;
        const uint32_t a1 = (q[j].z >> sh) & 0x0F0F0F0Fu, a3 = (q[j].w >> sh) & 0x0F0F0F0Fu;
        const int sc0 = byte_u(sc[0][s >> 2], s & 3), sc1 = byte_u(sc[1][s >> 2], s & 3);
        const int m0 = byte_u(mn[0][s >> 2], s & 3), m1 = byte_u(mn[1][s >> 2], s & 3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int c[4] = {0, 0, 0, 0};
            imma_k32(c, a0, a1, a2, a3, b[nt][s].x, b[nt][s].y);
            D[nt][0] += sc0 * c[0]; D[nt][1] += sc0 * c[1];
            D[nt][2] += sc1 * c[2]; D[nt][3] += sc1 * c[3];
            const int2 xs = __ldg(reinterpret_cast<const int2*>(a.xsum + (int64_t)(kt * 8 + s) * a.ncp + nt * 8 + 2 * t));
            Dm[nt][0] += m0 * xs.x; Dm[nt][1] += m0 * xs.y;
            Dm[nt][2] += m1 * xs.x; Dm[nt][3] += m1 * xs.y;
        }
    }
    const float d0 = half_bits_to_float((uint16_t)(h0.x & 0xFFFFu)), dm0 = half_bits_to_float((uint16_t)(h0.x >> 16));
    const float d1 = half_bits_to_float((uint16_t)(h1.x & 0xFFFFu)), dm1 = half_bits_to_float((uint16_t)(h1.x >> 16));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 cs = __ldg(reinterpret_cast<const float2*>(a.colscale + (int64_t)(kt * 256 / a.eb) * a.ncp + nt * 8 + 2 * t));
        acc[nt][0] = fmaf(cs.x, d0 * (float)D[nt][0] - dm0 * (float)Dm[nt][0], acc[nt][0]);
        acc[nt][1] = fmaf(cs.y, d0 * (float)D[nt][1] - dm0 * (float)Dm[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf(cs.x, d1 * (float)D[nt][2] - dm1 * (float)Dm[nt][2], acc[nt][2]);
        acc[nt][3] = fmaf(cs.y, d1 * (float)D[nt][3] - dm1 * (float)Dm[nt][3], acc[nt][3]);
    }
}

template <int NT>
__device__ __forceinline__ void tile_q6_k(const ImmaArgs& a, const uint8_t* tile, int kt, int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t w[24];
#pragma unroll
    for (int i = 0; i < 6; ++i) {
        const uint4 v = ldg_u4(tile + i * 512 + lane * 16);
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
    const uint4 s0 = ldg_u4(tile + 3072 + g * 16), s1 = ldg_u4(tile + 3072 + (g + 8) * 16);
    const float d0 = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(tile + 3328 + 2 * g)));
    const float d1 = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(tile + 3328 + 2 * (g + 8))));
    uint2 b[NT][8];
    load_b256<NT>(a, kt, g, t, b);
    const uint32_t sw0[4] = {s0.x, s0.y, s0.z, s0.w}, sw1[4] = {s1.x, s1.y, s1.z, s1.w};
    int D[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) D[nt][e] = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {       // c = (half, p)
        const int half = c >> 1, p = c & 1;
        const uint32_t qlA0 = w[6 * c], qlB0 = w[6 * c + 1], qh0 = w[6 * c + 2];
        const uint32_t qlA1 = w[6 * c + 3], qlB1 = w[6 * c + 4], qh1 = w[6 * c + 5];
#pragma unroll
        for (int Q = 0; Q < 4; ++Q) {   // quarter: 32-column slice of the 128-half
            const uint32_t l0 = (Q & 1) ? qlB0 : qlA0, l1 = (Q & 1) ? qlB1 : qlA1;
            const uint32_t n0 = (Q >= 2) ? (l0 >> 4) : l0, n1 = (Q >= 2) ? (l1 >> 4) : l1;
            const uint32_t hb0 = Q == 0 ? (qh0 << 4) : Q == 1 ? (qh0 << 2) : Q == 2 ? qh0 : (qh0 >> 2);
            const uint32_t hb1 = Q == 0 ? (qh1 << 4) : Q == 1 ? (qh1 << 2) : Q == 2 ? qh1 : (qh1 >> 2);
            const uint32_t a0 = (n0 & 0x0F0F0F0Fu) | (hb0 & 0x30303030u);  // unsigned 0..63; the -32 rides in the C init
            const uint32_t a1 = (n1 & 0x0F0F0F0Fu) | (hb1 & 0x30303030u);
            const int gi = 8 * half + 2 * Q + p;   // 16-column scale group
            const int blk = 4 * half + Q;          // 32-block of the tile
            const int sc0 = byte_s(sw0[gi >> 2], gi & 3), sc1 = byte_s(sw1[gi >> 2], gi & 3);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int2 ci = __ldg(reinterpret_cast<const int2*>(a.cinit16 + (int64_t)(kt * 16 + gi) * a.ncp + nt * 8 + 2 * t));
                int cc[4] = {ci.x, ci.y, ci.x, ci.y};
                imma_k16(cc, a0, a1, p ? b[nt][blk].y : b[nt][blk].x);
                D[nt][0] += sc0 * cc[0]; D[nt][1] += sc0 * cc[1];
                D[nt][2] += sc1 * cc[2]; D[nt][3] += sc1 * cc[3];
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 cs = __ldg(reinterpret_cast<const float2*>(a.colscale + (int64_t)(kt * 256 / a.eb) * a.ncp + nt * 8 + 2 * t));
        acc[nt][0] = fmaf(cs.x * d0, (float)D[nt][0], acc[nt][0]);
        acc[nt][1] = fmaf(cs.y * d0, (float)D[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf(cs.x * d1, (float)D[nt][2], acc[nt][2]);
        acc[nt][3] = fmaf(cs.y * d1, (float)D[nt][3], acc[nt][3]);
    }
}

// Q8_0: one tile = bpt 32-blocks; kt counts tiles.
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
            if (col < a.m * a.digits) b = __ldg(reinterpret_cast<const uint2*>(a.xq + (int64_t)col * a.k + (int64_t)blk32 * 32 + 8 * t));
            int c[4] = {0, 0, 0, 0};
            imma_k32(c, q.x, q.z, q.y, q.w, b.x, b.y);
            const float2 cs = __ldg(reinterpret_cast<const float2*>(a.colscale + (int64_t)(blk32 * 32 / a.eb) * a.ncp + nt * 8 + 2 * t));
            acc[nt][0] = fmaf(cs.x * d0, (float)c[0], acc[nt][0]);
            acc[nt][1] = fmaf(cs.y * d0, (float)c[1], acc[nt][1]);
            acc[nt][2] = fmaf(cs.x * d1, (float)c[2], acc[nt][2]);
            acc[nt][3] = fmaf(cs.y * d1, (float)c[3], acc[nt][3]);
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(IMMA_WARPS * 32) gemv_imma_kernel(const ImmaArgs a) {
    __shared__ float red[IMMA_WARPS][NT][4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int rt = blockIdx.x, s = 0;
    while (s < a.nseg - 1 && rt >= (a.seg[s].n + 15) / 16) { rt -= (a.seg[s].n + 15) / 16; ++s; }
    const ImmaSeg& sg = a.seg[s];
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    if (sg.dtype == T_Q4_K) {
        const int kts = a.k >> 8;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * Q4_K_TILE_BYTES;
        for (int kt = warp; kt < kts; kt += IMMA_WARPS) tile_q4_k<NT>(a, base + (int64_t)kt * Q4_K_TILE_BYTES, kt, lane, acc);
    } else if (sg.dtype == T_Q6_K) {
        const int kts = a.k >> 8;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * Q6_K_TILE_BYTES;
        for (int kt = warp; kt < kts; kt += IMMA_WARPS) tile_q6_k<NT>(a, base + (int64_t)kt * Q6_K_TILE_BYTES, kt, lane, acc);
    } else {
        const int bpt = sg.bpt, kts = (a.k >> 5) / bpt, tb = bpt * 544;
        const uint8_t* base = sg.wt + (int64_t)rt * kts * tb;
        for (int kt = warp; kt < kts; kt += IMMA_WARPS) tile_q8_0<NT>(a, base + (int64_t)kt * tb, kt, bpt, lane, acc);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][nt][e][lane] = acc[nt][e];
    __syncthreads();
    // element (row r of the tile, activation m): sum over warps and over the row's digit columns
    for (int idx = threadIdx.x; idx < 16 * a.m; idx += blockDim.x) {
        const int r = idx & 15, m = idx >> 4;
        const int64_t row = (int64_t)rt * 16 + r;
        if (row >= sg.n) continue;
        float v = 0.f;
        for (int d = 0; d < a.digits; ++d) {
            const int col = m * a.digits + d, nt = col >> 3, cc = col & 7;
            const int e = (r < 8 ? 0 : 2) + (cc & 1), ln = (r & 7) * 4 + (cc >> 1);
#pragma unroll
            for (int w = 0; w < IMMA_WARPS; ++w) v += red[w][nt][e][ln];
        }
        if (sg.bias) v += sg.bias[row];
        if (s == 0 && a.res) v += a.res[(int64_t)m * a.ldres + row];
        sg.y[(int64_t)m * sg.ldy + row] = v;
    }
}

cudaError_t ActWorkspace::alloc(int k_max_) {
    release();
    k_max = (k_max_ + 255) / 256 * 256;
    cudaError_t e;
    if ((e = cudaMalloc((void**)&xq, (size_t)NCP_MAX * k_max)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&colscale, (size_t)(k_max / 32) * NCP_MAX * 4)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&xsum, (size_t)(k_max / 32) * NCP_MAX * 4)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&cinit16, (size_t)(k_max / 16) * NCP_MAX * 4)) != cudaSuccess) return e;
    // unused digit columns are read (and multiplied by zero sums): keep them finite
    cudaMemset(xq, 0, (size_t)NCP_MAX * k_max);
    cudaMemset(colscale, 0, (size_t)(k_max / 32) * NCP_MAX * 4);
    cudaMemset(xsum, 0, (size_t)(k_max / 32) * NCP_MAX * 4);
    cudaMemset(cinit16, 0, (size_t)(k_max / 16) * NCP_MAX * 4);
    return cudaDeviceSynchronize();
}

void ActWorkspace::release() {
    if (xq) cudaFree(xq);
    if (colscale) cudaFree(colscale);
    if (xsum) cudaFree(xsum);
    if (cinit16) cudaFree(cinit16);
    xq = nullptr; colscale = nullptr; xsum = nullptr; cinit16 = nullptr; k_max = 0;
}

cudaError_t launch_quant_gemv(const float* x, int ldx, ImmaArgs& a, const ActWorkspace& ws, bool requantize, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    if (a.m > 16 || a.k > ws.k_max) return cudaErrorInvalidValue;
    // 3 digits while they fit one 8-column n-tile (m <= 2), else 2 digits
    a.digits = a.m <= 2 ? 3 : 2;
    const int cols = a.m * a.digits;
    a.ncp = cols <= 8 ? 8 : cols <= 16 ? 16 : 32;
    a.eb = (a.k % 256 == 0) ? 256 : 32;
    a.xq = ws.xq; a.colscale = ws.colscale; a.xsum = ws.xsum; a.cinit16 = ws.cinit16;
    if (requantize) {
        cudaError_t e = launch_act_quant(x, ldx, a.m, a.k, a.digits, a.eb, a.ncp, ws.xq, ws.colscale, ws.xsum, ws.cinit16, st);
        if (e != cudaSuccess) return e;
    }
    return launch_gemv_imma(a, st);
}

cudaError_t launch_gemv_imma(const ImmaArgs& a, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) tiles += (a.seg[s].n + 15) / 16;
    if (tiles == 0) return cudaSuccess;
    const int nt = a.ncp / 8;
    if (nt == 1) gemv_imma_kernel<1><<<tiles, IMMA_WARPS * 32, 0, st>>>(a);
    else if (nt == 2) gemv_imma_kernel<2><<<tiles, IMMA_WARPS * 32, 0, st>>>(a);
    else if (nt == 4) gemv_imma_kernel<4><<<tiles, IMMA_WARPS * 32, 0, st>>>(a);
    else return cudaErrorInvalidValue;
    return count_launch_and_check();
}

}  // namespace sp
