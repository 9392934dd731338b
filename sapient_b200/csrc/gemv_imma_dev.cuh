// Device-side building blocks of the tensor-core GEMV shared by its kernels (gemv_imma.cu: one CTA per tile row,
// per-warp streaming; gemv_ring.cu: persistent CTAs fed by a shared-memory ring): the integer mma wrappers, the
// register images of one weight tile per format, and the per-tile arithmetic. Layouts: gemv_imma.cuh.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemv_imma.cuh"
#include "sp_common.cuh"

namespace sp {

// d = a * b + c on the integer tensor path; c may be literal zeros.
__device__ __forceinline__ void imma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                         int c0, int c1, int c2, int c3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}
__device__ __forceinline__ void imma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, int c0, int c1, int c2, int c3) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

__device__ __forceinline__ uint4 ldg_u4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint4 ld_u4(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ int byte_u(uint32_t w, int i) { return (int)((w >> (8 * i)) & 0xFFu); }
__device__ __forceinline__ int byte_s(uint32_t w, int i) { return (int)(int8_t)((w >> (8 * i)) & 0xFFu); }

constexpr int IMMA_WARPS = 8;

// Everything of the activation side that one lane needs for one 256-column tile and n-tile:
// w[2 * blk], w[2 * blk + 1] = the k 4t.. and k 16+4t.. digit words of 32-block blk for digit column nt * 8 + g;
// ra / rb = word t of the a / b halves of the digit-sum record (xs32d or xs16d); cs = scales of columns 2t, 2t+1.
template <int NT>
struct BFrag {
    uint32_t w[NT][16];
    uint32_t ra32[NT], rb32[NT], ra16[NT], rb16[NT];
    float2 cs[NT];
};

// From global memory (digits laid out as in gemv_imma.cuh). Columns past the live ones read zeros.
template <int NT>
__device__ __forceinline__ void load_b_global(const ImmaArgs& a, int kt, int g, int t, bool q4, bool q6, BFrag<NT>& b) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
        if (col < a.m * a.digits) {
            const int8_t* base = a.xq + (int64_t)col * a.kp + (int64_t)kt * 256 + t * 64;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = ldg_u4(base + 16 * i);
                b.w[nt][4 * i] = v.x; b.w[nt][4 * i + 1] = v.y; b.w[nt][4 * i + 2] = v.z; b.w[nt][4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) b.w[nt][i] = 0u;
        }
        const int64_t rec = ((int64_t)kt * a.ncp + col) * 32 + 4 * t;
        b.ra32[nt] = q4 ? __ldg(reinterpret_cast<const uint32_t*>(a.xs32d + rec)) : 0u;
        b.rb32[nt] = q4 ? __ldg(reinterpret_cast<const uint32_t*>(a.xs32d + rec + 16)) : 0u;
        b.ra16[nt] = q6 ? __ldg(reinterpret_cast<const uint32_t*>(a.xs16d + rec)) : 0u;
        b.rb16[nt] = q6 ? __ldg(reinterpret_cast<const uint32_t*>(a.xs16d + rec + 16)) : 0u;
        b.cs[nt] = __ldg(reinterpret_cast<const float2*>(a.colscale + (int64_t)kt * a.ncp + nt * 8 + 2 * t));
    }
}

// ── Q4_K ──
struct Q4Regs {
    uint4 q[4];
    uint4 h0, h1;
};
template <bool GLOBAL>
__device__ __forceinline__ void load_q4_k(const uint8_t* tile, int lane, Q4Regs& r) {
    const int g = lane >> 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) r.q[j] = GLOBAL ? ldg_u4(tile + j * 512 + lane * 16) : ld_u4(tile + j * 512 + lane * 16);
    r.h0 = GLOBAL ? ldg_u4(tile + 2048 + g * 16) : ld_u4(tile + 2048 + g * 16);
    r.h1 = GLOBAL ? ldg_u4(tile + 2048 + (g + 8) * 16) : ld_u4(tile + 2048 + (g + 8) * 16);
}

template <int NT>
__device__ __forceinline__ void compute_q4_k(const Q4Regs& r, const BFrag<NT>& b, int lane, float (&acc)[NT][4]) {
    const int t = lane & 3;
    // 6-bit scales / mins of rows g and g+8 unpacked to one byte each (sub-blocks 0..3 | 4..7)
    uint32_t sc[2][2], mn[2][2];
    {
        const uint4 hh[2] = {r.h0, r.h1};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t u0 = hh[i].y, u1 = hh[i].z, u2 = hh[i].w;
            sc[i][0] = u0 & 0x3f3f3f3fu;
            sc[i][1] = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
            mn[i][0] = u1 & 0x3f3f3f3fu;
            mn[i][1] = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
        }
    }
    int D[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) D[nt][e] = 0;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int j = s >> 1, sh = (s & 1) * 4;
        const uint32_t a0 = (r.q[j].x >> sh) & 0x0F0F0F0Fu, a2 = (r.q[j].y >> sh) & 0x0F0F0F0Fu;
        const uint32_t a1 = (r.q[j].z >> sh) & 0x0F0F0F0Fu, a3 = (r.q[j].w >> sh) & 0x0F0F0F0Fu;
        const int sc0 = byte_u(sc[0][s >> 2], s & 3), sc1 = byte_u(sc[1][s >> 2], s & 3);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int c[4];
            imma_k32(c, a0, a1, a2, a3, b.w[nt][2 * s], b.w[nt][2 * s + 1], 0, 0, 0, 0);
            D[nt][0] += sc0 * c[0]; D[nt][1] += sc0 * c[1];
            D[nt][2] += sc1 * c[2]; D[nt][3] += sc1 * c[3];
        }
    }
    // minimum term: sum_s m_s * S_s as two k16 mma over the sub-block index (S = a + 64 b)
    const uint32_t am0 = t == 0 ? mn[0][0] : (t == 1 ? mn[0][1] : 0u);
    const uint32_t am1 = t == 0 ? mn[1][0] : (t == 1 ? mn[1][1] : 0u);
    const float d0 = half_bits_to_float((uint16_t)(r.h0.x & 0xFFFFu)), dm0 = half_bits_to_float((uint16_t)(r.h0.x >> 16));
    const float d1 = half_bits_to_float((uint16_t)(r.h1.x & 0xFFFFu)), dm1 = half_bits_to_float((uint16_t)(r.h1.x >> 16));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int ca[4], cb[4];
        imma_k16(ca, am0, am1, b.ra32[nt], 0, 0, 0, 0);
        imma_k16(cb, am0, am1, b.rb32[nt], 0, 0, 0, 0);
        const float2 cs = b.cs[nt];
        acc[nt][0] = fmaf(cs.x, d0 * (float)D[nt][0] - dm0 * (float)(ca[0] + 64 * cb[0]), acc[nt][0]);
        acc[nt][1] = fmaf(cs.y, d0 * (float)D[nt][1] - dm0 * (float)(ca[1] + 64 * cb[1]), acc[nt][1]);
        acc[nt][2] = fmaf(cs.x, d1 * (float)D[nt][2] - dm1 * (float)(ca[2] + 64 * cb[2]), acc[nt][2]);
        acc[nt][3] = fmaf(cs.y, d1 * (float)D[nt][3] - dm1 * (float)(ca[3] + 64 * cb[3]), acc[nt][3]);
    }
}

// ── Q6_K ──
struct Q6Regs {
    uint32_t w[24];
    uint4 s0, s1;
    uint32_t dd;  // d of row g | d of row g+8 << 16
};
template <bool GLOBAL>
__device__ __forceinline__ void load_q6_k(const uint8_t* tile, int lane, Q6Regs& r) {
    const int g = lane >> 2;
#pragma unroll
    for (int i = 0; i < 6; ++i) {
        const uint4 v = GLOBAL ? ldg_u4(tile + i * 512 + lane * 16) : ld_u4(tile + i * 512 + lane * 16);
        r.w[4 * i] = v.x; r.w[4 * i + 1] = v.y; r.w[4 * i + 2] = v.z; r.w[4 * i + 3] = v.w;
    }
    r.s0 = GLOBAL ? ldg_u4(tile + 3072 + g * 16) : ld_u4(tile + 3072 + g * 16);
    r.s1 = GLOBAL ? ldg_u4(tile + 3072 + (g + 8) * 16) : ld_u4(tile + 3072 + (g + 8) * 16);
    const uint16_t* dp = reinterpret_cast<const uint16_t*>(tile + 3328);
    r.dd = GLOBAL ? ((uint32_t)__ldg(dp + g) | ((uint32_t)__ldg(dp + g + 8) << 16)) : ((uint32_t)dp[g] | ((uint32_t)dp[g + 8] << 16));
}

template <int NT>
__device__ __forceinline__ void compute_q6_k(const Q6Regs& r, const BFrag<NT>& b, int lane, float (&acc)[NT][4]) {
    const int t = lane & 3;
    const uint32_t sw0[4] = {r.s0.x, r.s0.y, r.s0.z, r.s0.w}, sw1[4] = {r.s1.x, r.s1.y, r.s1.z, r.s1.w};
    int D[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) D[nt][e] = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {       // c = (half, p)
        const int half = c >> 1, p = c & 1;
        const uint32_t qlA0 = r.w[6 * c], qlB0 = r.w[6 * c + 1], qh0 = r.w[6 * c + 2];
        const uint32_t qlA1 = r.w[6 * c + 3], qlB1 = r.w[6 * c + 4], qh1 = r.w[6 * c + 5];
#pragma unroll
        for (int Q = 0; Q < 4; ++Q) {   // quarter: 32-column slice of the 128-half
            const uint32_t l0 = (Q & 1) ? qlB0 : qlA0, l1 = (Q & 1) ? qlB1 : qlA1;
            const uint32_t n0 = (Q >= 2) ? (l0 >> 4) : l0, n1 = (Q >= 2) ? (l1 >> 4) : l1;
            const uint32_t hb0 = Q == 0 ? (qh0 << 4) : Q == 1 ? (qh0 << 2) : Q == 2 ? qh0 : (qh0 >> 2);
            const uint32_t hb1 = Q == 0 ? (qh1 << 4) : Q == 1 ? (qh1 << 2) : Q == 2 ? qh1 : (qh1 >> 2);
            const uint32_t a0 = (n0 & 0x0F0F0F0Fu) | (hb0 & 0x30303030u);  // unsigned 0..63; the -32 is applied below
            const uint32_t a1 = (n1 & 0x0F0F0F0Fu) | (hb1 & 0x30303030u);
            const int gi = 8 * half + 2 * Q + p;   // 16-column scale group
            const int blk = 4 * half + Q;          // 32-block of the tile
            const int sc0 = byte_s(sw0[gi >> 2], gi & 3), sc1 = byte_s(sw1[gi >> 2], gi & 3);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int cc[4];
                imma_k16(cc, a0, a1, b.w[nt][2 * blk + p], 0, 0, 0, 0);
                D[nt][0] += sc0 * cc[0]; D[nt][1] += sc0 * cc[1];
                D[nt][2] += sc1 * cc[2]; D[nt][3] += sc1 * cc[3];
            }
        }
    }
    // zero point: sum_g sc_g * (-32 S_g) with the int8 scales themselves as the A fragment (S = a + 64 b)
    const float d0 = half_bits_to_float((uint16_t)(r.dd & 0xFFFFu)), d1 = half_bits_to_float((uint16_t)(r.dd >> 16));
    const uint32_t az0 = t == 0 ? r.s0.x : t == 1 ? r.s0.y : t == 2 ? r.s0.z : r.s0.w;  // scales 4t..4t+3 of row g
    const uint32_t az1 = t == 0 ? r.s1.x : t == 1 ? r.s1.y : t == 2 ? r.s1.z : r.s1.w;  // ... of row g+8
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int ca[4], cb[4];
        imma_k16(ca, az0, az1, b.ra16[nt], 0, 0, 0, 0);
        imma_k16(cb, az0, az1, b.rb16[nt], 0, 0, 0, 0);
        const float2 cs = b.cs[nt];
        acc[nt][0] = fmaf(cs.x * d0, (float)(D[nt][0] - 32 * (ca[0] + 64 * cb[0])), acc[nt][0]);
        acc[nt][1] = fmaf(cs.y * d0, (float)(D[nt][1] - 32 * (ca[1] + 64 * cb[1])), acc[nt][1]);
        acc[nt][2] = fmaf(cs.x * d1, (float)(D[nt][2] - 32 * (ca[2] + 64 * cb[2])), acc[nt][2]);
        acc[nt][3] = fmaf(cs.y * d1, (float)(D[nt][3] - 32 * (ca[3] + 64 * cb[3])), acc[nt][3]);
    }
}

// ── Q8_0, 8 blocks per tile, operands as for the K-quants (used by the streaming kernel) ──
struct Q8Regs {
    uint4 q[8];
    uint4 d0, d1;  // 8 f16 scales of row g / row g+8
};
template <bool GLOBAL>
__device__ __forceinline__ void load_q8_0(const uint8_t* tile, int lane, Q8Regs& r) {
    const int g = lane >> 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) r.q[j] = GLOBAL ? ldg_u4(tile + j * 512 + lane * 16) : ld_u4(tile + j * 512 + lane * 16);
    r.d0 = GLOBAL ? ldg_u4(tile + 4096 + g * 16) : ld_u4(tile + 4096 + g * 16);
    r.d1 = GLOBAL ? ldg_u4(tile + 4096 + (g + 8) * 16) : ld_u4(tile + 4096 + (g + 8) * 16);
}
template <int NT>
__device__ __forceinline__ void compute_q8_0(const Q8Regs& r, const BFrag<NT>& b, float (&acc)[NT][4]) {
    const uint32_t dw0[4] = {r.d0.x, r.d0.y, r.d0.z, r.d0.w}, dw1[4] = {r.d1.x, r.d1.y, r.d1.z, r.d1.w};
    float f[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) f[nt][e] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float d0 = half_bits_to_float((uint16_t)((dw0[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
        const float d1 = half_bits_to_float((uint16_t)((dw1[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int c[4];
            imma_k32(c, r.q[j].x, r.q[j].z, r.q[j].y, r.q[j].w, b.w[nt][2 * j], b.w[nt][2 * j + 1], 0, 0, 0, 0);
            f[nt][0] = fmaf(d0, (float)c[0], f[nt][0]); f[nt][1] = fmaf(d0, (float)c[1], f[nt][1]);
            f[nt][2] = fmaf(d1, (float)c[2], f[nt][2]); f[nt][3] = fmaf(d1, (float)c[3], f[nt][3]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        acc[nt][0] = fmaf(b.cs[nt].x, f[nt][0], acc[nt][0]); acc[nt][1] = fmaf(b.cs[nt].y, f[nt][1], acc[nt][1]);
        acc[nt][2] = fmaf(b.cs[nt].x, f[nt][2], acc[nt][2]); acc[nt][3] = fmaf(b.cs[nt].y, f[nt][3], acc[nt][3]);
    }
}

}  // namespace sp
