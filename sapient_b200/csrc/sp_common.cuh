// Shared definitions for the sm_100a kernels: ggml block geometry, f16 helpers and
// the bit-exact per-element block decoders.
//
// Block layouts (reference: crates/sapient-core/src/dtype.rs:56-69):
//   Q8_0  34 B / 32 weights : f16 d, 32 x i8
//   Q4_K 144 B / 256 weights: f16 d, f16 dmin, 12 B packed 6-bit (scale, min) x 8, 128 B nibbles
//   Q6_K 210 B / 256 weights: ql[128] low nibbles, qh[64] high 2 bits, i8 scales[16], f16 d
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sp {

enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30 };
constexpr int Q4_0_BYTES = 18;
constexpr int Q8_0_BYTES = 34;
constexpr int Q4_K_BYTES = 144;
constexpr int Q5_K_BYTES = 176;
constexpr int Q6_K_BYTES = 210;
constexpr int KV_PAGE = 16;  // tokens per KV page

__host__ __device__ inline int block_elems(int dtype) {
    return (dtype == T_Q4_K || dtype == T_Q5_K || dtype == T_Q6_K) ? 256 : ((dtype == T_Q8_0 || dtype == T_Q4_0) ? 32 : 1);
}
__host__ __device__ inline int block_bytes(int dtype) {
    switch (dtype) {
        case T_F32: return 4;
        case T_F16: case T_BF16: return 2;
        case T_Q4_0: return Q4_0_BYTES;
        case T_Q8_0: return Q8_0_BYTES;
        case T_Q4_K: return Q4_K_BYTES;
        case T_Q5_K: return Q5_K_BYTES;
        case T_Q6_K: return Q6_K_BYTES;
        default: return 0;
    }
}
// Bytes of one row of k weights (crates/sapient-core/src/dtype.rs:136-145).
__host__ __device__ inline int64_t row_bytes(int dtype, int64_t k) {
    return k / block_elems(dtype) * block_bytes(dtype);
}

__device__ __forceinline__ float half_bits_to_float(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }

// Byte j (0..11) of the Q4_K scale field held as three little-endian words.
__device__ __forceinline__ uint32_t k4_byte(uint32_t s0, uint32_t s1, uint32_t s2, int j) {
    const uint32_t w = j < 4 ? s0 : (j < 8 ? s1 : s2);
    return (w >> (8 * (j & 3))) & 0xFFu;
}
// 6-bit (scale, min) of sub-block j (crates/sapient-core/src/tensor.rs:567-576).
__device__ __forceinline__ void k4_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, uint32_t* sc, uint32_t* mn) {
    if (j < 4) {
        *sc = k4_byte(s0, s1, s2, j) & 63u;
        *mn = k4_byte(s0, s1, s2, j + 4) & 63u;
    } else {
        *sc = (k4_byte(s0, s1, s2, j + 4) & 0xFu) | ((k4_byte(s0, s1, s2, j - 4) >> 6) << 4);
        *mn = (k4_byte(s0, s1, s2, j + 4) >> 4) | ((k4_byte(s0, s1, s2, j) >> 6) << 4);
    }
}

// ── Bit-exact element decoders ───────────────────────────────────────────────
// Every product and the subtraction are rounded separately (__fmul_rn/__fsub_rn:
// never contracted to FMA) so the value equals the reference's dequantisation bit
// for bit (crates/sapient-core/src/tensor.rs:378-389,504-565).

__device__ __forceinline__ float dequant_q8_0_elem(const uint8_t* row, int64_t i) {
    const uint8_t* blk = row + (i >> 5) * Q8_0_BYTES;
    const float d = half_bits_to_float(ld_u16(blk));
    return __fmul_rn((float)(int8_t)blk[2 + (i & 31)], d);
}

__device__ __forceinline__ float dequant_q4_k_elem(const uint8_t* row, int64_t i) {
    const uint8_t* blk = row + (i >> 8) * Q4_K_BYTES;
    const int r = (int)(i & 255);
    const int g = r >> 6, hi = (r >> 5) & 1, l = r & 31;
    const float d = half_bits_to_float(ld_u16(blk));
    const float dmin = half_bits_to_float(ld_u16(blk + 2));
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(blk + 4);
    uint32_t sc, mn;
    k4_scale_min(s32[0], s32[1], s32[2], 2 * g + hi, &sc, &mn);
    const float dl = __fmul_rn(d, (float)sc);
    const float ml = __fmul_rn(dmin, (float)mn);
    const uint8_t qb = blk[16 + 32 * g + l];
    const float q = (float)(hi ? (qb >> 4) : (qb & 0x0F));
    return __fsub_rn(__fmul_rn(dl, q), ml);
}

// Q4_0 (crates/sapient-core/src/tensor.rs:362-377): 18 bytes per 32 weights = f16 d + 16 nibble bytes; elements 0..15
// are the low nibbles, 16..31 the high nibbles, value (q - 8) * d.
__device__ __forceinline__ float dequant_q4_0_elem(const uint8_t* row, int64_t i) {
    const uint8_t* blk = row + (i >> 5) * Q4_0_BYTES;
    const int j = (int)(i & 31);
    const float d = half_bits_to_float(ld_u16(blk));
    const uint8_t b = blk[2 + (j & 15)];
    const int q = (int)(j < 16 ? (b & 0x0F) : (b >> 4)) - 8;
    return __fmul_rn((float)q, d);
}

// Q5_K (crates/sapient-core/src/tensor.rs:421-467): 176 bytes per 256 weights = f16 d, f16 dmin, scales[12] (the Q4_K
// 6-bit packing), qh[32], qs[128]. Per 64-group g: low nibbles of qs[32 g + l] are sub-block 2 g, high nibbles 2 g + 1;
// the fifth bit of element l is PER ELEMENT, bit (2 g) resp. (2 g + 1) of qh[l]. Value d * sc * (q + 16 * bit) - dmin * m.
__device__ __forceinline__ float dequant_q5_k_elem(const uint8_t* row, int64_t i) {
    const uint8_t* blk = row + (i >> 8) * Q5_K_BYTES;
    const int r = (int)(i & 255);
    const int g = r >> 6, hi = (r >> 5) & 1, l = r & 31;
    const float d = half_bits_to_float(ld_u16(blk));
    const float dmin = half_bits_to_float(ld_u16(blk + 2));
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(blk + 4);
    uint32_t sc, mn;
    k4_scale_min(s32[0], s32[1], s32[2], 2 * g + hi, &sc, &mn);
    const float dl = __fmul_rn(d, (float)sc);
    const float ml = __fmul_rn(dmin, (float)mn);
    const uint8_t qb = blk[48 + 32 * g + l];
    const float fifth = ((blk[16 + l] >> (2 * g + hi)) & 1u) ? 16.0f : 0.0f;
    const float q = __fadd_rn((float)(hi ? (qb >> 4) : (qb & 0x0F)), fifth);
    return __fsub_rn(__fmul_rn(dl, q), ml);
}

__device__ __forceinline__ float dequant_q6_k_elem(const uint8_t* row, int64_t i) {
    const uint8_t* blk = row + (i >> 8) * Q6_K_BYTES;
    const int r = (int)(i & 255);
    const int half = r >> 7, quarter = (r >> 5) & 3, l = r & 31;
    const uint8_t qlb = blk[64 * half + l + ((quarter & 1) ? 32 : 0)];
    const uint32_t nib = (quarter >= 2) ? (qlb >> 4) : (qlb & 0x0F);
    const uint32_t hb = (blk[128 + 32 * half + l] >> (2 * quarter)) & 3u;
    const float q = (float)((int)(nib | (hb << 4)) - 32);
    const float sc = (float)(int8_t)blk[192 + 8 * half + (l >> 4) + 2 * quarter];
    const float d = half_bits_to_float(ld_u16(blk + 208));
    return __fmul_rn(__fmul_rn(d, sc), q);
}

__device__ __forceinline__ float dequant_elem(int dtype, const uint8_t* row, int64_t i) {
    switch (dtype) {
        case T_Q4_K: return dequant_q4_k_elem(row, i);
        case T_Q5_K: return dequant_q5_k_elem(row, i);
        case T_Q6_K: return dequant_q6_k_elem(row, i);
        case T_Q4_0: return dequant_q4_0_elem(row, i);
        case T_Q8_0: return dequant_q8_0_elem(row, i);
        case T_F16: return half_bits_to_float(ld_u16(row + 2 * i));
        case T_BF16: return __uint_as_float((uint32_t)ld_u16(row + 2 * i) << 16);
        default: return reinterpret_cast<const float*>(row)[i];
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

}  // namespace sp
