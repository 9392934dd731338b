// sapient_oracle.cpp — CPU restatement of the reference's x86_64 CPU path for
// quantized-GGUF decoder inference.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test-suite, the smoke
// check and the benchmark's CPU-baseline leg may load it; the CUDA library never
// links, imports or calls anything in this file.
//
// Every function follows the arithmetic of the reference (sapient v0.6.0, Rust)
// operation by operation: same operand order, same rounding points (no FMA
// contraction unless the reference uses an explicit fused instruction), same
// sequential accumulation order. Build with -O2 -ffp-contract=off (never
// -ffast-math). Citations give the reference file (path within its repository)
// and lines that each function restates.
//
// Parity status: pinned. The restatement reproduces the reference's own
// known-answer tests (Q6_K canonical block dot = 1920, RMSNorm/LayerNorm/RoPE/
// attention/KV-append/unpermute spot values) and is bit-identical to the
// independent numpy `gguf.quants.dequantize` on random-bit blocks; see
// tests/test_oracle_kat.py.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <vector>

#if defined(_OPENMP)
#include <immintrin.h>
#include <omp.h>
#endif

namespace {

// ggml type codes (crates/sapient-io/src/gguf.rs:88-129).
enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30 };

// Block sizes (crates/sapient-core/src/dtype.rs:56-69).
constexpr int QK = 32;
constexpr int QK_K = 256;
constexpr int Q4_0_BYTES = 18;
constexpr int Q8_0_BYTES = 34;
constexpr int Q4_K_BYTES = 144;
constexpr int Q5_K_BYTES = 176;
constexpr int Q6_K_BYTES = 210;

// ── IEEE half conversions (the `half` crate: to_f32 exact, from_f32 RNE) ─────
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? (0x200u | ((absx >> 13) & 0x3FFu)) : 0u));
    }
    if (absx >= 0x477FF000u) {  // rounds to >= 65520 → inf
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) {  // < 2^-25 (or exactly 2^-25 → ties to even 0)
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t hexp;
    if (e < -14) {  // subnormal half
        shift = (uint32_t)(13 + (-14 - e));
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    uint32_t out;
    if (hexp == 0) {
        out = q;  // may carry into exponent 1, which is the right encoding
    } else {
        out = ((hexp - 1) << 10) + q;  // q includes the implicit bit (0x400)
    }
    return (uint16_t)(sign | out);
}

inline float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// Rust f32::round — half away from zero.
inline float rust_round(float v) { return std::round(v); }

// crates/sapient-core/src/tensor.rs:567-576 / kernels/quant.rs:596-605.
inline void get_scale_min_k4(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// ── Dequantisation (crates/sapient-core/src/tensor.rs:341-576) ───────────────

// tensor.rs:504-527
void dequant_q4_k_block(const uint8_t* block, float* out) {
    const float d = f16_to_f32(rd16(block));
    const float dmin = f16_to_f32(rd16(block + 2));
    const uint8_t* scales = block + 4;
    const uint8_t* qs = block + 16;
    int out_idx = 0, q_off = 0, is = 0;
    for (int g = 0; g < QK_K / 64; ++g) {
        uint8_t sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        const float d1 = d * (float)sc1;
        const float m1v = dmin * (float)m1;
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d2 = d * (float)sc2;
        const float m2v = dmin * (float)m2;
        for (int l = 0; l < 32; ++l) {
            out[out_idx + l] = d1 * (float)(qs[q_off + l] & 0x0F) - m1v;
            out[out_idx + l + 32] = d2 * (float)(qs[q_off + l] >> 4) - m2v;
        }
        out_idx += 64;
        q_off += 32;
        is += 2;
    }
}

// tensor.rs:421-467 (format adjacent to the hot path; kept for the KAT).
void dequant_q5_k_block(const uint8_t* block, float* out) {
    const float d = f16_to_f32(rd16(block));
    const float dmin = f16_to_f32(rd16(block + 2));
    const uint8_t* scales = block + 4;
    const uint8_t* qh = block + 16;
    const uint8_t* ql = block + 48;
    int ql_off = 0, is = 0, out_idx = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int g = 0; g < QK_K / 64; ++g) {
        uint8_t sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        const float d1 = d * (float)sc1;
        const float m1v = dmin * (float)m1;
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d2 = d * (float)sc2;
        const float m2v = dmin * (float)m2;
        for (int l = 0; l < 32; ++l) {
            const float hi = (qh[l] & u1) ? 16.0f : 0.0f;
            out[out_idx + l] = d1 * ((float)(ql[ql_off + l] & 0x0F) + hi) - m1v;
            const float hi2 = (qh[l] & u2) ? 16.0f : 0.0f;
            out[out_idx + l + 32] = d2 * ((float)(ql[ql_off + l] >> 4) + hi2) - m2v;
        }
        out_idx += 64;
        ql_off += 32;
        is += 2;
        if (is % 8 == 0) { u1 = 1; u2 = 2; } else { u1 <<= 2; u2 <<= 2; }
    }
}

// tensor.rs:534-565
void dequant_q6_k_block(const uint8_t* block, float* out) {
    const uint8_t* ql = block;
    const uint8_t* qh = block + 128;
    const int8_t* sc = (const int8_t*)(block + 192);
    const float d = f16_to_f32(rd16(block + 208));
    int out_idx = 0, ql_off = 0, qh_off = 0, sc_base = 0;
    for (int half = 0; half < QK_K / 128; ++half) {
        for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const float q1 = (float)((int)((ql[ql_off + l] & 0x0F) | ((qh[qh_off + l] & 3) << 4)) - 32);
            const float q2 = (float)((int)((ql[ql_off + l + 32] & 0x0F) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32);
            const float q3 = (float)((int)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32);
            const float q4 = (float)((int)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32);
            out[out_idx + l] = d * (float)sc[sc_base + is] * q1;
            out[out_idx + l + 32] = d * (float)sc[sc_base + is + 2] * q2;
            out[out_idx + l + 64] = d * (float)sc[sc_base + is + 4] * q3;
            out[out_idx + l + 96] = d * (float)sc[sc_base + is + 6] * q4;
        }
        out_idx += 128;
        ql_off += 64;
        qh_off += 32;
        sc_base += 8;
    }
}

int64_t block_elems(int dtype) {
    switch (dtype) {
        case T_Q4_0: case T_Q8_0: return QK;
        case T_Q4_K: case T_Q5_K: case T_Q6_K: return QK_K;
        default: return 1;
    }
}
int64_t block_bytes(int dtype) {
    switch (dtype) {
        case T_F32: return 4;
        case T_F16: case T_BF16: return 2;
        case T_Q4_0: return Q4_0_BYTES;
        case T_Q8_0: return Q8_0_BYTES;
        case T_Q4_K: return Q4_K_BYTES;
        case T_Q5_K: return Q5_K_BYTES;
        case T_Q6_K: return Q6_K_BYTES;
        default: return -1;
    }
}
// crates/sapient-core/src/dtype.rs:136-145
int64_t byte_count(int dtype, int64_t numel) {
    int64_t be = block_elems(dtype), bb = block_bytes(dtype);
    if (bb < 0) return -1;
    return numel / be * bb;
}

// tensor.rs:341-498 (arms used by GGUF decoder models).
int dequant_any(int dtype, const uint8_t* bytes, int64_t numel, float* out) {
    switch (dtype) {
        case T_F32:
            std::memcpy(out, bytes, (size_t)numel * 4);
            return 0;
        case T_F16:
            for (int64_t i = 0; i < numel; ++i) out[i] = f16_to_f32(rd16(bytes + 2 * i));
            return 0;
        case T_BF16:
            for (int64_t i = 0; i < numel; ++i) out[i] = bf16_to_f32(rd16(bytes + 2 * i));
            return 0;
        case T_Q4_0:  // tensor.rs:362-377
            for (int64_t b = 0; b < numel / QK; ++b) {
                const uint8_t* blk = bytes + b * Q4_0_BYTES;
                const float d = f16_to_f32(rd16(blk));
                for (int j = 0; j < QK / 2; ++j) {
                    const int lo = (int)(blk[2 + j] & 0x0F) - 8;
                    const int hi = (int)(blk[2 + j] >> 4) - 8;
                    out[b * QK + j] = (float)lo * d;
                    out[b * QK + j + QK / 2] = (float)hi * d;
                }
            }
            return 0;
        case T_Q8_0:  // tensor.rs:378-389
            for (int64_t b = 0; b < numel / QK; ++b) {
                const uint8_t* blk = bytes + b * Q8_0_BYTES;
                const float d = f16_to_f32(rd16(blk));
                for (int j = 0; j < QK; ++j) out[b * QK + j] = (float)(int8_t)blk[2 + j] * d;
            }
            return 0;
        case T_Q4_K:
            for (int64_t b = 0; b < numel / QK_K; ++b) dequant_q4_k_block(bytes + b * Q4_K_BYTES, out + b * QK_K);
            return 0;
        case T_Q5_K:
            for (int64_t b = 0; b < numel / QK_K; ++b) dequant_q5_k_block(bytes + b * Q5_K_BYTES, out + b * QK_K);
            return 0;
        case T_Q6_K:
            for (int64_t b = 0; b < numel / QK_K; ++b) dequant_q6_k_block(bytes + b * Q6_K_BYTES, out + b * QK_K);
            return 0;
        default:
            return -2;
    }
}

// ── Q8_0 quantiser (kernels/quant.rs:223-235; forward/common.rs:336-348) ─────
void quantize_q8_0_block(const float* x, uint8_t* out) {
    float max_abs = 0.0f;
    for (int i = 0; i < QK; ++i) max_abs = std::fmax(max_abs, std::fabs(x[i]));
    const float scale = max_abs / 127.0f;
    const uint16_t d = f32_to_f16(scale);
    const float inv_scale = scale > 0.0f ? 1.0f / scale : 0.0f;
    out[0] = (uint8_t)(d & 0xFF);
    out[1] = (uint8_t)(d >> 8);
    for (int i = 0; i < QK; ++i) {
        float r = rust_round(x[i] * inv_scale);
        r = std::fmin(std::fmax(r, -127.0f), 127.0f);
        out[2 + i] = (uint8_t)(int8_t)r;
    }
}

// ── Row dot products (x86_64 paths) ─────────────────────────────────────────

// kernels/quant.rs:625-652 — one sequential f32 accumulator, dequant-then-multiply.
float dot_q4_k_row_f32(const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    int64_t x_off = 0;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const uint8_t* block = row + b * Q4_K_BYTES;
        const float d = f16_to_f32(rd16(block));
        const float dmin = f16_to_f32(rd16(block + 2));
        const uint8_t* scales = block + 4;
        const uint8_t* qs = block + 16;
        int q_off = 0, is = 0;
        for (int g = 0; g < QK_K / 64; ++g) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            const float d1 = d * (float)sc1;
            const float m1v = dmin * (float)m1;
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            const float d2 = d * (float)sc2;
            const float m2v = dmin * (float)m2;
            for (int l = 0; l < 32; ++l) {
                acc += (d1 * (float)(qs[q_off + l] & 0x0F) - m1v) * x[x_off + l];
                acc += (d2 * (float)(qs[q_off + l] >> 4) - m2v) * x[x_off + l + 32];
            }
            x_off += 64;
            q_off += 32;
            is += 2;
        }
    }
    return acc;
}

// kernels/quant.rs:104-114,197-205 — Q4_0: per block (lo * x[j] + hi * x[j + 16]) summed, times d; blocks added in order.
float dot_q4_0_row_f32(const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    for (int64_t b = 0; b < k / QK; ++b) {
        const uint8_t* block = row + b * Q4_0_BYTES;
        const float d = f16_to_f32(rd16(block));
        float bacc = 0.0f;
        for (int j = 0; j < QK / 2; ++j) {
            const int lo = (int)(block[2 + j] & 0x0F) - 8;
            const int hi = (int)(block[2 + j] >> 4) - 8;
            bacc += (float)lo * x[b * QK + j] + (float)hi * x[b * QK + j + QK / 2];
        }
        acc += bacc * d;
    }
    return acc;
}

// kernels/quant.rs:1626-1665 — Q5_K scalar row dot (the fifth bit is per element: bit planes of qh[l]).
float dot_q5_k_row_f32(const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    int64_t x_off = 0;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const uint8_t* block = row + b * Q5_K_BYTES;
        const float d = f16_to_f32(rd16(block));
        const float dmin = f16_to_f32(rd16(block + 2));
        const uint8_t* scales = block + 4;
        const uint8_t* qh = block + 16;
        const uint8_t* ql = block + 48;
        int ql_off = 0, is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int g = 0; g < QK_K / 64; ++g) {
            uint8_t sc1, m1, sc2, m2;
            get_scale_min_k4(is, scales, &sc1, &m1);
            const float d1 = d * (float)sc1;
            const float m1v = dmin * (float)m1;
            get_scale_min_k4(is + 1, scales, &sc2, &m2);
            const float d2 = d * (float)sc2;
            const float m2v = dmin * (float)m2;
            for (int l = 0; l < 32; ++l) {
                const float hi1 = (qh[l] & u1) ? 16.0f : 0.0f;
                const float hi2 = (qh[l] & u2) ? 16.0f : 0.0f;
                acc += (d1 * ((float)(ql[ql_off + l] & 0x0F) + hi1) - m1v) * x[x_off + l];
                acc += (d2 * ((float)(ql[ql_off + l] >> 4) + hi2) - m2v) * x[x_off + l + 32];
            }
            x_off += 64;
            ql_off += 32;
            is += 2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
    return acc;
}

// kernels/quant.rs:2573-2613
float dot_q6_k_row_f32(const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    int64_t x_off = 0;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const uint8_t* block = row + b * Q6_K_BYTES;
        const uint8_t* ql = block;
        const uint8_t* qh = block + 128;
        const int8_t* sc = (const int8_t*)(block + 192);
        const float d = f16_to_f32(rd16(block + 208));
        int ql_off = 0, qh_off = 0, sc_base = 0;
        for (int half = 0; half < QK_K / 128; ++half) {
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const float q1 = (float)((int)((ql[ql_off + l] & 0x0F) | ((qh[qh_off + l] & 3) << 4)) - 32);
                const float q2 = (float)((int)((ql[ql_off + l + 32] & 0x0F) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32);
                const float q3 = (float)((int)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32);
                const float q4 = (float)((int)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32);
                acc += d * (float)sc[sc_base + is] * q1 * x[x_off + l];
                acc += d * (float)sc[sc_base + is + 2] * q2 * x[x_off + l + 32];
                acc += d * (float)sc[sc_base + is + 4] * q3 * x[x_off + l + 64];
                acc += d * (float)sc[sc_base + is + 6] * q4 * x[x_off + l + 96];
            }
            x_off += 128;
            ql_off += 64;
            qh_off += 32;
            sc_base += 8;
        }
    }
    return acc;
}

// kernels/quant.rs:543-580 — the AVX2+FMA row dot, restated lane by lane.
// Each 4-byte load is widened into the LOW four lanes of a 256-bit register
// (upper lanes zero), so only lanes 0..3 ever carry data: lane j accumulates,
// with fused multiply-adds, elements j, 4+j, 8+j, … of the block in index order;
// the row accumulator is fma(block_acc, scale, row_acc) per lane; the final
// horizontal sum is (l0+l1)+(l2+l3).
float dot_q8_0_row_f32_avx2(const uint8_t* row, const float* x, int64_t k) {
    float row_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int64_t b = 0; b < k / QK; ++b) {
        const uint8_t* block = row + b * Q8_0_BYTES;
        const float scale = f16_to_f32(rd16(block));
        const int8_t* q = (const int8_t*)(block + 2);
        const float* xp = x + b * QK;
        float block_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int g = 0; g < 4; ++g) {
            for (int j = 0; j < 4; ++j) block_acc[j] = std::fmaf((float)q[8 * g + j], xp[8 * g + j], block_acc[j]);
            for (int j = 0; j < 4; ++j) block_acc[j] = std::fmaf((float)q[8 * g + 4 + j], xp[8 * g + 4 + j], block_acc[j]);
        }
        for (int j = 0; j < 4; ++j) row_acc[j] = std::fmaf(block_acc[j], scale, row_acc[j]);
    }
    // lo + hi (hi lanes are zero), then movehdup/add, movehl/add.
    const float s0 = row_acc[0] + 0.0f, s1 = row_acc[1] + 0.0f, s2 = row_acc[2] + 0.0f, s3 = row_acc[3] + 0.0f;
    return (s0 + s1) + (s2 + s3);
}

// kernels/quant.rs:253-260,528-534 — the portable (non-AVX2) row dot.
float dot_q8_0_row_f32_scalar(const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    for (int64_t b = 0; b < k / QK; ++b) {
        const uint8_t* block = row + b * Q8_0_BYTES;
        const float d = f16_to_f32(rd16(block));
        float bacc = 0.0f;
        for (int j = 0; j < QK; ++j) bacc += (float)(int8_t)block[2 + j] * x[b * QK + j];
        acc += bacc * d;
    }
    return acc;
}

// ── The same row dots, R rows at a time ─────────────────────────────────────
// Pure speed-up of the checker: every row keeps its own accumulator and sees exactly the operations of the
// single-row functions above, in the same order (nothing is contracted or reassociated: -ffp-contract=off, no
// fast-math), so the results are bit-identical; the R independent dependency chains merely overlap in the pipeline
// instead of each waiting for its own previous add. tests/test_oracle_kat.py compares the two paths bit for bit.
constexpr int ROWS_R = 8;

// Lanes of a 256-bit register = 8 consecutive weight rows; every lane runs the scalar sequence (separate multiply,
// subtract, multiply, add: no fused operations).
void dot_q4_k_rows(const uint8_t* rows, int64_t row_bytes, const float* x, int64_t k, float* out) {
    __m256 acc = _mm256_setzero_ps();
    int64_t x_off = 0;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const uint8_t* block[ROWS_R];
        alignas(32) float d[ROWS_R], dmin[ROWS_R];
        for (int r = 0; r < ROWS_R; ++r) {
            block[r] = rows + r * row_bytes + b * Q4_K_BYTES;
            d[r] = f16_to_f32(rd16(block[r]));
            dmin[r] = f16_to_f32(rd16(block[r] + 2));
        }
        int q_off = 0, is = 0;
        for (int g = 0; g < QK_K / 64; ++g) {
            alignas(32) float d1[ROWS_R], m1v[ROWS_R], d2[ROWS_R], m2v[ROWS_R];
            for (int r = 0; r < ROWS_R; ++r) {
                uint8_t sc1, m1, sc2, m2;
                get_scale_min_k4(is, block[r] + 4, &sc1, &m1);
                d1[r] = d[r] * (float)sc1;
                m1v[r] = dmin[r] * (float)m1;
                get_scale_min_k4(is + 1, block[r] + 4, &sc2, &m2);
                d2[r] = d[r] * (float)sc2;
                m2v[r] = dmin[r] * (float)m2;
            }
            const __m256 vd1 = _mm256_load_ps(d1), vm1 = _mm256_load_ps(m1v), vd2 = _mm256_load_ps(d2), vm2 = _mm256_load_ps(m2v);
            for (int l = 0; l < 32; ++l) {
                const __m256i q = _mm256_setr_epi32(block[0][16 + q_off + l], block[1][16 + q_off + l], block[2][16 + q_off + l],
                                                    block[3][16 + q_off + l], block[4][16 + q_off + l], block[5][16 + q_off + l],
                                                    block[6][16 + q_off + l], block[7][16 + q_off + l]);
                const __m256 lo = _mm256_cvtepi32_ps(_mm256_and_si256(q, _mm256_set1_epi32(0x0F)));
                const __m256 hi = _mm256_cvtepi32_ps(_mm256_srli_epi32(q, 4));
                const __m256 xa = _mm256_set1_ps(x[x_off + l]), xb = _mm256_set1_ps(x[x_off + l + 32]);
                acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_sub_ps(_mm256_mul_ps(vd1, lo), vm1), xa));
                acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_sub_ps(_mm256_mul_ps(vd2, hi), vm2), xb));
            }
            x_off += 64;
            q_off += 32;
            is += 2;
        }
    }
    _mm256_storeu_ps(out, acc);
}

void dot_q6_k_rows(const uint8_t* rows, int64_t row_bytes, const float* x, int64_t k, float* out) {
    __m256 acc = _mm256_setzero_ps();
    int64_t x_off = 0;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const uint8_t* block[ROWS_R];
        alignas(32) float d[ROWS_R];
        for (int r = 0; r < ROWS_R; ++r) {
            block[r] = rows + r * row_bytes + b * Q6_K_BYTES;
            d[r] = f16_to_f32(rd16(block[r] + 208));
        }
        const __m256 vd = _mm256_load_ps(d);
        int ql_off = 0, qh_off = 0, sc_base = 0;
        for (int half = 0; half < QK_K / 128; ++half) {
            for (int is = 0; is < 2; ++is) {
                // d * sc for the four 16-wide scale groups this run of l uses (the product the scalar code forms first)
                __m256 ds[4];
                for (int q = 0; q < 4; ++q) {
                    alignas(32) float t[ROWS_R];
                    for (int r = 0; r < ROWS_R; ++r) t[r] = (float)(int8_t)block[r][192 + sc_base + is + 2 * q];
                    ds[q] = _mm256_mul_ps(vd, _mm256_load_ps(t));
                }
                for (int l = 16 * is; l < 16 * is + 16; ++l) {
                    __m256i la, lb, h;
                    {
                        const int oa = ql_off + l, ob = ql_off + l + 32, oh = 128 + qh_off + l;
                        la = _mm256_setr_epi32(block[0][oa], block[1][oa], block[2][oa], block[3][oa], block[4][oa], block[5][oa], block[6][oa], block[7][oa]);
                        lb = _mm256_setr_epi32(block[0][ob], block[1][ob], block[2][ob], block[3][ob], block[4][ob], block[5][ob], block[6][ob], block[7][ob]);
                        h = _mm256_setr_epi32(block[0][oh], block[1][oh], block[2][oh], block[3][oh], block[4][oh], block[5][oh], block[6][oh], block[7][oh]);
                    }
                    const __m256i m4 = _mm256_set1_epi32(0x0F), m2 = _mm256_set1_epi32(3), off = _mm256_set1_epi32(32);
                    const __m256i i1 = _mm256_sub_epi32(_mm256_or_si256(_mm256_and_si256(la, m4), _mm256_slli_epi32(_mm256_and_si256(h, m2), 4)), off);
                    const __m256i i2 = _mm256_sub_epi32(_mm256_or_si256(_mm256_and_si256(lb, m4), _mm256_slli_epi32(_mm256_and_si256(_mm256_srli_epi32(h, 2), m2), 4)), off);
                    const __m256i i3 = _mm256_sub_epi32(_mm256_or_si256(_mm256_srli_epi32(la, 4), _mm256_slli_epi32(_mm256_and_si256(_mm256_srli_epi32(h, 4), m2), 4)), off);
                    const __m256i i4 = _mm256_sub_epi32(_mm256_or_si256(_mm256_srli_epi32(lb, 4), _mm256_slli_epi32(_mm256_and_si256(_mm256_srli_epi32(h, 6), m2), 4)), off);
                    acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_mul_ps(ds[0], _mm256_cvtepi32_ps(i1)), _mm256_set1_ps(x[x_off + l])));
                    acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_mul_ps(ds[1], _mm256_cvtepi32_ps(i2)), _mm256_set1_ps(x[x_off + l + 32])));
                    acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_mul_ps(ds[2], _mm256_cvtepi32_ps(i3)), _mm256_set1_ps(x[x_off + l + 64])));
                    acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_mul_ps(ds[3], _mm256_cvtepi32_ps(i4)), _mm256_set1_ps(x[x_off + l + 96])));
                }
            }
            x_off += 128;
            ql_off += 64;
            qh_off += 32;
            sc_base += 8;
        }
    }
    _mm256_storeu_ps(out, acc);
}

int g_q8_mode = 0;  // 0 = AVX2+FMA order (what x86_64 CI runs), 1 = portable scalar order
// 0 = the reference's order: one running f32 accumulator per output over the whole row. 1 = a second valid evaluation
// order of the same products, for measuring how far two correct implementations drift apart: the sum of each
// 256-element super-block is formed first and then added to the row total.
int g_kquant_order = 0;
int g_rows_at_once = 0;  // 1: matmul_nt walks K-quant rows ROWS_R at a time (tests; a timing run keeps the reference's one-row-per-call loop)

float dot_kquant_row_blocked(int dtype, const uint8_t* row, const float* x, int64_t k) {
    float acc = 0.0f;
    const int64_t bb = dtype == T_Q4_K ? Q4_K_BYTES : Q6_K_BYTES;
    for (int64_t b = 0; b < k / QK_K; ++b) {
        const float part = dtype == T_Q4_K ? dot_q4_k_row_f32(row + b * bb, x + b * QK_K, QK_K) : dot_q6_k_row_f32(row + b * bb, x + b * QK_K, QK_K);
        acc += part;
    }
    return acc;
}

float dot_row(int dtype, const uint8_t* row, const float* x, int64_t k) {
    if (g_kquant_order == 1 && (dtype == T_Q4_K || dtype == T_Q6_K)) return dot_kquant_row_blocked(dtype, row, x, k);
    switch (dtype) {
        case T_Q4_K: return dot_q4_k_row_f32(row, x, k);
        case T_Q6_K: return dot_q6_k_row_f32(row, x, k);
        case T_Q4_0: return dot_q4_0_row_f32(row, x, k);
        case T_Q5_K: return dot_q5_k_row_f32(row, x, k);
        case T_Q8_0: return g_q8_mode == 0 ? dot_q8_0_row_f32_avx2(row, x, k) : dot_q8_0_row_f32_scalar(row, x, k);
        default: return std::numeric_limits<float>::quiet_NaN();
    }
}

// ── matmul_nt (kernels/matmul.rs:114-145,575-689,862-943,1111-1167) ──────────
// Y[M,N] = X[M,K] · Wᵀ. For M > 1 the x86 path runs M independent GEMVs; every
// output element is one call of the row dot, so threading over output rows cannot
// change any result.
// Status: 0 ok, 1 = k not a multiple of the block size (SapientError::Internal),
// 2 = unsupported dtype.
int matmul_nt(int dtype, const float* x, const uint8_t* w, int64_t m, int64_t k, int64_t n, float* y) {
    if (dtype == T_Q4_K || dtype == T_Q5_K || dtype == T_Q6_K) {
        if (k % 256 != 0) return 1;
    } else if (dtype == T_Q8_0 || dtype == T_Q4_0) {
        if (k % 32 != 0) return 1;
    } else if (dtype == T_F32 || dtype == T_F16 || dtype == T_BF16) {
        // Float weights are not reached by the quantised configurations; a plain
        // sequential dot stands in for the reference's SGEMM (summation order of
        // that third-party routine is not restated).
        std::vector<float> wf((size_t)(n * k));
        dequant_any(dtype, w, n * k, wf.data());
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < n; ++j)
            for (int64_t i = 0; i < m; ++i) {
                float acc = 0.0f;
                for (int64_t t = 0; t < k; ++t) acc += x[i * k + t] * wf[(size_t)(j * k + t)];
                y[i * n + j] = acc;
            }
        return 0;
    } else {
        return 2;
    }
    const int64_t row_bytes = byte_count(dtype, k);
    if ((dtype == T_Q4_K || dtype == T_Q6_K) && g_kquant_order == 0 && g_rows_at_once) {
        // ROWS_R output rows at a time (bit-identical to the loop below, see dot_q4_k_rows)
        const int64_t groups = n / ROWS_R;
#pragma omp parallel for schedule(static)
        for (int64_t gidx = 0; gidx < groups; ++gidx) {
            const int64_t j = gidx * ROWS_R;
            float o[ROWS_R];
            for (int64_t i = 0; i < m; ++i) {
                if (dtype == T_Q4_K) dot_q4_k_rows(w + j * row_bytes, row_bytes, x + i * k, k, o);
                else dot_q6_k_rows(w + j * row_bytes, row_bytes, x + i * k, k, o);
                for (int r = 0; r < ROWS_R; ++r) y[i * n + j + r] = o[r];
            }
        }
        for (int64_t j = groups * ROWS_R; j < n; ++j)
            for (int64_t i = 0; i < m; ++i) y[i * n + j] = dot_row(dtype, w + j * row_bytes, x + i * k, k);
        return 0;
    }
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        const uint8_t* row = w + j * row_bytes;
        for (int64_t i = 0; i < m; ++i) y[i * n + j] = dot_row(dtype, row, x + i * k, k);
    }
    return 0;
}

// ── Norms (kernels/layernorm.rs:17-105) ──────────────────────────────────────
void rms_norm(const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y) {
    for (int64_t o = 0; o < rows; ++o) {
        const float* s = x + o * dim;
        float sum = 0.0f;
        for (int64_t i = 0; i < dim; ++i) sum += s[i] * s[i];
        const float rms_sq = sum / (float)dim;
        const float inv_rms = 1.0f / std::sqrt(rms_sq + eps);
        for (int64_t i = 0; i < dim; ++i) y[o * dim + i] = s[i] * inv_rms * (w ? w[i] : 1.0f);
    }
}

void layer_norm(const float* x, const float* w, const float* b, int64_t rows, int64_t dim, float eps, float* y) {
    for (int64_t o = 0; o < rows; ++o) {
        const float* s = x + o * dim;
        float sum = 0.0f;
        for (int64_t i = 0; i < dim; ++i) sum += s[i];
        const float mean = sum / (float)dim;
        float vs = 0.0f;
        for (int64_t i = 0; i < dim; ++i) vs += (s[i] - mean) * (s[i] - mean);
        const float var = vs / (float)dim;
        const float inv_std = 1.0f / std::sqrt(var + eps);
        for (int64_t i = 0; i < dim; ++i) {
            const float normed = (s[i] - mean) * inv_std;
            float v;
            if (w && b) v = normed * w[i] + b[i];
            else if (w) v = normed * w[i];
            else if (b) v = normed + b[i];
            else v = normed;
            y[o * dim + i] = v;
        }
    }
}

// ── RoPE (kernels/rope.rs:18-136), layout [n_heads, seq, head_dim] ───────────
void rope(const float* x, int64_t n_heads, int64_t seq, int64_t head_dim, const int64_t* positions, float base,
          int64_t rotary_dim, float* out) {
    std::memcpy(out, x, (size_t)(n_heads * seq * head_dim) * 4);
    const int64_t half = rotary_dim / 2;
    for (int64_t h = 0; h < n_heads; ++h)
        for (int64_t s = 0; s < seq; ++s) {
            const int64_t base_idx = (h * seq + s) * head_dim;
            const float pos = (float)positions[s];
            for (int64_t i = 0; i < half; ++i) {
                const float freq = (pos / 1.0f) / std::pow(base, 2.0f * (float)i / (float)rotary_dim);
                const float sin_f = std::sin(freq), cos_f = std::cos(freq);
                const float x0 = x[base_idx + i], x1 = x[base_idx + i + half];
                out[base_idx + i] = x0 * cos_f - x1 * sin_f;
                out[base_idx + i + half] = x1 * cos_f + x0 * sin_f;
            }
        }
}

// ── Attention (kernels/attention.rs:98-305; forward/common.rs:595-617) ───────
// q [H, sq, hd]; k, v [Hkv, sk, hd]; mask [sq, sk] additive or null.
// With mask == null the built-in causal rule attends keys 0..=qi+(sk-sq).
void attention(const float* q, const float* k, const float* v, int64_t H, int64_t Hkv, int64_t sq, int64_t sk,
               int64_t hd, const float* mask, float* out) {
    const float scale = 1.0f / std::sqrt((float)hd);
    const int64_t kv_rep = H / Hkv;
    const int64_t kv_offset = sk > sq ? sk - sq : 0;
#pragma omp parallel for schedule(dynamic)
    for (int64_t h = 0; h < H; ++h) {
        const int64_t kv_h = h / kv_rep;
        const float* k_head = k + kv_h * sk * hd;
        const float* v_head = v + kv_h * sk * hd;
        for (int64_t qi = 0; qi < sq; ++qi) {
            const float* q_row = q + (h * sq + qi) * hd;
            float* o_row = out + (h * sq + qi) * hd;
            const int64_t attend_len = mask ? sk : std::min(qi + kv_offset + 1, sk);
            const float* mask_row = mask ? mask + qi * sk : nullptr;
            float m = -std::numeric_limits<float>::infinity();
            float l = 0.0f;
            for (int64_t d = 0; d < hd; ++d) o_row[d] = 0.0f;
            for (int64_t ki = 0; ki < attend_len; ++ki) {
                const float* k_row = k_head + ki * hd;
                float dot = 0.0f;
                for (int64_t d = 0; d < hd; ++d) dot += q_row[d] * k_row[d];
                const float raw_s = dot * scale;
                const float s = raw_s + (mask_row ? mask_row[ki] : 0.0f);
                if (s == -std::numeric_limits<float>::infinity()) continue;
                const float m_new = s > m ? s : m;
                const float p = std::exp(s - m_new);
                const float correction = std::exp(m - m_new);
                const float* v_row = v_head + ki * hd;
                for (int64_t d = 0; d < hd; ++d) o_row[d] = correction * o_row[d] + p * v_row[d];
                l = correction * l + p;
                m = m_new;
            }
            const float inv_l = (l == 0.0f) ? 1.0f / std::numeric_limits<float>::epsilon() : 1.0f / l;
            for (int64_t d = 0; d < hd; ++d) o_row[d] *= inv_l;
        }
    }
}

void causal_mask(int64_t sq, int64_t sk, float* data) {  // attention.rs:292-305
    const int64_t offset = sk > sq ? sk - sq : 0;
    for (int64_t qi = 0; qi < sq; ++qi)
        for (int64_t ki = 0; ki < sk; ++ki)
            data[qi * sk + ki] = (ki > qi + offset) ? -std::numeric_limits<float>::infinity() : 0.0f;
}

// ── Elementwise (kernels/elementwise.rs:61-69,120-143) ───────────────────────
inline float silu1(float v) { return v / (1.0f + std::exp(-v)); }
inline float gelu1(float v) {
    const float SQRT_2_OVER_PI = 0.79788456f;
    const float COEF = 0.044715f;
    const float inner = SQRT_2_OVER_PI * (v + COEF * v * v * v);
    return 0.5f * v * (1.0f + std::tanh(inner));
}

// ── KV cache (forward/common.rs:355-538) ─────────────────────────────────────
// kind 0: f32 storage; 1: Q8_0 blocks (the reference's choice when hd % 32 == 0);
// 2: f32 storage holding values rounded through IEEE half (models an fp16 cache).
struct KvCache {
    int kind = 0;
    int64_t n_kv = 0, max_seq = 0, hd = 0;
    std::vector<float> f;     // [n_kv, max_seq, hd]
    std::vector<uint8_t> q8;  // [n_kv, max_seq, hd/32*34]
    void init(int kind_, int64_t n_kv_, int64_t max_seq_, int64_t hd_) {
        kind = kind_; n_kv = n_kv_; max_seq = max_seq_; hd = hd_;
        if (kind == 1) q8.assign((size_t)(n_kv * max_seq * (hd / 32) * 34), 0);
        else f.assign((size_t)(n_kv * max_seq * hd), 0.0f);
    }
    // Appends new_k [n_kv, new_seq, hd] at current_seq (sliding left on overflow) and
    // returns the live prefix [n_kv, total, hd] as f32. Returns total, or -1 on error.
    int64_t update(int64_t current_seq, const float* new_k, int64_t new_seq, std::vector<float>& out) {
        if (new_seq > max_seq) return -1;
        int64_t total = current_seq + new_seq;
        const int64_t shift = total > max_seq ? total - max_seq : 0;
        const int64_t insert_pos = shift > 0 ? current_seq - shift : current_seq;
        if (kind == 1) {
            const int64_t bph = hd / 32, bpp = bph * 34;
            auto pos_off = [&](int64_t hi, int64_t si) { return (size_t)((hi * max_seq + si) * bpp); };
            if (shift > 0) {
                const int64_t keep = current_seq - shift;
                for (int64_t hi = 0; hi < n_kv; ++hi)
                    for (int64_t si = 0; si < keep; ++si)
                        std::memmove(&q8[pos_off(hi, si)], &q8[pos_off(hi, si + shift)], (size_t)bpp);
            }
            for (int64_t hi = 0; hi < n_kv; ++hi)
                for (int64_t si = 0; si < new_seq; ++si) {
                    const float* src = new_k + (hi * new_seq + si) * hd;
                    uint8_t* dst = &q8[pos_off(hi, insert_pos + si)];
                    for (int64_t b = 0; b < bph; ++b) quantize_q8_0_block(src + b * 32, dst + b * 34);
                }
            if (shift > 0) total = max_seq;
            out.assign((size_t)(n_kv * total * hd), 0.0f);
            for (int64_t hi = 0; hi < n_kv; ++hi)
                for (int64_t si = 0; si < total; ++si) {
                    const uint8_t* src = &q8[pos_off(hi, si)];
                    float* dst = &out[(size_t)((hi * total + si) * hd)];
                    for (int64_t b = 0; b < bph; ++b) {
                        const float d = f16_to_f32(rd16(src + b * 34));
                        for (int j = 0; j < 32; ++j) dst[b * 32 + j] = (float)(int8_t)src[b * 34 + 2 + j] * d;
                    }
                }
            return total;
        }
        if (shift > 0) {
            const int64_t keep = current_seq - shift;
            for (int64_t hi = 0; hi < n_kv; ++hi)
                for (int64_t si = 0; si < keep; ++si)
                    std::memmove(&f[(size_t)((hi * max_seq + si) * hd)], &f[(size_t)((hi * max_seq + si + shift) * hd)],
                                 (size_t)hd * 4);
        }
        for (int64_t hi = 0; hi < n_kv; ++hi)
            for (int64_t si = 0; si < new_seq; ++si) {
                const float* src = new_k + (hi * new_seq + si) * hd;
                float* dst = &f[(size_t)((hi * max_seq + insert_pos + si) * hd)];
                if (kind == 2) for (int64_t d = 0; d < hd; ++d) dst[d] = f16_to_f32(f32_to_f16(src[d]));
                else std::memcpy(dst, src, (size_t)hd * 4);
            }
        if (shift > 0) total = max_seq;
        out.assign((size_t)(n_kv * total * hd), 0.0f);
        for (int64_t hi = 0; hi < n_kv; ++hi)
            std::memcpy(&out[(size_t)(hi * total * hd)], &f[(size_t)(hi * max_seq * hd)], (size_t)(total * hd) * 4);
        return total;
    }
};

// ── Embedding gather (forward/common.rs:164-217) ─────────────────────────────
int embed_tokens(int dtype, const uint8_t* table, int64_t vocab, int64_t hidden, const uint32_t* ids, int64_t n,
                 float* out) {
    const int64_t row_bytes = byte_count(dtype, hidden);
    if (row_bytes < 0) return 2;
    for (int64_t i = 0; i < n; ++i) {
        if ((int64_t)ids[i] >= vocab) return 3;  // "token id out of vocab range"
        if (dequant_any(dtype, table + (int64_t)ids[i] * row_bytes, hidden, out + i * hidden) != 0) return 2;
    }
    return 0;
}

// sampler.rs:161-168 — Iterator::max_by(partial_cmp): the LAST maximum wins; a
// comparison involving NaN counts as Equal (so the later element replaces).
int64_t argmax_last(const float* v, int64_t n) {
    if (n <= 0) return 0;
    int64_t best = 0;
    for (int64_t i = 1; i < n; ++i) {
        const float a = v[best], b = v[i];
        // max_by keeps the later element unless cmp(best, cand) == Greater.
        const bool greater = (a > b);  // false for NaN → Equal → later wins
        if (!greater) best = i;
    }
    return best;
}

// gguf_weights.rs:114-154 — inverse of the llama.cpp q/k row permutation.
void unpermute_qk_rows(const uint8_t* src, int64_t n_head, int64_t head_dim, int64_t row_bytes, uint8_t* dst) {
    const int64_t half = head_dim / 2;
    for (int64_t h = 0; h < n_head; ++h)
        for (int64_t a = 0; a < 2; ++a)
            for (int64_t b = 0; b < half; ++b) {
                const int64_t hf_row = h * head_dim + a * half + b;
                const int64_t gguf_row = h * head_dim + b * 2 + a;
                std::memcpy(dst + hf_row * row_bytes, src + gguf_row * row_bytes, (size_t)row_bytes);
            }
}

// ── Whole-model engine (forward/llama.rs:316-539; forward/phi.rs:277-557) ────
struct OTensor {
    int dtype = 0;
    std::vector<int64_t> dims;
    std::vector<uint8_t> bytes;
    int64_t numel() const { int64_t n = 1; for (auto d : dims) n *= d; return n; }
};

struct SoModelDesc {
    int32_t arch;        // 0: Llama/Qwen family (RMSNorm, SwiGLU, sequential block); 1: Phi-2 (LayerNorm, parallel block, GELU)
    int32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;
    int32_t max_ctx;     // KV window (kv_cache_ctx, forward/common.rs:25-37)
    int32_t rotary_dim;  // head_dim for full RoPE
    float norm_eps, rope_theta;
    int32_t kv_mode;     // 0 reference (Q8_0 when hd%32==0 else f32), 1 fp16-rounded, 2 f32
};

struct Engine {
    SoModelDesc d{};
    std::map<std::string, OTensor> w;
    std::vector<KvCache> kc, vc;
    int64_t seq_len = 0;
    std::string err;
    std::vector<float> trace;  // hidden state after every layer of the last forward: [L, seq, hidden]
    int64_t trace_seq = 0;

    const OTensor* get(const std::string& name) const {
        auto it = w.find(name);
        return it == w.end() ? nullptr : &it->second;
    }
    std::vector<float> f32_of(const OTensor& t) const {
        std::vector<float> o((size_t)t.numel());
        dequant_any(t.dtype, t.bytes.data(), t.numel(), o.data());
        return o;
    }
    void init_cache() {
        kc.resize(d.n_layers);
        vc.resize(d.n_layers);
        int kind;
        if (d.kv_mode == 0) kind = (d.head_dim % 32 == 0) ? 1 : 0;
        else if (d.kv_mode == 1) kind = 2;
        else kind = 0;
        for (int l = 0; l < d.n_layers; ++l) {
            kc[l].init(kind, d.n_kv_heads, d.max_ctx, d.head_dim);
            vc[l].init(kind, d.n_kv_heads, d.max_ctx, d.head_dim);
        }
        seq_len = 0;
    }
    // linear_3d_bias (forward/backend.rs:64-70; forward/common.rs:220-240,556-569)
    bool linear(const std::vector<float>& x, int64_t seq, const std::string& name, std::vector<float>& y,
                int64_t* out_dim) {
        const OTensor* wt = get("model." + name + ".weight");
        if (!wt) wt = get(name + ".weight");
        if (!wt) { err = "missing weight '" + name + "'"; return false; }
        const int64_t n = wt->dims[0], k = wt->dims[1];
        if ((int64_t)x.size() != seq * k) { err = "linear weight in_dim mismatch at " + name; return false; }
        y.assign((size_t)(seq * n), 0.0f);
        int st = matmul_nt(wt->dtype, x.data(), wt->bytes.data(), seq, k, n, y.data());
        if (st != 0) { err = "matmul_nt failed at " + name; return false; }
        const OTensor* bt = get("model." + name + ".bias");
        if (!bt) bt = get(name + ".bias");
        if (bt) {
            std::vector<float> b = f32_of(*bt);
            if ((int64_t)b.size() != n) { err = "bias length mismatch at " + name; return false; }
            for (size_t i = 0; i < y.size(); ++i) y[i] += b[i % (size_t)n];
        }
        *out_dim = n;
        return true;
    }
    bool norm_weight(const std::string& name, std::vector<float>& wv, std::vector<float>* bv, bool* has_b) {
        const OTensor* t = get("model." + name + ".weight");
        if (!t) { err = "missing weight '" + name + "'"; return false; }
        wv = f32_of(*t);
        if (bv) {
            const OTensor* b = get("model." + name + ".bias");
            *has_b = b != nullptr;
            if (b) *bv = f32_of(*b);
        }
        return true;
    }
    static void split_heads(const std::vector<float>& x, int64_t seq, int64_t nh, int64_t hd, std::vector<float>& o) {
        o.resize((size_t)(nh * seq * hd));  // [seq, nh, hd] → [nh, seq, hd]
        for (int64_t s = 0; s < seq; ++s)
            for (int64_t h = 0; h < nh; ++h)
                std::memcpy(&o[(size_t)((h * seq + s) * hd)], &x[(size_t)((s * nh + h) * hd)], (size_t)hd * 4);
    }
    static void merge_heads(const std::vector<float>& x, int64_t seq, int64_t nh, int64_t hd, std::vector<float>& o) {
        o.resize((size_t)(nh * seq * hd));
        for (int64_t s = 0; s < seq; ++s)
            for (int64_t h = 0; h < nh; ++h)
                std::memcpy(&o[(size_t)((s * nh + h) * hd)], &x[(size_t)((h * seq + s) * hd)], (size_t)hd * 4);
    }

    // forward_hidden (llama.rs:344-380; phi.rs:330-370)
    bool forward_hidden(const uint32_t* ids, int64_t seq, bool use_cache, std::vector<float>& x) {
        if (seq <= 0) { err = "empty input"; return false; }
        const OTensor* emb = get("model.embed_tokens.weight");
        if (!emb) { err = "missing embedding weights"; return false; }
        const int64_t hidden = d.hidden;
        x.assign((size_t)(seq * hidden), 0.0f);
        int st = embed_tokens(emb->dtype, emb->bytes.data(), emb->dims[0], hidden, ids, seq, x.data());
        if (st == 3) { err = "token id out of vocab range"; return false; }
        if (st != 0) { err = "unsupported embedding dtype"; return false; }
        int64_t start_pos;
        if (use_cache) start_pos = seq_len;
        else { seq_len = 0; start_pos = 0; }
        std::vector<int64_t> positions((size_t)seq);
        for (int64_t i = 0; i < seq; ++i) positions[(size_t)i] = start_pos + i;
        trace.assign((size_t)(d.n_layers * seq * hidden), 0.0f);
        trace_seq = seq;
        for (int l = 0; l < d.n_layers; ++l) {
            bool ok = d.arch == 1 ? phi_layer(x, seq, l, positions, use_cache) : llama_layer(x, seq, l, positions, use_cache);
            if (!ok) return false;
            std::memcpy(&trace[(size_t)(l * seq * hidden)], x.data(), (size_t)(seq * hidden) * 4);
        }
        if (use_cache) seq_len = std::min<int64_t>(start_pos + seq, d.max_ctx);
        std::vector<float> nw, nb, y((size_t)(seq * hidden));
        bool has_b = false;
        if (d.arch == 1) {
            std::string nm = get("model.final_layernorm.weight") ? "final_layernorm" : "norm";
            if (!norm_weight(nm, nw, &nb, &has_b)) return false;
            layer_norm(x.data(), nw.data(), has_b ? nb.data() : nullptr, seq, hidden, d.norm_eps, y.data());
        } else {
            if (!norm_weight("norm", nw, nullptr, nullptr)) return false;
            rms_norm(x.data(), nw.data(), seq, hidden, d.norm_eps, y.data());
        }
        x.swap(y);
        return true;
    }

    bool attend(std::vector<float>& q, std::vector<float>& k, std::vector<float>& v, int64_t seq, int l,
                bool use_cache, std::vector<float>& merged) {
        const int64_t H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim;
        int64_t sk = seq;
        std::vector<float> kk, vv;
        const float *kp = k.data(), *vp = v.data();
        if (use_cache) {
            int64_t t1 = kc[l].update(seq_len, k.data(), seq, kk);
            int64_t t2 = vc[l].update(seq_len, v.data(), seq, vv);
            if (t1 < 0 || t2 < 0) { err = "new tokens exceed max cache size"; return false; }
            sk = t1; kp = kk.data(); vp = vv.data();
        }
        std::vector<float> mask((size_t)(seq * sk));
        causal_mask(seq, sk, mask.data());
        std::vector<float> attn((size_t)(H * seq * hd));
        attention(q.data(), kp, vp, H, Hkv, seq, sk, hd, mask.data(), attn.data());
        merge_heads(attn, seq, H, hd, merged);
        return true;
    }

    // llama.rs:400-539
    bool llama_layer(std::vector<float>& x, int64_t seq, int l, const std::vector<int64_t>& positions, bool use_cache) {
        const int64_t hidden = d.hidden, H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim;
        const std::string pfx = "layers." + std::to_string(l);
        std::vector<float> nw, h((size_t)(seq * hidden));
        if (!norm_weight(pfx + ".input_layernorm", nw, nullptr, nullptr)) return false;
        rms_norm(x.data(), nw.data(), seq, hidden, d.norm_eps, h.data());
        std::vector<float> q2, k2, v2;
        int64_t nq, nk, nv;
        if (!linear(h, seq, pfx + ".self_attn.q_proj", q2, &nq)) return false;
        if (!linear(h, seq, pfx + ".self_attn.k_proj", k2, &nk)) return false;
        if (!linear(h, seq, pfx + ".self_attn.v_proj", v2, &nv)) return false;
        std::vector<float> q, k, v, qr, kr;
        split_heads(q2, seq, H, hd, q);
        split_heads(k2, seq, Hkv, hd, k);
        split_heads(v2, seq, Hkv, hd, v);
        qr.resize(q.size());
        kr.resize(k.size());
        rope(q.data(), H, seq, hd, positions.data(), d.rope_theta, d.rotary_dim, qr.data());
        rope(k.data(), Hkv, seq, hd, positions.data(), d.rope_theta, d.rotary_dim, kr.data());
        std::vector<float> merged;
        if (!attend(qr, kr, v, seq, l, use_cache, merged)) return false;
        std::vector<float> o;
        int64_t no;
        if (!linear(merged, seq, pfx + ".self_attn.o_proj", o, &no)) return false;
        for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + o[i];
        if (!norm_weight(pfx + ".post_attention_layernorm", nw, nullptr, nullptr)) return false;
        rms_norm(x.data(), nw.data(), seq, hidden, d.norm_eps, h.data());
        std::vector<float> gate, up, down;
        int64_t ng, nu, nd;
        // Dense SwiGLU: gate/up have no bias lookup in the reference (bk.linear_3d).
        const OTensor* gw = get("model." + pfx + ".mlp.gate_proj.weight");
        const OTensor* uw = get("model." + pfx + ".mlp.up_proj.weight");
        const OTensor* dw = get("model." + pfx + ".mlp.down_proj.weight");
        if (!gw || !uw || !dw) { err = "missing mlp weight at " + pfx; return false; }
        ng = gw->dims[0]; nu = uw->dims[0]; nd = dw->dims[0];
        gate.assign((size_t)(seq * ng), 0.0f);
        up.assign((size_t)(seq * nu), 0.0f);
        if (matmul_nt(gw->dtype, h.data(), gw->bytes.data(), seq, gw->dims[1], ng, gate.data())) { err = "gate matmul"; return false; }
        if (matmul_nt(uw->dtype, h.data(), uw->bytes.data(), seq, uw->dims[1], nu, up.data())) { err = "up matmul"; return false; }
        for (size_t i = 0; i < gate.size(); ++i) gate[i] = silu1(gate[i]) * up[i];
        down.assign((size_t)(seq * nd), 0.0f);
        if (matmul_nt(dw->dtype, gate.data(), dw->bytes.data(), seq, dw->dims[1], nd, down.data())) { err = "down matmul"; return false; }
        for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + down[i];
        return true;
    }

    // phi.rs:373-503 (Phi-1/1.5/2 parallel block)
    bool phi_layer(std::vector<float>& x, int64_t seq, int l, const std::vector<int64_t>& positions, bool use_cache) {
        const int64_t hidden = d.hidden, H = d.n_heads, Hkv = d.n_kv_heads, hd = d.head_dim;
        const std::string pfx = "layers." + std::to_string(l);
        std::vector<float> nw, nb, h((size_t)(seq * hidden));
        bool has_b = false;
        if (!norm_weight(pfx + ".input_layernorm", nw, &nb, &has_b)) return false;
        layer_norm(x.data(), nw.data(), has_b ? nb.data() : nullptr, seq, hidden, d.norm_eps, h.data());
        std::vector<float> q2, k2, v2;
        int64_t nq, nk, nv;
        if (!linear(h, seq, pfx + ".self_attn.q_proj", q2, &nq)) return false;
        if (!linear(h, seq, pfx + ".self_attn.k_proj", k2, &nk)) return false;
        if (!linear(h, seq, pfx + ".self_attn.v_proj", v2, &nv)) return false;
        std::vector<float> q, k, v, qr, kr;
        split_heads(q2, seq, H, hd, q);
        split_heads(k2, seq, Hkv, hd, k);
        split_heads(v2, seq, Hkv, hd, v);
        qr.resize(q.size());
        kr.resize(k.size());
        rope(q.data(), H, seq, hd, positions.data(), d.rope_theta, d.rotary_dim, qr.data());
        rope(k.data(), Hkv, seq, hd, positions.data(), d.rope_theta, d.rotary_dim, kr.data());
        // Parallel MLP from the same normalised input: fc1 → tanh-GELU → fc2.
        std::vector<float> ff1, ff;
        int64_t n1, n2;
        if (!linear(h, seq, pfx + ".mlp.fc1", ff1, &n1)) return false;
        for (auto& t : ff1) t = gelu1(t);
        if (!linear(ff1, seq, pfx + ".mlp.fc2", ff, &n2)) return false;
        std::vector<float> merged;
        if (!attend(qr, kr, v, seq, l, use_cache, merged)) return false;
        std::vector<float> o;
        int64_t no;
        const std::string oname = get("model." + pfx + ".self_attn.dense.weight") ? ".self_attn.dense" : ".self_attn.o_proj";
        if (!linear(merged, seq, pfx + oname, o, &no)) return false;
        for (size_t i = 0; i < x.size(); ++i) {
            const float parallel_res = o[i] + ff[i];
            x[i] = x[i] + parallel_res;
        }
        return true;
    }

    const OTensor* lm_head() const {  // weights.rs:88-109 (untied unless absent)
        const OTensor* t = get("lm_head.weight");
        if (!t) t = get("model.lm_head.weight");
        if (!t) t = get("model.embed_tokens.weight");
        return t;
    }
    // common.rs:621-650 (+ phi.rs:277-287 lm_head bias)
    bool logits_rows(const float* hid, int64_t rows, float* out) {
        const OTensor* lh = lm_head();
        if (!lh) { err = "missing lm_head.weight"; return false; }
        const int64_t v = lh->dims[0];
        if (matmul_nt(lh->dtype, hid, lh->bytes.data(), rows, d.hidden, v, out)) { err = "lm_head matmul"; return false; }
        if (d.arch == 1) {
            const OTensor* b = get("model.lm_head.bias");
            if (!b) b = get("lm_head.bias");
            if (b) {
                std::vector<float> bv = f32_of(*b);
                for (int64_t r = 0; r < rows; ++r)
                    for (int64_t i = 0; i < std::min<int64_t>(v, (int64_t)bv.size()); ++i) out[r * v + i] += bv[(size_t)i];
            }
        }
        return true;
    }
};

}  // namespace

// ═════════════════════════════ C interface (ctypes) ══════════════════════════
extern "C" {

int so_dequant(int dtype, const uint8_t* bytes, int64_t numel, float* out) { return dequant_any(dtype, bytes, numel, out); }
int64_t so_byte_count(int dtype, int64_t numel) { return byte_count(dtype, numel); }
void so_quantize_q8_0(const float* x, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / QK; ++b) quantize_q8_0_block(x + b * QK, out + b * Q8_0_BYTES);
}
void so_set_q8_mode(int mode) { g_q8_mode = mode; }
float so_dot_row(int dtype, const uint8_t* row, const float* x, int64_t k) { return dot_row(dtype, row, x, k); }
int so_matmul_nt(int dtype, const float* x, const uint8_t* w, int64_t m, int64_t k, int64_t n, float* y) {
    return matmul_nt(dtype, x, w, m, k, n, y);
}
void so_rms_norm(const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y) { rms_norm(x, w, rows, dim, eps, y); }
void so_layer_norm(const float* x, const float* w, const float* b, int64_t rows, int64_t dim, float eps, float* y) {
    layer_norm(x, w, b, rows, dim, eps, y);
}
void so_rope(const float* x, int64_t n_heads, int64_t seq, int64_t head_dim, const int64_t* positions, float base,
             int64_t rotary_dim, float* out) {
    rope(x, n_heads, seq, head_dim, positions, base, rotary_dim, out);
}
void so_attention(const float* q, const float* k, const float* v, int64_t H, int64_t Hkv, int64_t sq, int64_t sk,
                  int64_t hd, const float* mask, float* out) {
    attention(q, k, v, H, Hkv, sq, sk, hd, mask, out);
}
void so_causal_mask(int64_t sq, int64_t sk, float* out) { causal_mask(sq, sk, out); }
void so_silu(const float* x, int64_t n, float* y) { for (int64_t i = 0; i < n; ++i) y[i] = silu1(x[i]); }
void so_gelu(const float* x, int64_t n, float* y) { for (int64_t i = 0; i < n; ++i) y[i] = gelu1(x[i]); }
void so_add(const float* a, const float* b, int64_t n, float* y) { for (int64_t i = 0; i < n; ++i) y[i] = a[i] + b[i]; }
void so_mul(const float* a, const float* b, int64_t n, float* y) { for (int64_t i = 0; i < n; ++i) y[i] = a[i] * b[i]; }
int so_embed(int dtype, const uint8_t* table, int64_t vocab, int64_t hidden, const uint32_t* ids, int64_t n, float* out) {
    return embed_tokens(dtype, table, vocab, hidden, ids, n, out);
}
int64_t so_argmax(const float* v, int64_t n) { return argmax_last(v, n); }
void so_unpermute_qk_rows(const uint8_t* src, int64_t n_head, int64_t head_dim, int64_t row_bytes, uint8_t* dst) {
    unpermute_qk_rows(src, n_head, head_dim, row_bytes, dst);
}
uint16_t so_f32_to_f16(float f) { return f32_to_f16(f); }
float so_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// KV cache object for the append/slide known-answer tests.
void* so_kv_create(int kind, int64_t n_kv, int64_t max_seq, int64_t hd) {
    auto* c = new KvCache();
    c->init(kind, n_kv, max_seq, hd);
    return c;
}
void so_kv_destroy(void* c) { delete (KvCache*)c; }
// out must hold n_kv * min(current+new, max_seq) * hd floats; returns the live length.
int64_t so_kv_update(void* c, int64_t current_seq, const float* new_k, int64_t new_seq, float* out) {
    std::vector<float> o;
    int64_t t = ((KvCache*)c)->update(current_seq, new_k, new_seq, o);
    if (t >= 0) std::memcpy(out, o.data(), o.size() * 4);
    return t;
}
void so_kv_raw_f32(void* c, float* out) {
    auto* k = (KvCache*)c;
    std::memcpy(out, k->f.data(), k->f.size() * 4);
}

void* so_engine_create(const SoModelDesc* desc) {
    auto* e = new Engine();
    e->d = *desc;
    e->init_cache();
    return e;
}
void so_engine_destroy(void* e) { delete (Engine*)e; }
int so_engine_set_tensor(void* ev, const char* name, int dtype, const int64_t* dims, int ndim, const uint8_t* bytes,
                         int64_t nbytes) {
    auto* e = (Engine*)ev;
    OTensor t;
    t.dtype = dtype;
    t.dims.assign(dims, dims + ndim);
    int64_t want = byte_count(dtype, t.numel());
    if (want != nbytes) { e->err = std::string("byte size mismatch for ") + name; return 1; }
    std::string nm(name);
    // forward/common.rs:48-86 — 2-D F16/BF16 linears are quantised online to Q8_0.
    const bool skip = nm.find("norm") != std::string::npos || nm.find("bias") != std::string::npos ||
                      nm.find("embed") != std::string::npos || nm.find("lm_head") != std::string::npos;
    if (ndim == 2 && !skip && (dtype == T_F16 || dtype == T_BF16) && t.numel() >= 32 && t.numel() % 32 == 0) {
        std::vector<float> f((size_t)t.numel());
        dequant_any(dtype, bytes, t.numel(), f.data());
        t.dtype = T_Q8_0;
        t.bytes.resize((size_t)(t.numel() / 32 * 34));
        for (int64_t b = 0; b < t.numel() / 32; ++b) quantize_q8_0_block(&f[(size_t)(b * 32)], &t.bytes[(size_t)(b * 34)]);
    } else {
        t.bytes.assign(bytes, bytes + nbytes);
    }
    e->w[nm] = std::move(t);
    return 0;
}
const char* so_engine_error(void* e) { return ((Engine*)e)->err.c_str(); }
void so_engine_reset_cache(void* e) { ((Engine*)e)->seq_len = 0; }
int64_t so_engine_truncate_cache(void* ev, int64_t n) {
    auto* e = (Engine*)ev;
    e->seq_len = std::min(e->seq_len, n);
    return e->seq_len;
}
int64_t so_engine_seq_len(void* e) { return ((Engine*)e)->seq_len; }
// llama.rs:316-319 — last-position logits.
int so_engine_forward_logits(void* ev, const uint32_t* ids, int64_t n, int use_cache, float* logits) {
    auto* e = (Engine*)ev;
    std::vector<float> x;
    if (!e->forward_hidden(ids, n, use_cache != 0, x)) return 1;
    return e->logits_rows(&x[(size_t)((n - 1) * e->d.hidden)], 1, logits) ? 0 : 1;
}
// llama.rs:323-335 — all-position logits; cached != 0 appends to the KV cache.
int so_engine_forward_all_logits(void* ev, const uint32_t* ids, int64_t n, int cached, float* logits) {
    auto* e = (Engine*)ev;
    std::vector<float> x;
    if (!e->forward_hidden(ids, n, cached != 0, x)) return 1;
    return e->logits_rows(x.data(), n, logits) ? 0 : 1;
}
// Hidden state after layer `layer` of the most recent forward, [seq, hidden].
int64_t so_engine_trace(void* ev, int layer, float* out) {
    auto* e = (Engine*)ev;
    const int64_t n = e->trace_seq * e->d.hidden;
    if (layer < 0 || layer >= e->d.n_layers || e->trace.empty()) return -1;
    if (!out) return e->trace_seq;
    std::memcpy(out, &e->trace[(size_t)(layer * n)], (size_t)n * 4);
    return e->trace_seq;
}
// Thread count of the parallel loops from here on (n <= 0: leave as is). Launchers such as torch.distributed.run
// export OMP_NUM_THREADS=1 to their children; a timing run sets the count it wants explicitly.
void so_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
void so_set_kquant_order(int mode) { g_kquant_order = mode ? 1 : 0; }
void so_set_rows_at_once(int on) { g_rows_at_once = on ? 1 : 0; }
int so_num_threads() {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
