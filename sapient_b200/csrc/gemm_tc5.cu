// Large-M dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for prefill and batched decode.
//
// y[m, n] = sum_k x[m, k] * W[n, k] for m >= TC5_MIN_M activation rows. The GEMV kernel (gemv_imma.cu) streams the whole
// weight matrix once per 16 activation rows and its instruction count grows with the row count; here a CTA rebuilds
// each weight tile ONCE, as fp16, and the tensor core multiplies it with up to 256 activation rows:
//   * CTA tile: 128 weight rows (the MMA's M) x NB <= 256 activation rows (the MMA's N), K walked in chunks of 128
//     through a ring of 2-4 shared-memory stages;
//   * 16 producer warps, two per 16-row tile of the CTA tile (one per 64-column group of the stage): each lane reads
//     the 16-byte pieces the tiled layout holds for it (coalesced) — 32 weights, rows g and g+8 — from the
//     tile-repacked ggml blocks (the layout the GEMV reads, gemv_imma.cuh). The raw words of the NEXT chunk are in
//     flight in a second register set while the warp waits for the stage to be free (mbarrier `empty`), converts the
//     current words to fp16 (quants become exact floats by bit tricks, one f32 multiply-add applies scale and
//     minimum, one rounding to fp16), stores them in the K-major 128-byte-swizzled layout the tensor core reads, and
//     arrives on the stage's `full` mbarrier;
//     one producer thread also has TMA fetch the stage's activation tile (cp.async.bulk.tensor.2d with the 128-byte
//     swizzle, completing on the same mbarrier by byte count; rows past the matrix arrive as zeros);
//   * 1 thread issues, per chunk, eight tcgen05.mma (128 x NB x 16, kind::f16, fp32 accumulation in tensor memory)
//     and commits them to the stage's `empty` mbarrier — no block-wide barrier anywhere in the loop;
//   * epilogue, by the 16 producer warps once the last chunk is handed over: tcgen05.ld brings the accumulators back
//     (one weight row per thread, 16 activation rows per instruction; warp w serves TMEM lanes 32 (w % 4) .. +31),
//     bias / residual are added and y is written with n contiguous across the warp.
// fp16 rather than bf16 operands: same instruction kind and rate, and the 11-bit significand keeps the result within
// ~2e-4 relative L2 of the f32 reference (bf16 would sit at ~2e-3, above the 1e-3 parity bar). Each weight is computed
// in f32 from exact operands and rounded to fp16 once (Q8_0: the exact product of int8 and f16 scale, in half2).
// Exact-class mode (Tc5Args::exact, the default of the callers): an fp16 operand carries 11 bits, so weights and
// activations are each handed over as TWO fp16 numbers — the value rounded to fp16 and the fp16 of what that rounding
// dropped (activation rows are first scaled by a power of two into (-1, 1), the epilogue multiplies it back) — and every
// 16-column step issues three MMAs into the same accumulators: W_hi X_hi + W_lo X_hi + W_hi X_lo (the remainder x
// remainder term is below f32 rounding). A tensor-memory stage then holds both weight parts (128 columns, ring of two),
// a shared-memory stage both activation tiles of the chunk (or, for tiles of more than 128 rows, 64 columns of both with
// two hand-overs per chunk on that side). The result sits at ~1e-6 per product, the level of the integer GEMV.
// Every wait on an mbarrier is bounded; on expiry the kernel raises g_tc5_timeout, still frees its tensor memory
// and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <type_traits>

#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

constexpr int TC5_PRODUCER_WARPS = 16;        // two per 16-row tile: one per 64-column group of the stage
constexpr int TC5_THREADS = 32 * (TC5_PRODUCER_WARPS + 2);  // + the MMA warp + the TMA warp
// Warp 0 (the oldest, which the scheduler favours) owns the tensor memory and its lane 0 issues the MMAs; warp 1 lane 0 runs the TMA.
constexpr int TC5_MMA_WARP = 0, TC5_FIRST_PRODUCER = 2;
constexpr int TC5_MAX_STAGES = 8;              // ring of activation tiles in shared memory
constexpr int TC5_A_STAGES = 4;                // ring of weight tiles in tensor memory, 64 columns (128 fp16 per row) each
constexpr int TC5_TMEM_COLS = 512;             // columns 0 .. 255: accumulators; 256 + 64 s ..: weight stage s
constexpr int TC5_BM = 128;                    // weight rows per CTA
constexpr int TC5_BK = 128;                    // columns per stage = two 128-byte swizzle rows of fp16 activations
constexpr int TC5_NB_MAX = 256;                // activation rows per CTA
constexpr int TC5_SMEM_LIMIT = 192 * 1024;
constexpr int TC5_SMEM_MIN = 120 * 1024;       // more than half an SM's shared memory: one CTA per SM, which owns all of its tensor memory
constexpr int TC5_SPIN_LIMIT = 1 << 22;

__device__ int g_tc5_timeout = 0;

__device__ __forceinline__ uint32_t tc5_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t tc5_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address / 16
    d |= (uint64_t)1 << 16;                    // leading-dimension byte offset / 16 (not used by swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride-dimension byte offset / 16: next 8-row group
    d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                    // 128-byte swizzle
    return d;
}

// Instruction descriptor, kind::f16: fp16 A and B, fp32 D, both K-major, M = 128, N = nb.
__device__ __forceinline__ uint32_t tc5_idesc(int nb) {
    return (1u << 4) | ((uint32_t)(nb >> 3) << 17) | ((uint32_t)(TC5_BM >> 4) << 24);
}

__device__ __forceinline__ void tc5_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with the A operand (weights) read from tensor memory: lane = weight row, 8 columns = 16 fp16 along K.
__device__ __forceinline__ void tc5_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same, always accumulating.
__device__ __forceinline__ void tc5_mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.eq.u32 p, 1, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc)
        : "memory");
}

// 16 lanes x 8 columns of tensor memory from a warp, in the layout of an mma accumulator fragment: lane (g, t) gives
// columns 2 t, 2 t + 1 of lane g (v[0], v[1]) and of lane g + 8 (v[2], v[3]).
__device__ __forceinline__ void tc5_tmem_st(uint32_t taddr, const uint32_t (&v)[4]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3])
                 : "memory");
}

__device__ __forceinline__ void tc5_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc5_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc5_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc5_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool tc5_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = tc5_smem_u32(bar);
    for (int i = 0; i < TC5_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    return (uint32_t)__half_as_ushort(__float2half_rn(a)) | ((uint32_t)__half_as_ushort(__float2half_rn(b)) << 16);
}
__device__ __forceinline__ __half2 h2_bits(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t bits_h2(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Bytes 0 and 2 (resp. 1 and 3) of v, each below 1024, as exact halves: the bit pattern 0x6400 | n is the half 1024 + n.
__device__ __forceinline__ __half2 bytes02(uint32_t v, uint32_t mask, float bias) {
    return __hsub2(h2_bits((v & mask) | 0x64006400u), __float2half2_rn(bias));
}

// Producer warp w of the CTA rebuilds 16-row tile w of the CTA's 8 tiles; lane (g = lane / 4, t = lane % 4) reads, per
// 64-column chunk, exactly the 16-byte pieces the tile layout stores for it (coalesced: 512 B per warp and piece) and
// gets 32 weights: rows g and g + 8, eight runs of 4 consecutive columns. Raw words are fetched one chunk ahead.
struct Tc5Raw {
    uint4 q[3];     // Q4_K: q[0]; Q8_0: q[0], q[1] (two 32-blocks); Q6_K: three pieces = the 12 words of the chunk's half
    uint4 hdr[2];   // rows g / g+8 — Q4_K: d|dmin + 12 scale bytes; Q6_K: 16 int8 scales; Q8_0: x = d of block 0 | block 1 << 16
    uint32_t dd;    // Q6_K: d of row g | d of row g+8 << 16
};

// Read-only global loads as volatile asm: they stay where the code puts them (a chunk ahead of their use).
__device__ __forceinline__ uint4 tc5_ldg16(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t tc5_ldg4(const uint8_t* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];\n" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t tc5_ldg2(const uint8_t* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return v;
}

// Q8_0 rows whose width is a multiple of 128 but not of 256 are tiled four 32-blocks (128 columns) at a time: one tile
// per chunk, its 64-column groups 0 and 1 are what a wider tile calls groups cq and cq + 2.
constexpr int T_Q8_0_HALF = 1000 + T_Q8_0;

template <int DT>
__device__ __forceinline__ void tc5_load(const uint8_t* tile, int lane, int cq, Tc5Raw& r) {
    const int g = lane >> 2;
    if (DT == T_Q8_0_HALF) {
        r.q[0] = tc5_ldg16(tile + (2 * cq) * 512 + lane * 16);
        r.q[1] = tc5_ldg16(tile + (2 * cq + 1) * 512 + lane * 16);
        r.hdr[0].x = tc5_ldg4(tile + 2048 + (g * 4 + 2 * cq) * 2);        // d of blocks 2cq, 2cq+1
        r.hdr[1].x = tc5_ldg4(tile + 2048 + ((g + 8) * 4 + 2 * cq) * 2);
    } else if (DT == T_Q4_K) {
        r.q[0] = tc5_ldg16(tile + cq * 512 + lane * 16);
        r.hdr[0] = tc5_ldg16(tile + 2048 + g * 16);
        r.hdr[1] = tc5_ldg16(tile + 2048 + (g + 8) * 16);
    } else if (DT == T_Q8_0) {
        r.q[0] = tc5_ldg16(tile + (2 * cq) * 512 + lane * 16);
        r.q[1] = tc5_ldg16(tile + (2 * cq + 1) * 512 + lane * 16);
        r.hdr[0].x = tc5_ldg4(tile + 4096 + (g * 8 + 2 * cq) * 2);        // d of blocks 2cq, 2cq+1
        r.hdr[1].x = tc5_ldg4(tile + 4096 + ((g + 8) * 8 + 2 * cq) * 2);
    } else {
        const int half = cq >> 1;
#pragma unroll
        for (int i = 0; i < 3; ++i) r.q[i] = tc5_ldg16(tile + (3 * half + i) * 512 + lane * 16);
        r.hdr[0] = tc5_ldg16(tile + 3072 + g * 16);
        r.hdr[1] = tc5_ldg16(tile + 3072 + (g + 8) * 16);
        r.dd = tc5_ldg2(tile + 3328 + 2 * g) | (tc5_ldg2(tile + 3328 + 2 * (g + 8)) << 16);
    }
}

// Byte b (< 128) of v as the float 0.5 + n / 256: bit pattern 0x3F000000 | n << 16. With it a weight s * n + c costs one
// byte permute and one fused multiply-add: fmaf(half_plus(v, b), 256 s, c - 128 s).
__device__ __forceinline__ float half_plus(uint32_t v, int b) { return __uint_as_float(__byte_perm(v, 0x3F000000u, 0x7044 | (b << 8))); }

// Byte b of v as an exact f32 (0x4B000000 | n is the float 2^23 + n).
__device__ __forceinline__ float byte_f32(uint32_t v, int b) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540 | b)) - 8388608.0f;
}

__device__ __forceinline__ uint32_t u4_word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// A thread's 32 rebuilt weights: o[cg] is its share of columns 16 cg .. 16 cg + 15 of the 64-column group, as the four
// words tc5_tmem_st takes: lane (g, t) holds columns 16 cg + 4 t .. + 3 of tile rows g (words 0, 1) and g + 8 (2, 3).
typedef uint32_t Tc5Out[4][4];
__device__ __forceinline__ void tc5_put(Tc5Out& o, int cg, int hi8, uint32_t c01, uint32_t c23) {
    o[cg][2 * hi8] = c01;
    o[cg][2 * hi8 + 1] = c23;
}
// EXACT: ol receives what the rounding to fp16 dropped (f - half(f), itself rounded to fp16): hi + lo holds the f32
// weight to ~2^-22 of its magnitude (2^-24 absolute once the remainder is subnormal, i.e. for |w| < 0.06: then still
// ~2^-19 of a 0.02-sized weight).
template <bool EXACT>
__device__ __forceinline__ void tc5_put4f(Tc5Out& o, Tc5Out& ol, int cg, int hi8, float f0, float f1, float f2, float f3) {
    const __half2 h01 = __floats2half2_rn(f0, f1), h23 = __floats2half2_rn(f2, f3);
    tc5_put(o, cg, hi8, bits_h2(h01), bits_h2(h23));
    if (EXACT)
        tc5_put(ol, cg, hi8, bits_h2(__floats2half2_rn(f0 - __low2float(h01), f1 - __high2float(h01))),
                bits_h2(__floats2half2_rn(f2 - __low2float(h23), f3 - __high2float(h23))));
}

// Converts the raw words of chunk group cq to the thread's 32 fp16 weights.
template <int DT, bool EXACT>
__device__ __forceinline__ void tc5_convert(const Tc5Raw& r, int cq, Tc5Out& o, Tc5Out& ol) {
    if (DT == T_Q4_K) {
#pragma unroll
        for (int hi8 = 0; hi8 < 2; ++hi8) {
            const uint4 hd = r.hdr[hi8];
            const float d = half_bits_to_float((uint16_t)(hd.x & 0xFFFFu)), dmin = half_bits_to_float((uint16_t)(hd.x >> 16));
            // the 6-bit (scale, minimum) pairs of sub-blocks 2 cq and 2 cq + 1, one per byte
            uint32_t sc2, mn2;
            if (cq < 2) {
                sc2 = (hd.y >> (16 * cq)) & 0x3F3Fu;
                mn2 = (hd.z >> (16 * cq)) & 0x3F3Fu;
            } else {
                const int sh = 16 * (cq - 2);
                const uint32_t x = hd.w >> sh;
                sc2 = (x & 0x0F0Fu) | (((hd.y >> sh) >> 2) & 0x3030u);
                mn2 = ((x >> 4) & 0x0F0Fu) | (((hd.z >> sh) >> 2) & 0x3030u);
            }
            // Nibbles become floats two at a time: (w & 0x000F000F) | 0x64006400 is the half pair (1024 + q, 1024 + q') of
            // bytes 0 and 2, with mask 0x00F000F0 it is (1024 + 16 q, ..) of their high nibbles; the halves widen to f32
            // exactly. d * sc and dmin * mn are exact in f32 (11-bit x 6-bit), so weight = dl * q - ml comes out of one
            // fused multiply-add against a constant that is itself rounded once in f32 (2^-14 dl at most, far below the
            // fp16 rounding that follows).
            float sl[2], cl[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {  // low nibbles: sub-block 2 cq, high nibbles: 2 cq + 1
                const float dl = d * byte_f32(sc2, hh), ml = dmin * byte_f32(mn2, hh);
                sl[hh] = hh ? 0.0625f * dl : dl;
                cl[hh] = fmaf(hh ? -64.0f : -1024.0f, dl, -ml);
            }
#pragma unroll
            for (int h16 = 0; h16 < 2; ++h16) {
                const uint32_t w = u4_word(r.q[0], 2 * hi8 + h16), w8 = w >> 8;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const uint32_t mask = hh ? 0x00F000F0u : 0x000F000Fu;
                    const __half2 p02 = h2_bits((w & mask) | 0x64006400u), p13 = h2_bits((w8 & mask) | 0x64006400u);
                    tc5_put4f<EXACT>(o, ol, 2 * hh + h16, hi8, fmaf(__low2float(p02), sl[hh], cl[hh]), fmaf(__low2float(p13), sl[hh], cl[hh]),
                                     fmaf(__high2float(p02), sl[hh], cl[hh]), fmaf(__high2float(p13), sl[hh], cl[hh]));
                }
            }
        }
    } else if (DT == T_Q8_0 || DT == T_Q8_0_HALF) {
#pragma unroll
        for (int hi8 = 0; hi8 < 2; ++hi8) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                const __half2 d = __half2half2(__ushort_as_half((uint16_t)(r.hdr[hi8].x >> (16 * blk))));
#pragma unroll
                for (int h16 = 0; h16 < 2; ++h16) {
                    const uint32_t v = u4_word(r.q[blk], 2 * hi8 + h16) ^ 0x80808080u;  // int8 -> offset-128 unsigned
                    if (EXACT) {  // int8 x f16 scale is exact in f32 (8 + 11 bits): leading part and remainder
                        const float2 q02 = __half22float2(bytes02(v, 0x00FF00FFu, 1152.f)), q13 = __half22float2(bytes02(v >> 8, 0x00FF00FFu, 1152.f));
                        const float df = __low2float(d);
                        tc5_put4f<true>(o, ol, 2 * blk + h16, hi8, q02.x * df, q13.x * df, q02.y * df, q13.y * df);
                    } else {
                        const uint32_t e02 = bits_h2(__hmul2(bytes02(v, 0x00FF00FFu, 1152.f), d));       // columns +0, +2
                        const uint32_t e13 = bits_h2(__hmul2(bytes02(v >> 8, 0x00FF00FFu, 1152.f), d));  // columns +1, +3
                        tc5_put(o, 2 * blk + h16, hi8, __byte_perm(e02, e13, 0x5410), __byte_perm(e02, e13, 0x7632));
                    }
                }
            }
        }
    } else {  // Q6_K
        const int half = cq >> 1, odd = cq & 1;
#pragma unroll
        for (int hi8 = 0; hi8 < 2; ++hi8) {
            const float d = half_bits_to_float((uint16_t)(r.dd >> (16 * hi8)));
            // int8 scales 8 half + 4 odd + 2 ab + p of the row: one word
            const uint32_t sw = u4_word(r.hdr[hi8], 2 * half + odd);
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                // the 12 words of the half: for p = 0, 1: qlA_g, qlB_g, qh_g, qlA_g8, qlB_g8, qh_g8
                const int base = 6 * p + 3 * hi8;
                const uint32_t qh = u4_word(r.q[(base + 2) >> 2], (base + 2) & 3);
#pragma unroll
                for (int ab = 0; ab < 2; ++ab) {  // qlA: columns l, qlB: columns 32 + l  (l = 16 p + 4 t + b)
                    const uint32_t ql = u4_word(r.q[(base + ab) >> 2], (base + ab) & 3);
                    const int quarter = 2 * odd + ab;
                    const float dsc = d * (float)(int8_t)((sw >> (8 * (2 * ab + p))) & 0xFFu);  // exact in f32 (11-bit x 8-bit)
                    // dsc * (q - 32) = 256 dsc * (0.5 + q / 256) - 160 dsc: both constants exact, one rounding in the fma
                    const float s256 = 256.0f * dsc, c = -160.0f * dsc;
                    const uint32_t q = ((odd ? (ql >> 4) : ql) & 0x0F0F0F0Fu) | (((qh >> (2 * quarter)) & 0x03030303u) << 4);
                    tc5_put4f<EXACT>(o, ol, 2 * ab + p, hi8, fmaf(half_plus(q, 0), s256, c), fmaf(half_plus(q, 1), s256, c),
                                     fmaf(half_plus(q, 2), s256, c), fmaf(half_plus(q, 3), s256, c));
                }
            }
        }
    }
}

// One producer warp's pass over the CTA's chunks, for one weight format and one of the two 64-column groups of a
// chunk. c_begin and n_chunks are even, so the warp alternates between groups SUB and SUB + 2 of a superblock tile and
// moves to the next tile every second chunk: all offsets inside a tile are compile-time constants.
template <int DT, int SUB, bool EXACT>
__device__ __forceinline__ bool tc5_produce(const uint8_t* tile_row, bool row_live, int c_begin, int n_chunks, int lane, uint32_t a_base,
                                            uint64_t* full_a, uint64_t* empty_a) {
    constexpr bool HALF = DT == T_Q8_0_HALF;  // one tile per chunk: group SUB of every tile, any c_begin and n_chunks
    constexpr int TILE_BYTES = DT == T_Q4_K ? Q4_K_TILE_BYTES : DT == T_Q6_K ? Q6_K_TILE_BYTES : HALF ? 4 * 544 : 8 * 544;
    bool ok = true;
    const uint8_t* tile = tile_row + (int64_t)(HALF ? c_begin : c_begin >> 1) * TILE_BYTES;
    int s = -1, u = 0;  // stage of the current chunk and the number of times the ring has wrapped
    // EXACT: a stage is 128 columns wide — the leading parts in its first 64 columns, the remainders in the other 64 — and
    // the ring has two stages instead of four; one hand-over per chunk either way.
    constexpr int STAGES = EXACT ? TC5_A_STAGES / 2 : TC5_A_STAGES, STAGE_COLS = EXACT ? 128 : 64;
    auto build = [&](const Tc5Raw& raw, int cq) {  // next chunk: rebuild the weights in registers, wait for its stage, store
        if (++s == STAGES) { s = 0; ++u; }
        Tc5Out o, ol;
        if (row_live) {
            tc5_convert<DT, EXACT>(raw, cq, o, ol);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) { o[i >> 2][i & 3] = 0u; ol[i >> 2][i & 3] = 0u; }  // rows past the matrix
        }
        if (u > 0) ok = ok && tc5_wait(&empty_a[s], (uint32_t)((u - 1) & 1));  // the MMAs that last read this stage are done
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) tc5_tmem_st(a_base + (uint32_t)(STAGE_COLS * s + 8 * cg), o[cg]);
        if (EXACT) {
#pragma unroll
            for (int cg = 0; cg < 4; ++cg) tc5_tmem_st(a_base + (uint32_t)(STAGE_COLS * s + 64 + 8 * cg), ol[cg]);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) tc5_arrive(&full_a[s]);
    };
    // two register sets: the loads of the next chunk are in flight while a chunk is rebuilt
    Tc5Raw raw_a, raw_b;
    if (row_live) tc5_load<DT>(tile, lane, SUB, raw_a);
    for (int c = 0; c < n_chunks; c += 2) {
        if (HALF) {
            if (row_live && c + 1 < n_chunks) tc5_load<DT>(tile + TILE_BYTES, lane, SUB, raw_b);
            build(raw_a, SUB);
            tile += 2 * TILE_BYTES;
            if (row_live && c + 2 < n_chunks) tc5_load<DT>(tile, lane, SUB, raw_a);
            if (c + 1 < n_chunks) build(raw_b, SUB);
        } else {
            if (row_live) tc5_load<DT>(tile, lane, SUB + 2, raw_b);
            build(raw_a, SUB);
            tile += TILE_BYTES;
            if (row_live && c + 2 < n_chunks) tc5_load<DT>(tile, lane, SUB, raw_a);
            build(raw_b, SUB + 2);
        }
    }
    return ok;
}

struct Tc5Args {
    Tc5Seg seg[3];      // up to three matrices sharing the activations (q|k|v, gate|up); CTAs are dealt to them in order
    int nseg;
    int k;              // columns (k % 256 == 0; Q8_0 alone: k % 128 == 0)
    const __half* xh;   // activations as fp16 [m][k]
    int m;
    int ldy;
    const float* res;   // [m][ldres] or null, added to segment 0 (may alias its y)
    int ldres;
    // Work items = (128-row weight tile, 256-row activation tile) pairs, m_tiles consecutive items per weight tile.
    // CTAs 0 .. full_items-1 take one item each over the whole K range; the items after them (the last, partial wave
    // of the grid) are each shared by tail_split CTAs that take a part of the K range. Each writes its partial tile to
    // split_buf[(item - full_items) * tail_split + part][256 activation rows][128 weight rows]; the CTA that arrives
    // last at split_cnt[item - full_items] adds the parts in part order (after the residual, when y holds it in place)
    // and writes y: the order of the f32 additions is fixed, results do not vary from run to run.
    int m_tiles, full_items, tail_split;
    float* split_buf;
    unsigned* split_cnt;
    int stage_bytes;    // 256 * (widest activation tile of the launch, rounded to 16): two boxes of 64 columns
    int stages;         // depth of the activation ring that fits shared memory (3..8)
    // 1: exact-class operands. xh holds [2 m][k]: rows 0..m-1 the fp16 leading parts of the activations, rows m..2m-1
    // their remainders; the weights are split the same way by the producers (a weight stage of tensor memory holds both
    // parts; an activation stage of shared memory holds both tiles of the chunk (1) or, for tiles of more than 128 rows,
    // 64 columns of both row planes (2)). Every chunk of K is multiplied three times
    // into the same accumulators — W_hi X_hi, W_lo X_hi, W_hi X_lo (the remainder x remainder term is below f32 rounding).
    int exact;
    const float* xscale;  // exact: [m] power-of-two factors the rows of xh were divided by
};

__global__ void __launch_bounds__(TC5_THREADS, 1) gemm_tc5_kernel(const Tc5Args a, const __grid_constant__ CUtensorMap tmap_x) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_a[TC5_A_STAGES], empty_a[TC5_A_STAGES], full_b[TC5_MAX_STAGES], empty_b[TC5_MAX_STAGES], done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int split_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* smem = smem_raw + ((1024u - (tc5_smem_u32(smem_raw) & 1023u)) & 1023u);
    // which matrix of the launch this CTA works on, and its 128-row tile there
    int item = blockIdx.x, part = 0, parts = 1;
    if (item >= a.full_items) {
        const int t = item - a.full_items;
        item = a.full_items + t / a.tail_split;
        part = t % a.tail_split;
        parts = a.tail_split;
    }
    int bx = item / a.m_tiles, si = 0;
    while (si < a.nseg - 1 && bx >= (a.seg[si].n + TC5_BM - 1) / TC5_BM) { bx -= (a.seg[si].n + TC5_BM - 1) / TC5_BM; ++si; }
    const Tc5Seg& sg = a.seg[si];
    const int DT = (sg.dtype == T_Q8_0 && (a.k & 255)) ? T_Q8_0_HALF : sg.dtype;
    const int TILE_BYTES = DT == T_Q4_K ? Q4_K_TILE_BYTES : DT == T_Q6_K ? Q6_K_TILE_BYTES : 8 * 544;  // per 256 columns
    const int n0 = bx * TC5_BM, m0 = (item % a.m_tiles) * TC5_NB_MAX;
    const int rows_here = min(TC5_NB_MAX, a.m - m0);
    const int nb = (rows_here + 15) & ~15;  // the MMA's N
    const int n_tile_rows = (sg.n + 15) >> 4;
    const int64_t row_tile_bytes = (int64_t)(a.k >> 7) * (TILE_BYTES >> 1);  // one 16-row tile row: k / 256 tiles (Q8_0: k / 128 half tiles)
    // this CTA's share of the K range (all of it unless the launch splits K)
    const int all_chunks = a.k / TC5_BK;
    // even boundaries (all_chunks is even): a producer warp then always starts on the first half of a superblock tile
    const int even = (a.k & 255) ? ~0 : ~1;  // (widths that are odd multiples of 128 exist only with one tile per chunk)
    const int c_begin = (int)((int64_t)part * all_chunks / parts) & even, c_end = (int)((int64_t)(part + 1) * all_chunks / parts) & even;
    const int n_chunks = c_end - c_begin;

    if (warp == TC5_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5_smem_u32(&tmem_slot)), "r"(TC5_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s < TC5_A_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc5_smem_u32(&full_a[s])), "r"(TC5_PRODUCER_WARPS) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&empty_a[s])) : "memory");
        }
        for (int s = 0; s < a.stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&full_b[s])) : "memory");  // the TMA thread, + bytes
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&empty_b[s])) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&done_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_wait();  // activations come from the previous kernel
    pdl_trigger();

    bool ok = true;
    const int pw = warp - TC5_FIRST_PRODUCER;  // producer index 0..15 (negative: the two service warps)
    if (pw >= 0) {
        // ── producers: a warp may touch only the 32 tensor-memory lanes of its quarter (warp % 4); the four producers of
        //    a quarter take its two 16-row tiles x the two 64-column groups of each chunk ──
        const int tile_w = 2 * (warp & 3) + ((pw >> 2) & 1), sub = pw >> 3;
        const int rt = (n0 >> 4) + tile_w;
        const bool row_live = rt < n_tile_rows;
        const uint8_t* tile_row = sg.wt + (int64_t)rt * row_tile_bytes;
        // lanes 16 tile_w .. + 15, columns of stage 0 of the weight ring
        const uint32_t a_base = tmem + ((uint32_t)(16 * tile_w) << 16) + (uint32_t)(TC5_NB_MAX + 32 * sub);
#define SP_PRODUCE(T)                                                                                                      \
    ok = a.exact ? (sub ? tc5_produce<T, 1, true>(tile_row, row_live, c_begin, n_chunks, lane, a_base, full_a, empty_a)    \
                        : tc5_produce<T, 0, true>(tile_row, row_live, c_begin, n_chunks, lane, a_base, full_a, empty_a))   \
                 : (sub ? tc5_produce<T, 1, false>(tile_row, row_live, c_begin, n_chunks, lane, a_base, full_a, empty_a)   \
                        : tc5_produce<T, 0, false>(tile_row, row_live, c_begin, n_chunks, lane, a_base, full_a, empty_a))
        if (DT == T_Q4_K) SP_PRODUCE(T_Q4_K);
        else if (DT == T_Q6_K) SP_PRODUCE(T_Q6_K);
        else if (DT == T_Q8_0) SP_PRODUCE(T_Q8_0);
        else SP_PRODUCE(T_Q8_0_HALF);
#undef SP_PRODUCE
    } else if (warp == TC5_MMA_WARP) {
        if (lane == 0) {
            // ── MMA issuer ──
            // The issuing thread is the serial part of the pipeline: per chunk two waits, eight MMAs whose operands are one
            // add away from per-stage bases, two commits.
            const uint32_t idesc = tc5_idesc(nb);
            const uint64_t bd0 = tc5_desc(tc5_smem_u32(smem));
            const uint32_t bd_hi = (uint32_t)(bd0 >> 32), bd_lo0 = (uint32_t)bd0;
            const uint32_t stage16 = (uint32_t)a.stage_bytes >> 4, half16 = stage16 >> 1;
            // two compile-time variants of the loop: the issuing thread is the serial part, a run-time test per MMA costs
            // MODE 0: operands rounded to fp16. MODE 1: exact-class, an activation stage holds both tiles of a chunk (twice
            // stage_bytes; tiles of up to 128 rows). MODE 2: exact-class, an activation stage holds 64 columns of both row
            // planes (stage_bytes; two hand-overs per chunk), so that 256-row tiles still have a ring of three stages.
            auto issue_all = [&](auto mode_tag) {
                constexpr int MODE = decltype(mode_tag)::value;
                constexpr bool EX = MODE != 0;
                constexpr int A_STAGES = EX ? TC5_A_STAGES / 2 : TC5_A_STAGES;
                constexpr uint32_t A_COLS = EX ? 128u : 64u;
                const uint32_t b16 = MODE == 1 ? 2u * stage16 : stage16;
                uint32_t accumulate = 0u;
                for (int c = 0, sa = 0, ua = 0, sb = 0, ub = 0; c < n_chunks; ++c, ++sa) {
                    if (sa == A_STAGES) { sa = 0; ++ua; }
                    if (MODE != 2) {
                        if (sb == a.stages) { sb = 0; ++ub; }
                        ok = ok && tc5_wait(&full_b[sb], (uint32_t)(ub & 1));  // after one expired wait nothing else is waited for
                    }
                    ok = ok && tc5_wait(&full_a[sa], (uint32_t)(ua & 1));
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t At = tmem + (uint32_t)TC5_NB_MAX + A_COLS * (uint32_t)sa;
                    if (MODE != 2) {
                        const uint32_t bd_lo = bd_lo0 + (uint32_t)sb * b16;  // the address field: no carry out of the low word
#pragma unroll
                        for (int i = 0; i < 8; ++i) {  // 16 columns each: 8 columns of tensor memory, 32 bytes inside the swizzle row (+2 x 16 B)
                            const uint32_t lo = bd_lo + (uint32_t)(i >> 2) * half16 + 2u * (i & 3);
                            uint64_t bd;
                            asm("mov.b64 %0, {%1, %2};\n" : "=l"(bd) : "r"(lo), "r"(bd_hi));
                            if (i == 0) tc5_mma_ts(tmem, At, bd, idesc, accumulate);
                            else tc5_mma_ts_acc(tmem, At + 8u * i, bd, idesc);            // W (or W_hi) X (X_hi)
                            if (MODE == 1) {
                                uint64_t bdl;  // the remainders' tile follows the leading parts' tile in the stage
                                asm("mov.b64 %0, {%1, %2};\n" : "=l"(bdl) : "r"(lo + stage16), "r"(bd_hi));
                                tc5_mma_ts_acc(tmem, At + 64u + 8u * i, bd, idesc);       // W_lo X_hi
                                tc5_mma_ts_acc(tmem, At + 8u * i, bdl, idesc);            // W_hi X_lo
                            }
                        }
                        tc5_commit(&empty_b[sb]);
                        ++sb;
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (sb == a.stages) { sb = 0; ++ub; }
                            ok = ok && tc5_wait(&full_b[sb], (uint32_t)(ub & 1));
                            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                            const uint32_t bd_lo = bd_lo0 + (uint32_t)sb * stage16;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t i = 4u * h + j;
                                uint64_t bd, bdl;  // the leading parts' box, then the remainders' box
                                asm("mov.b64 %0, {%1, %2};\n" : "=l"(bd) : "r"(bd_lo + 2u * j), "r"(bd_hi));
                                asm("mov.b64 %0, {%1, %2};\n" : "=l"(bdl) : "r"(bd_lo + half16 + 2u * j), "r"(bd_hi));
                                if (i == 0) tc5_mma_ts(tmem, At, bd, idesc, accumulate);
                                else tc5_mma_ts_acc(tmem, At + 8u * i, bd, idesc);          // W_hi X_hi
                                tc5_mma_ts_acc(tmem, At + 64u + 8u * i, bd, idesc);           // W_lo X_hi
                                tc5_mma_ts_acc(tmem, At + 8u * i, bdl, idesc);                // W_hi X_lo
                            }
                            tc5_commit(&empty_b[sb]);
                            ++sb;
                        }
                    }
                    accumulate = 1u;
                    tc5_commit(&empty_a[sa]);
                }
            };
            if (a.exact == 2) issue_all(std::integral_constant<int, 2>{});
            else if (a.exact == 1) issue_all(std::integral_constant<int, 1>{});
            else issue_all(std::integral_constant<int, 0>{});
            tc5_commit(&done_bar);  // arrives when every MMA above has completed
        }
    } else if (lane == 0) {
        // ── TMA: per chunk the activation tile as two boxes of (64 columns x nb_max rows), counted in bytes on `full_b` ──
        // exact == 1: a stage is the chunk's two tiles (leading parts, then remainders: rows m0 + m ..), twice stage_bytes.
        // exact == 2: a stage is 64 columns of the chunk — the leading parts' box and the remainders' box — two hand-overs
        // per chunk, so that 256-row tiles still have a ring of three stages.
        const int per_chunk = a.exact == 2 ? 2 : 1;
        const int b_bytes = a.exact == 1 ? 2 * a.stage_bytes : a.stage_bytes;
        for (int h = 0, sb = 0, ub = 0; h < n_chunks * per_chunk; ++h, ++sb) {
            const int c = a.exact == 2 ? (h >> 1) : h, half = a.exact == 2 ? (h & 1) : 0;
            if (sb == a.stages) { sb = 0; ++ub; }
            if (ub > 0) ok = ok && tc5_wait(&empty_b[sb], (uint32_t)((ub - 1) & 1));
            const uint32_t bar = tc5_smem_u32(&full_b[sb]);
            const uint32_t dst = tc5_smem_u32(smem + (size_t)sb * b_bytes);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(b_bytes) : "memory");
            for (int bx = 0; bx < (a.exact == 1 ? 4 : 2); ++bx) {
                // plain: the chunk's two 64-column boxes; exact 1: the same for both row planes; exact 2: one 64-column box
                // of each row plane
                const int plane = a.exact == 1 ? (bx >> 1) : a.exact == 2 ? bx : 0;
                const int colbox = a.exact == 2 ? half : (bx & 1);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                        dst + bx * (a.stage_bytes / 2)),
                    "l"(&tmap_x), "r"((c_begin + c) * TC5_BK + 64 * colbox), "r"(m0 + plane * a.m), "r"(bar)
                    : "memory");
            }
        }
    }
    if (pw >= 0) {
        // ── epilogue, by the producers once their last chunk is handed over: warp w reads TMEM lanes 32 (w % 4) .. +31
        //    (= weight rows), 16 columns (= activation rows) at a time, column groups pw / 4, pw / 4 + 4, .. ──
        __syncwarp();
        ok = ok && tc5_wait(&done_bar, 0u);
        ok = __all_sync(0xFFFFFFFFu, ok);  // one verdict for the warp: the loads below are warp-collective
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const int q4 = warp & 3;
        const int n = n0 + 32 * q4 + lane;
        float* const pbuf = parts > 1 ? a.split_buf + ((size_t)(item - a.full_items) * parts + part) * (size_t)(TC5_NB_MAX * TC5_BM) : nullptr;
        if (ok) {
            const float bias = (sg.bias && n < sg.n && part == 0) ? sg.bias[n] : 0.f;
            const bool add_res = a.res && si == 0 && parts == 1;
            float* yb = sg.y;
            for (int gi = pw >> 2; gi < nb / 16; gi += TC5_PRODUCER_WARPS / 4) {
                uint32_t r[16];
                const uint32_t taddr = tmem + ((uint32_t)(32 * q4) << 16) + (uint32_t)(gi * 16);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (parts > 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + gi * 16 + j;
                        const float sc = (a.xscale && m < a.m) ? a.xscale[m] : 1.f;
                        pbuf[(gi * 16 + j) * TC5_BM + 32 * q4 + lane] = fmaf(__uint_as_float(r[j]), sc, bias);
                    }
                } else if (n < sg.n) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + gi * 16 + j;
                        if (m < a.m) {
                            float v = a.xscale ? fmaf(__uint_as_float(r[j]), a.xscale[m], bias) : __uint_as_float(r[j]) + bias;
                            if (add_res) v += a.res[(int64_t)m * a.ldres + n];
                            yb[(int64_t)m * a.ldy + n] = v;
                        }
                    }
                }
            }
        }
        if (parts > 1) {
            // Every producer warp comes here whatever its `ok` (the named barrier counts all 16 warps). The last CTA
            // of the item to arrive sums the parts in part order: no CTA ever waits for another.
            __threadfence();
            asm volatile("bar.sync 1, %0;\n" ::"r"(TC5_PRODUCER_WARPS * 32) : "memory");
            if (pw == 0 && lane == 0) split_last = atomicAdd(&a.split_cnt[item - a.full_items], 1u) == (unsigned)(parts - 1);
            asm volatile("bar.sync 1, %0;\n" ::"r"(TC5_PRODUCER_WARPS * 32) : "memory");
            if (split_last) {
                __threadfence();
                const float* all = a.split_buf + (size_t)(item - a.full_items) * parts * (size_t)(TC5_NB_MAX * TC5_BM);
                const bool in_place = a.res && si == 0;  // y holds the residual (the launcher splits only when res == y)
                for (int idx = pw * 32 + lane; idx < nb * TC5_BM; idx += TC5_PRODUCER_WARPS * 32) {
                    const int mm = idx / TC5_BM, nn = idx - mm * TC5_BM;
                    const int m = m0 + mm, nrow = n0 + nn;
                    if (m < a.m && nrow < sg.n) {
                        float v = in_place ? sg.y[(int64_t)m * a.ldy + nrow] : 0.f;
                        for (int p2 = 0; p2 < parts; ++p2) v += __ldcg(all + (size_t)p2 * (TC5_NB_MAX * TC5_BM) + idx);
                        sg.y[(int64_t)m * a.ldy + nrow] = v;
                    }
                }
                if (pw == 0 && lane == 0) a.split_cnt[item - a.full_items] = 0u;  // ready for the next launch
            }
        }
    }
    if (!ok) atomicExch(&g_tc5_timeout, 1);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == TC5_MMA_WARP) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TC5_TMEM_COLS) : "memory");
}

// x[m, k] f32 -> fp16, one thread per 8 columns.
__global__ void x_to_f16_kernel(const float* __restrict__ x, int ldx, int k, __half* __restrict__ out, int64_t total8) {
    pdl_wait();
    pdl_trigger();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = k / 8;
    const int64_t m = i / per_row;
    const int c = (int)(i - m * per_row) * 8;
    const float4 p0 = *reinterpret_cast<const float4*>(x + m * ldx + c), p1 = *reinterpret_cast<const float4*>(x + m * ldx + c + 4);
    *reinterpret_cast<uint4*>(out + m * k + c) =
        make_uint4(pack_h2(p0.x, p0.y), pack_h2(p0.z, p0.w), pack_h2(p1.x, p1.y), pack_h2(p1.z, p1.w));
}

// Row m of x[m, k] (f32), scaled by the power of two that brings it into (-1, 1): out[m] = fp16 leading parts,
// out[m_rows + m] = fp16 of what the first rounding dropped, rowscale[m] = the inverse of the scale. One block per row.
__global__ void __launch_bounds__(256) x_to_f16_hilo_kernel(const float* __restrict__ x, int ldx, int k, int m_rows, __half* __restrict__ out,
                                                            float* __restrict__ rowscale) {
    __shared__ float sh[8];
    pdl_wait();
    pdl_trigger();
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = x + (int64_t)m * ldx;
    float amax = 0.f;
    for (int c = threadIdx.x * 8; c < k; c += 256 * 8) {
        const float4 p0 = *reinterpret_cast<const float4*>(row + c), p1 = *reinterpret_cast<const float4*>(row + c + 4);
        amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(p0.x), fabsf(p0.y)), fmaxf(fabsf(p0.z), fabsf(p0.w))),
                                 fmaxf(fmaxf(fabsf(p1.x), fabsf(p1.y)), fmaxf(fabsf(p1.z), fabsf(p1.w)))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (lane == 0) sh[warp] = amax;
    __syncthreads();
    amax = sh[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, sh[w]);
    float up = 1.f, down = 1.f;
    if (amax > 0.f && amax < INFINITY) {
        const int e = max(-100, min(100, ilogbf(amax) + 1));  // amax < 2^e
        up = scalbnf(1.0f, -e);
        down = scalbnf(1.0f, e);
    }
    if (threadIdx.x == 0) rowscale[m] = down;
    for (int c = threadIdx.x * 8; c < k; c += 256 * 8) {
        const float4 p0 = *reinterpret_cast<const float4*>(row + c), p1 = *reinterpret_cast<const float4*>(row + c + 4);
        const float v[8] = {p0.x * up, p0.y * up, p0.z * up, p0.w * up, p1.x * up, p1.y * up, p1.z * up, p1.w * up};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
            hi[j] = bits_h2(h);
            lo[j] = bits_h2(__floats2half2_rn(v[2 * j] - __low2float(h), v[2 * j + 1] - __high2float(h)));
        }
        *reinterpret_cast<uint4*>(out + (int64_t)m * k + c) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(out + ((int64_t)m + m_rows) * k + c) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// Reads and clears the flag a bounded mbarrier wait of gemm_tc5_kernel raises when it runs out (the kernel then skips
// its epilogue, so y is stale). Synchronous copy from the device the calling thread has current: call it only where
// the stream has been synchronised already. 1 = a wait expired since the last call, 0 = none, -1 = CUDA error.
static std::atomic<int> g_tc5_launched[SP_MAX_DEVICES];  // per device: a launch has happened since the flag was last read
int tc5_take_timeout() {
    if (g_tc5_launched[current_device_index()].exchange(0) == 0) return 0;
    int flag = 0;
    if (cudaMemcpyFromSymbol(&flag, g_tc5_timeout, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (flag) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc5_timeout, &zero, sizeof(int));
    }
    return flag ? 1 : 0;
}

bool tc5_supported(int dtype, int64_t k) {
    if (dtype == T_Q8_0) return k % 128 == 0;  // the tiling switches to four blocks per tile when k is not a multiple of 256
    return k % 256 == 0 && (dtype == T_Q4_K || dtype == T_Q6_K);
}

cudaError_t launch_x_to_f16(const float* x, int ldx, int m, int k, __half* out, cudaStream_t st) {
    if (m <= 0) return cudaSuccess;
    const int64_t total8 = (int64_t)m * k / 8;
    cudaError_t le = launch_pdl(x_to_f16_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, st, x, ldx, k, out, total8);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_x_to_f16_hilo(const float* x, int ldx, int m, int k, __half* out, float* rowscale, cudaStream_t st) {
    if (m <= 0) return cudaSuccess;
    if (k % 8 != 0 || !rowscale) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(x_to_f16_hilo_kernel, dim3((unsigned)m), dim3(256), 0, st, x, ldx, k, m, out, rowscale);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Up to three matrices sharing the activations in one launch. res (added to segment 0) may alias its y. The items of the
// grid's last, partial wave are split along K over as many CTAs as fill the SMs (see Tc5Args) when the caller provides
// scratch for their partial tiles, unless there is a residual that is not in place.

cudaError_t Tc5Scratch::alloc() {
    release();
    parts_cap = (size_t)device_sm_count();
    cudaError_t e = cudaMalloc((void**)&buf, parts_cap * TC5_NB_MAX * TC5_BM * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&cnt, TC5_SPLIT_MAX_ITEMS * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(cnt, 0, TC5_SPLIT_MAX_ITEMS * sizeof(unsigned));
    if (e != cudaSuccess) release();
    return e;
}

void Tc5Scratch::release() {
    if (buf) cudaFree(buf);
    if (cnt) cudaFree(cnt);
    buf = nullptr; cnt = nullptr; parts_cap = 0;
}

cudaError_t launch_gemm_tc5_multi(const Tc5Seg* segs, int nseg, int k, const __half* xh, int m, int ldy, const float* res, int ldres,
                                  cudaStream_t st, const Tc5Scratch* scratch, const float* xscale) {
    if (m <= 0 || nseg <= 0) return cudaSuccess;
    const bool exact = xscale != nullptr;
    if (nseg > 3 || k % 128 != 0) return cudaErrorInvalidValue;
    Tc5Args a{};
    int tiles = 0;
    for (int i = 0; i < nseg; ++i) {
        if (!tc5_supported(segs[i].dtype, k) || segs[i].n <= 0) return cudaErrorInvalidValue;
        a.seg[i] = segs[i];
        tiles += (segs[i].n + TC5_BM - 1) / TC5_BM;
    }
    static PerDeviceOnce attr_once;
    const int sm_count = device_sm_count();
    const int nb_max = std::min(TC5_NB_MAX, (m + 15) & ~15);
    const int stage_bytes = nb_max * 256;
    // exact-class operands: whole-chunk activation stages (two tiles) while at least three fit, else half-chunk stages
    const int exact_mode = !xscale ? 0 : (TC5_SMEM_LIMIT / (2 * stage_bytes) >= 3 ? 1 : 2);
    const int b_stage_bytes = exact_mode == 1 ? 2 * stage_bytes : stage_bytes;
    const int stages = std::min(TC5_MAX_STAGES, TC5_SMEM_LIMIT / b_stage_bytes);
    const int smem_bytes = std::max(stages * b_stage_bytes + 1024, TC5_SMEM_MIN);  // + slack to align the stages to 1024 B
    const int m_tiles = (m + TC5_NB_MAX - 1) / TC5_NB_MAX;
    const int chunks = k / TC5_BK, items = tiles * m_tiles;
    int full_items = items, tail_split = 1;
    const bool in_place = nseg == 1 && res && res == segs[0].y;
    if ((!res || in_place) && scratch && scratch->buf && scratch->cnt) {
        int tail = items % sm_count;
        if (tail > 0) {
            int first = (items - tail) / m_tiles * m_tiles;  // whole weight tiles only
            tail = items - first;
            const int ts = std::min({8, sm_count / tail, chunks / 4});  // (chunks of K: a split part keeps at least four)
            if (ts >= 2 && tail <= TC5_SPLIT_MAX_ITEMS && (size_t)tail * ts <= scratch->parts_cap) { full_items = first; tail_split = ts; }
        }
    }
    // TMA descriptor of the fp16 activations [m][k]: boxes of 64 columns x nb_max rows, 128-byte swizzle, zero fill
    static const PFN_encodeTiled encode = [] {  // initialised once, thread-safe
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess) fn = nullptr;
        return reinterpret_cast<PFN_encodeTiled>(fn);
    }();
    if (!encode) return cudaErrorNotSupported;
    CUtensorMap tmap;
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)(exact ? 2 * m : m)};
        const cuuint64_t gstride[1] = {(cuuint64_t)k * sizeof(__half)};
        const cuuint32_t box[2] = {64u, (cuuint32_t)nb_max};
        const cuuint32_t estr[2] = {1u, 1u};
        if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xh), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    a.nseg = nseg; a.k = k; a.xh = xh; a.m = m; a.ldy = ldy; a.res = res; a.ldres = ldres;
    a.m_tiles = m_tiles; a.full_items = full_items; a.tail_split = tail_split;
    a.stage_bytes = stage_bytes; a.stages = stages;
    a.exact = exact_mode;
    a.xscale = xscale;
    constexpr int SMEM_CAP = TC5_SMEM_LIMIT + 1024;
    cudaError_t le;
    le = attr_once.run([] { return cudaFuncSetAttribute(gemm_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_CAP); });
    if (le != cudaSuccess) return le;
    if (tail_split > 1) { a.split_buf = scratch->buf; a.split_cnt = scratch->cnt; }
    const int grid = full_items + (items - full_items) * tail_split;
    g_tc5_launched[current_device_index()].store(1);
    le = launch_pdl(gemm_tc5_kernel, dim3((unsigned)grid), dim3(TC5_THREADS), smem_bytes, st, a, tmap);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_gemm_tc5(const uint8_t* wt, int dtype, int n, int k, const __half* xh, int m, float* y, int ldy, const float* bias,
                            const float* res, int ldres, cudaStream_t st, const Tc5Scratch* scratch, const float* xscale) {
    Tc5Seg sg{wt, y, bias, dtype, n};
    return launch_gemm_tc5_multi(&sg, 1, k, xh, m, ldy, res, ldres, st, scratch, xscale);
}

}  // namespace sp
