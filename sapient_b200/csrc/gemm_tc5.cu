// Large-M dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for prefill and batched decode.
//
// y[m, n] = sum_k x[m, k] * W[n, k] for m >= 64 activation rows. The GEMV kernel (gemv_imma.cu) streams the whole
// weight matrix once per 16 activation rows; here a CTA dequantises each weight tile ONCE and multiplies it with up to
// 256 activation rows:
//   * CTA tile: 128 weight rows (the MMA's M) x NB <= 256 activation rows (the MMA's N), K walked in chunks of 64;
//   * per chunk the 512 threads rebuild 128 x 64 weights from the tile-repacked ggml blocks (the same layout the GEMV
//     reads, gemv_imma.cuh) — exact f32 dequantisation, rounded once to fp16 — into shared memory in the K-major
//     128-byte-swizzled layout the tensor core reads, and copy the matching 64 columns of the fp16 activations; the
//     global loads of the next chunk are issued into registers before the current one is handed to the tensor core;
//   * one thread issues four tcgen05.mma (128 x NB x 16, kind::f16, fp32 accumulation in tensor memory) and commits
//     them to an mbarrier; two shared-memory stages let the next chunk be rebuilt while the MMAs run;
//   * epilogue: tcgen05.ld brings the accumulators back (one weight row per thread, 16 activation rows per
//     instruction), bias / residual are added and y is written with n contiguous across the warp.
// fp16 rather than bf16 operands: same instruction kind and rate, and the 11-bit significand keeps the result
// within 2e-4 relative L2 of the f32 reference (bf16 would sit at ~2e-3, above the 1e-3 parity bar).
// Every wait on an mbarrier is bounded; on expiry the kernel raises g_tc5_timeout, still frees its tensor memory
// and returns.
#include <cuda_fp16.h>

#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

constexpr int TC5_THREADS = 512;
constexpr int TC5_BM = 128;                    // weight rows per CTA
constexpr int TC5_BK = 64;                     // columns per chunk = one 128-byte swizzle row of fp16
constexpr int TC5_NB_MAX = 256;                // activation rows per CTA
constexpr int TC5_A_BYTES = TC5_BM * 128;      // 16 KB
constexpr int TC5_B_BYTES = TC5_NB_MAX * 128;  // 32 KB
constexpr int TC5_STAGE_BYTES = TC5_A_BYTES + TC5_B_BYTES;
constexpr int TC5_SMEM = 2 * TC5_STAGE_BYTES + 1024;  // + slack to align the stages to 1024 B
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

// The raw words one thread needs for 16 consecutive columns — sixteenth-block (hh, h16) of 64-column group cq — of weight
// row rr of a 16-row tile: fetched one chunk ahead (tc5_load), turned into f32 weights when the stage is free
// (tc5_compute). hh selects the 32-column sub-block (low / high nibbles), h16 its first or second 16 columns.
struct Tc5Raw {
    uint32_t w[8];  // Q4_K / Q8_0: 4 words of nibbles / int8; Q6_K: 4 ql words + 4 qh words
    uint4 hdr;      // Q4_K: d|dmin, 12 scale bytes; Q6_K: x = int8 scale, y = d bits; Q8_0: x = d bits
};

template <int DT>
__device__ __forceinline__ void tc5_load(const uint8_t* tile, int rr, int cq, int hh, int h16, Tc5Raw& r) {
    const int g = rr & 7, hi8 = rr >> 3;
    const uint32_t* w32 = reinterpret_cast<const uint32_t*>(tile);
    if (DT == T_Q4_K) {
        r.hdr = __ldg(reinterpret_cast<const uint4*>(tile + 2048 + rr * 16));
#pragma unroll
        for (int t = 0; t < 4; ++t) r.w[t] = __ldg(w32 + cq * 128 + (g * 4 + t) * 4 + hi8 * 2 + h16);
    } else if (DT == T_Q8_0) {
        const int bb = 2 * cq + hh;
        r.hdr.x = __ldg(reinterpret_cast<const uint16_t*>(tile + 4096 + (rr * 8 + bb) * 2));
#pragma unroll
        for (int t = 0; t < 4; ++t) r.w[t] = __ldg(w32 + bb * 128 + (g * 4 + t) * 4 + hi8 * 2 + h16);
    } else {  // Q6_K: h16 is p of the block layout (l = 16 p + 4 t + b)
        const int half = cq >> 1, quarter = 2 * (cq & 1) + hh;
        const int8_t* scales = reinterpret_cast<const int8_t*>(tile + 3072 + rr * 16);
        r.hdr.x = (uint32_t)(uint8_t)__ldg(scales + 8 * half + h16 + 2 * quarter);
        r.hdr.y = __ldg(reinterpret_cast<const uint16_t*>(tile + 3328 + rr * 2));
        const int cc = (half << 1) | h16;
        const int sl = 6 * cc + (hh ? 1 : 0) + hi8 * 3, sh = 6 * cc + 2 + hi8 * 3;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            r.w[t] = __ldg(w32 + (sl >> 2) * 128 + (g * 4 + t) * 4 + (sl & 3));
            r.w[4 + t] = __ldg(w32 + (sh >> 2) * 128 + (g * 4 + t) * 4 + (sh & 3));
        }
    }
}

// Exact f32 dequantisation (every product rounded separately, as the reference does) of the 16 columns.
template <int DT>
__device__ __forceinline__ void tc5_compute(const Tc5Raw& r, int cq, int hh, float (&v)[16]) {
    if (DT == T_Q4_K) {
        const float d = half_bits_to_float((uint16_t)(r.hdr.x & 0xFFFFu)), dmin = half_bits_to_float((uint16_t)(r.hdr.x >> 16));
        uint32_t sc, mn;
        k4_scale_min(r.hdr.y, r.hdr.z, r.hdr.w, 2 * cq + hh, &sc, &mn);
        const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (r.w[t] >> (8 * b)) & 0xFFu;
                const float q = (float)(hh ? (byte >> 4) : (byte & 15u));
                v[4 * t + b] = __fsub_rn(__fmul_rn(dl, q), ml);
            }
    } else if (DT == T_Q8_0) {
        const float d = half_bits_to_float((uint16_t)r.hdr.x);
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int b = 0; b < 4; ++b) v[4 * t + b] = __fmul_rn((float)(int8_t)((r.w[t] >> (8 * b)) & 0xFFu), d);
    } else {  // Q6_K
        const int quarter = 2 * (cq & 1) + hh;
        const float dsc = __fmul_rn(half_bits_to_float((uint16_t)r.hdr.y), (float)(int8_t)(r.hdr.x & 0xFFu));
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t lb = (r.w[t] >> (8 * b)) & 0xFFu, hb = (r.w[4 + t] >> (8 * b)) & 0xFFu;
                const uint32_t nib = (cq & 1) ? (lb >> 4) : (lb & 15u);
                const int q = (int)(nib | (((hb >> (2 * quarter)) & 3u) << 4)) - 32;
                v[4 * t + b] = __fmul_rn(dsc, (float)q);
            }
    }
}

struct Tc5Args {
    const uint8_t* wt;  // tiled weights
    int dtype, n, k;    // n rows, k columns (k % 256 == 0)
    const __half* xh;   // activations as fp16 [m][k]
    int m;
    float* y;
    int ldy;
    const float* bias;  // [n] or null
    const float* res;   // [m][ldres] or null (may alias y)
    int ldres;
};

template <int DT>
__global__ void __launch_bounds__(TC5_THREADS, 1) gemm_tc5_kernel(const Tc5Args a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t mbar[2];
    __shared__ uint32_t tmem_slot;
    constexpr int TILE_BYTES = DT == T_Q4_K ? Q4_K_TILE_BYTES : DT == T_Q6_K ? Q6_K_TILE_BYTES : 8 * 544;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* smem = smem_raw + ((1024u - (tc5_smem_u32(smem_raw) & 1023u)) & 1023u);
    const int n0 = blockIdx.x * TC5_BM, m0 = blockIdx.y * TC5_NB_MAX;
    const int rows_here = min(TC5_NB_MAX, a.m - m0);
    const int nb = (rows_here + 15) & ~15;                       // the MMA's N
    const int tmem_cols = nb <= 32 ? 32 : nb <= 64 ? 64 : nb <= 128 ? 128 : 256;
    const int kts = a.k >> 8, n_tile_rows = (a.n + 15) >> 4;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5_smem_u32(&tmem_slot)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&mbar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5_smem_u32(&mbar[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_wait();  // activations come from the previous kernel
    pdl_trigger();

    const int row = tid >> 2, hh = (tid >> 1) & 1, h16 = tid & 1;  // this thread's weight row of the tile and 16-column slice
    const int rt = (n0 >> 4) + (row >> 4), rr = row & 15;
    const bool row_live = rt < n_tile_rows;
    const uint8_t* tile_row = a.wt + (int64_t)rt * kts * TILE_BYTES;
    const uint32_t idesc = tc5_idesc(nb);
    const int n_chunks = a.k / TC5_BK;
    bool ok = true;
    constexpr int B_PER_THREAD = TC5_NB_MAX * 8 / TC5_THREADS;  // 16-byte pieces of the activation tile per thread
    Tc5Raw raw;
    uint4 braw[B_PER_THREAD];
    auto fetch = [&](int c) {  // global loads of chunk c into registers
        if (row_live) tc5_load<DT>(tile_row + (int64_t)(c >> 2) * TILE_BYTES, rr, c & 3, hh, h16, raw);
#pragma unroll
        for (int i = 0; i < B_PER_THREAD; ++i) {
            const int idx = tid + i * TC5_THREADS, r = idx >> 3, ch = idx & 7;
            braw[i] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < nb * 8 && m0 + r < a.m)
                braw[i] = __ldg(reinterpret_cast<const uint4*>(a.xh + (int64_t)(m0 + r) * a.k + (int64_t)c * TC5_BK + ch * 8));
        }
    };
    fetch(0);
    for (int c = 0; c < n_chunks; ++c) {
        const int s = c & 1;
        uint8_t* As = smem + s * TC5_STAGE_BYTES;
        uint8_t* Bs = As + TC5_A_BYTES;
        if (c >= 2) ok = tc5_wait(&mbar[s], (uint32_t)(((c >> 1) - 1) & 1)) && ok;  // the MMAs of chunk c - 2 have read this stage
        // A: 16 dequantised weights of this thread's row, rounded to fp16, into the swizzled K-major tile
        {
            float v[16];
            if (row_live) tc5_compute<DT>(raw, c & 3, hh, v);
            else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const uint4 q = make_uint4(pack_h2(v[8 * p], v[8 * p + 1]), pack_h2(v[8 * p + 2], v[8 * p + 3]),
                                           pack_h2(v[8 * p + 4], v[8 * p + 5]), pack_h2(v[8 * p + 6], v[8 * p + 7]));
                const int chunk16 = 4 * hh + 2 * h16 + p;
                *reinterpret_cast<uint4*>(As + row * 128 + ((chunk16 ^ (row & 7)) << 4)) = q;
            }
        }
        // B: 64 columns of nb activation rows (fp16 already), 16 bytes per copy
#pragma unroll
        for (int i = 0; i < B_PER_THREAD; ++i) {
            const int idx = tid + i * TC5_THREADS, r = idx >> 3, ch = idx & 7;
            if (idx < nb * 8) *reinterpret_cast<uint4*>(Bs + r * 128 + ((ch ^ (r & 7)) << 4)) = braw[i];
        }
        if (c + 1 < n_chunks) fetch(c + 1);  // in flight while this chunk is fenced, multiplied and the stage wait runs
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy stores -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint64_t ad = tc5_desc(tc5_smem_u32(As)), bd = tc5_desc(tc5_smem_u32(Bs));
#pragma unroll
            for (int k = 0; k < TC5_BK / 16; ++k)  // 16 columns = 32 bytes further inside the swizzle row: +2 in units of 16 B
                tc5_mma(tmem, ad + 2 * k, bd + 2 * k, idesc, (c > 0 || k > 0) ? 1u : 0u);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc5_smem_u32(&mbar[s]))
                         : "memory");
        }
    }
    // all MMAs are committed in order: the last commit covers every earlier one
    {
        const int last = n_chunks - 1;
        ok = tc5_wait(&mbar[last & 1], (uint32_t)((last >> 1) & 1)) && ok;
    }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    ok = __syncthreads_and(ok);  // one verdict for the block: the loads below are warp-collective
    if (ok) {
        // warp w reads TMEM lanes 32 (w % 4) .. +31 (= weight rows), 16 columns (= activation rows) per instruction
        const int q4 = warp & 3;
        const int n = n0 + 32 * q4 + lane;
        const float bias = (a.bias && n < a.n) ? a.bias[n] : 0.f;
        for (int gi = warp >> 2; gi < nb / 16; gi += TC5_THREADS / 128) {
            uint32_t r[16];
            const uint32_t taddr = tmem + ((uint32_t)(32 * q4) << 16) + (uint32_t)(gi * 16);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                  "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (n < a.n) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = m0 + gi * 16 + j;
                    if (m < a.m) {
                        float v = __uint_as_float(r[j]) + bias;
                        if (a.res) v += a.res[(int64_t)m * a.ldres + n];
                        a.y[(int64_t)m * a.ldy + n] = v;
                    }
                }
            }
        }
    } else if (tid == 0) {
        atomicExch(&g_tc5_timeout, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols) : "memory");
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

bool tc5_supported(int dtype, int64_t k) { return k % 256 == 0 && (dtype == T_Q4_K || dtype == T_Q6_K || dtype == T_Q8_0); }

cudaError_t launch_x_to_f16(const float* x, int ldx, int m, int k, __half* out, cudaStream_t st) {
    if (m <= 0) return cudaSuccess;
    const int64_t total8 = (int64_t)m * k / 8;
    cudaError_t le = launch_pdl(x_to_f16_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, st, x, ldx, k, out, total8);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

cudaError_t launch_gemm_tc5(const uint8_t* wt, int dtype, int n, int k, const __half* xh, int m, float* y, int ldy, const float* bias,
                            const float* res, int ldres, cudaStream_t st) {
    if (m <= 0 || n <= 0) return cudaSuccess;
    if (!tc5_supported(dtype, k)) return cudaErrorInvalidValue;
    static bool attr_set[3] = {false, false, false};
    Tc5Args a{wt, dtype, n, k, xh, m, y, ldy, bias, res, ldres};
    const dim3 grid((unsigned)((n + TC5_BM - 1) / TC5_BM), (unsigned)((m + TC5_NB_MAX - 1) / TC5_NB_MAX));
    cudaError_t le;
    const int which = dtype == T_Q4_K ? 0 : dtype == T_Q6_K ? 1 : 2;
    if (!attr_set[which]) {
        le = which == 0   ? cudaFuncSetAttribute(gemm_tc5_kernel<T_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC5_SMEM)
             : which == 1 ? cudaFuncSetAttribute(gemm_tc5_kernel<T_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC5_SMEM)
                          : cudaFuncSetAttribute(gemm_tc5_kernel<T_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC5_SMEM);
        if (le != cudaSuccess) return le;
        attr_set[which] = true;
    }
    if (which == 0) le = launch_pdl(gemm_tc5_kernel<T_Q4_K>, grid, dim3(TC5_THREADS), TC5_SMEM, st, a);
    else if (which == 1) le = launch_pdl(gemm_tc5_kernel<T_Q6_K>, grid, dim3(TC5_THREADS), TC5_SMEM, st, a);
    else le = launch_pdl(gemm_tc5_kernel<T_Q8_0>, grid, dim3(TC5_THREADS), TC5_SMEM, st, a);
    if (le != cudaSuccess) return le;
    return count_launch_and_check();
}

}  // namespace sp
