// Tensor-core GEMV for 11 to 32 activation rows in ONE pass over the weights (exact integer products, three digits).
//
// The tile-row kernel (gemv_imma.cu) gives a CTA one 16-row tile row and lets its warps split the k-tiles, so every warp
// needs its own activation digits and fetches them from L2 into registers: fine for a few rows, but at 10 rows per pass
// a 32-row step streams the weights four times and waits on ~90 dependent L2 loads per tile. Here the roles are turned
// round: a CTA owns EIGHT tile rows (128 weight rows, one per warp) and walks the k-tiles of its K range together, so
// the digits of a k-tile — up to 96 columns x 256 bytes — are staged once per CTA in shared memory (cp.async, double
// buffered) and read by all eight warps, while each warp keeps its weight tile in registers (the next one prefetched)
// and reuses it for every 32-column group of digits. The per-tile arithmetic is the tile-row kernel's
// (gemv_imma_dev.cuh: compute_q4_k / compute_q6_k / compute_q8_0 on four n-tiles at a time), so results differ from the
// pass-wise path only by the order in which the k-tiles of a row are added.
//
// Small matrices do not have enough 128-row groups to fill the GPU: K is then split over several CTAs per group, which
// write their partial [rows x 128] blocks to scratch; the CTA that arrives last adds them in split order (same bits
// every run) and finishes the rows (bias, residual).
#include <cuda_runtime.h>

#include "gemv_imma_dev.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu

constexpr int ROWS_WARPS = 8;          // tile rows per CTA
constexpr int ROWS_COL_BYTES = 272;    // one digit column of a k-tile in shared memory: 256 + 16, so the eight columns of an n-tile do not share banks
constexpr int ROWS_MAX_GROUPS = 3;     // 32-column groups of digits: 96 columns = 32 rows x 3 digits

struct RowsArgs {
    ImmaArgs a;        // one segment (a.seg[0]); digits planned for a.m rows with a.eb == 256
    int groups;        // ceil(a.m * a.digits / 32)
    int splits;        // CTAs per 128-row group along K
    int kts_per_split;
    float* part;       // [splits][a.m][n] partial outputs (splits > 1)
    unsigned* cnt;     // [row groups] arrival counters, zero between launches
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}

// Stage layout: digits [ncp][272 B] | xs32d records [ncp][32 B] | xs16d records [ncp][32 B] | column scales [ncp] f32
__host__ __device__ inline int rows_stage_bytes(int ncp) { return ncp * (ROWS_COL_BYTES + 32 + 32 + 4); }

template <int FMT>
struct RowsTile;  // register image of one weight tile per format
template <> struct RowsTile<T_Q4_K> { Q4Regs r; };
template <> struct RowsTile<T_Q6_K> { Q6Regs r; };
template <> struct RowsTile<T_Q8_0> { Q8Regs r; };

template <int FMT>
__device__ __forceinline__ int rows_tile_bytes() { return FMT == T_Q4_K ? Q4_K_TILE_BYTES : FMT == T_Q6_K ? Q6_K_TILE_BYTES : 8 * 544; }

template <int FMT>
__device__ __forceinline__ void rows_load(const uint8_t* tile, int lane, RowsTile<FMT>& w) {
    if constexpr (FMT == T_Q4_K) load_q4_k<true>(tile, lane, w.r);
    else if constexpr (FMT == T_Q6_K) load_q6_k<true>(tile, lane, w.r);
    else load_q8_0<true>(tile, lane, w.r);
}

template <int FMT>
__device__ __forceinline__ void rows_compute(const RowsTile<FMT>& w, const BFrag<4>& b, int lane, float (&acc)[4][4]) {
    if constexpr (FMT == T_Q4_K) compute_q4_k<4>(w.r, b, lane, acc);
    else if constexpr (FMT == T_Q6_K) compute_q6_k<4>(w.r, b, lane, acc);
    else compute_q8_0<4>(w.r, b, acc);
}

template <int FMT, int G>
__global__ void __launch_bounds__(ROWS_WARPS * 32, 1) gemv_rows_kernel(const RowsArgs p) {
    extern __shared__ __align__(16) uint8_t rows_smem[];
    __shared__ int sh_last;
    const ImmaArgs& a = p.a;
    const ImmaSeg& sg = a.seg[0];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n_tiles = (sg.n + 15) / 16;
    const int rt = blockIdx.x * ROWS_WARPS + warp;
    const bool live = rt < n_tiles;
    const int KT = a.k >> 8;
    const int kt0 = blockIdx.y * p.kts_per_split, kt1 = min(KT, kt0 + p.kts_per_split);
    const int ncp = a.ncp, cols = a.m * a.digits;
    const int stage_bytes = rows_stage_bytes(ncp);
    const int tb = rows_tile_bytes<FMT>();
    const uint8_t* wbase = sg.wt + (int64_t)(live ? rt : 0) * KT * tb;

    float acc[G][4][4];
#pragma unroll
    for (int c = 0; c < G; ++c)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) acc[c][nt][0] = acc[c][nt][1] = acc[c][nt][2] = acc[c][nt][3] = 0.f;

    RowsTile<FMT> wa, wb;
    if (live && kt0 < kt1) rows_load<FMT>(wbase + (int64_t)kt0 * tb, lane, wa);  // weights do not depend on the producer
    pdl_wait();
    pdl_trigger();

    auto fetch = [&](int kt, int buf) {
        uint8_t* st = rows_smem + (size_t)buf * stage_bytes;
        // digits: 16 chunks of 16 bytes per column; columns past the live ones arrive as zeros
        for (int idx = threadIdx.x; idx < ncp * 16; idx += ROWS_WARPS * 32) {
            const int col = idx >> 4, ch = idx & 15;
            cp_async16(st + col * ROWS_COL_BYTES + ch * 16, a.xq + (int64_t)col * a.kp + (int64_t)kt * 256 + ch * 16, col < cols ? 16 : 0);
        }
        uint8_t* r32 = st + ncp * ROWS_COL_BYTES;
        uint8_t* r16 = r32 + ncp * 32;
        uint8_t* cs = r16 + ncp * 32;
        for (int idx = threadIdx.x; idx < ncp * 2; idx += ROWS_WARPS * 32) {
            cp_async16(r32 + idx * 16, a.xs32d + ((int64_t)kt * ncp) * 32 + idx * 16, 16);
            cp_async16(r16 + idx * 16, a.xs16d + ((int64_t)kt * ncp) * 32 + idx * 16, 16);
        }
        for (int idx = threadIdx.x; idx < ncp / 4; idx += ROWS_WARPS * 32)
            cp_async16(cs + idx * 16, a.colscale + (int64_t)kt * ncp + idx * 4, 16);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    if (kt0 < kt1) fetch(kt0, 0);
    for (int kt = kt0, buf = 0; kt < kt1; ++kt, buf ^= 1) {
        if (kt + 1 < kt1) {
            fetch(kt + 1, buf ^ 1);  // that stage was consumed before the barrier that ended the last iteration
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        if (live) {
            if (kt + 1 < kt1) rows_load<FMT>(wbase + (int64_t)(kt + 1) * tb, lane, wb);
            const uint8_t* st = rows_smem + (size_t)buf * stage_bytes;
            const uint8_t* r32 = st + ncp * ROWS_COL_BYTES;
            const uint8_t* r16 = r32 + ncp * 32;
            const float* cs = reinterpret_cast<const float*>(r16 + ncp * 32);
#pragma unroll
            for (int c = 0; c < G; ++c) {
                BFrag<4> b;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int col = c * 32 + nt * 8 + g;
                    const uint8_t* dcol = st + col * ROWS_COL_BYTES + t * 64;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = *reinterpret_cast<const uint4*>(dcol + 16 * i);
                        b.w[nt][4 * i] = v.x; b.w[nt][4 * i + 1] = v.y; b.w[nt][4 * i + 2] = v.z; b.w[nt][4 * i + 3] = v.w;
                    }
                    b.ra32[nt] = (FMT == T_Q4_K) ? *reinterpret_cast<const uint32_t*>(r32 + col * 32 + 4 * t) : 0u;
                    b.rb32[nt] = (FMT == T_Q4_K) ? *reinterpret_cast<const uint32_t*>(r32 + col * 32 + 16 + 4 * t) : 0u;
                    b.ra16[nt] = (FMT == T_Q6_K) ? *reinterpret_cast<const uint32_t*>(r16 + col * 32 + 4 * t) : 0u;
                    b.rb16[nt] = (FMT == T_Q6_K) ? *reinterpret_cast<const uint32_t*>(r16 + col * 32 + 16 + 4 * t) : 0u;
                    b.cs[nt] = *reinterpret_cast<const float2*>(cs + c * 32 + nt * 8 + 2 * t);
                }
                rows_compute<FMT>(wa, b, lane, acc[c]);
            }
            if (kt + 1 < kt1) wa = wb;
        }
        __syncthreads();  // the stage may be refilled from the next iteration on
    }

    // ── epilogue: digit columns of a row are added through shared memory (the stages are free now) ──
    float* sw = reinterpret_cast<float*>(rows_smem) + (size_t)warp * 16 * (G * 32 + 1);  // [16 rows][G * 32 + 1]
    constexpr int LDW = G * 32 + 1;
    if (live) {
#pragma unroll
        for (int c = 0; c < G; ++c)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int col = c * 32 + nt * 8 + 2 * t;
                sw[g * LDW + col] = acc[c][nt][0]; sw[g * LDW + col + 1] = acc[c][nt][1];
                sw[(g + 8) * LDW + col] = acc[c][nt][2]; sw[(g + 8) * LDW + col + 1] = acc[c][nt][3];
            }
    }
    __syncwarp();
    const int row0 = rt * 16;
    const int D = a.digits;
    if (p.splits == 1) {
        if (live)
            for (int idx = lane; idx < 16 * a.m; idx += 32) {
                const int r = idx & 15, m = idx >> 4, row = row0 + r;
                if (row < sg.n) {
                    float v = 0.f;
                    for (int d = 0; d < D; ++d) v += sw[r * LDW + m * D + d];
                    if (sg.bias) v += sg.bias[row];
                    if (a.res) v += a.res[(int64_t)m * a.ldres + row];
                    sg.y[(int64_t)m * sg.ldy + row] = v;
                }
            }
        return;
    }
    // K split over several CTAs: partial rows to scratch, the last CTA of the group adds them in split order
    if (live)
        for (int idx = lane; idx < 16 * a.m; idx += 32) {
            const int r = idx & 15, m = idx >> 4, row = row0 + r;
            if (row < sg.n) {
                float v = 0.f;
                for (int d = 0; d < D; ++d) v += sw[r * LDW + m * D + d];
                p.part[((int64_t)blockIdx.y * a.m + m) * sg.n + row] = v;
            }
        }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(p.cnt + blockIdx.x, 1u);
        sh_last = prev == (unsigned)p.splits - 1u;
        if (sh_last) {
            atomicExch(p.cnt + blockIdx.x, 0u);  // ready for the next launch (which starts after this grid)
            __threadfence();
        }
    }
    __syncthreads();
    if (!sh_last) return;
    const int rows_cta = min(ROWS_WARPS * 16, sg.n - (int)blockIdx.x * ROWS_WARPS * 16);
    for (int idx = threadIdx.x; idx < rows_cta * a.m; idx += ROWS_WARPS * 32) {
        const int r = idx % rows_cta, m = idx / rows_cta, row = blockIdx.x * ROWS_WARPS * 16 + r;
        float v = 0.f;
        for (int s = 0; s < p.splits; ++s) v += __ldcg(p.part + ((int64_t)s * a.m + m) * sg.n + row);
        if (sg.bias) v += sg.bias[row];
        if (a.res) v += a.res[(int64_t)m * a.ldres + row];
        sg.y[(int64_t)m * sg.ldy + row] = v;
    }
}

bool rows_supported(int dtype, int64_t k) {
    return (dtype == T_Q4_K || dtype == T_Q6_K || dtype == T_Q8_0) && k % 256 == 0;
}

size_t RowsScratch::part_floats() { return (size_t)4 << 20; }  // 16 MB: splits * rows * n of one segment launch must fit

cudaError_t RowsScratch::alloc() {
    release();
    cudaError_t e;
    if ((e = cudaMalloc((void**)&part, part_floats() * 4)) != cudaSuccess) return e;
    if ((e = cudaMalloc((void**)&cnt, CNT_MAX * 4)) != cudaSuccess) return e;
    return cudaMemset(cnt, 0, CNT_MAX * 4);
}

void RowsScratch::release() {
    if (part) cudaFree(part);
    if (cnt) cudaFree(cnt);
    part = nullptr;
    cnt = nullptr;
}

template <int FMT, int G>
static cudaError_t launch_rows_inst(const RowsArgs& p, dim3 grid, size_t smem, cudaStream_t st) {
    static PerDeviceOnce big_smem;
    cudaError_t e = big_smem.run([] { return cudaFuncSetAttribute(gemv_rows_kernel<FMT, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); });
    if (e != cudaSuccess) return e;
    return launch_pdl(gemv_rows_kernel<FMT, G>, grid, dim3(ROWS_WARPS * 32), smem, st, p);
}

// One launch per segment of `a` (each segment has one format). a.m <= 32 rows, digits planned with a.eb == 256.
cudaError_t launch_gemv_rows(const ImmaArgs& a, const RowsScratch& sc, cudaStream_t st) {
    if (a.m <= 0) return cudaSuccess;
    const int cols = a.m * a.digits;
    if (a.eb != 256 || a.k % 256 != 0 || cols > ROWS_MAX_GROUPS * 32 || a.ncp < cols || a.ncp % 32 != 0 || a.tp) return cudaErrorInvalidValue;
    const int sms = device_sm_count();
    const int KT = a.k >> 8;
    for (int s = 0; s < a.nseg; ++s) {
        RowsArgs p;
        p.a = a;
        p.a.seg[0] = a.seg[s];
        p.a.nseg = 1;
        if (s != 0) p.a.res = nullptr;  // the residual belongs to the first segment
        const ImmaSeg& sg = p.a.seg[0];
        if (!rows_supported(sg.dtype, a.k) || (sg.dtype == T_Q8_0 && sg.bpt != 8)) return cudaErrorInvalidValue;
        p.groups = (cols + 31) / 32;
        const int row_groups = ((sg.n + 15) / 16 + ROWS_WARPS - 1) / ROWS_WARPS;
        // one CTA per SM is resident (registers): split K until two waves are filled, at least two k-tiles per CTA
        int splits = 1;
        while (row_groups * splits < 2 * sms && KT / (splits * 2) >= 2 && (size_t)(splits * 2) * a.m * sg.n <= RowsScratch::part_floats() &&
               row_groups <= RowsScratch::CNT_MAX)
            splits *= 2;
        if (splits > 1 && (!sc.part || !sc.cnt)) splits = 1;
        p.splits = splits;
        p.kts_per_split = (KT + splits - 1) / splits;
        p.splits = (KT + p.kts_per_split - 1) / p.kts_per_split;  // no empty split
        p.part = sc.part;
        p.cnt = sc.cnt;
        const size_t stage = 2 * (size_t)rows_stage_bytes(a.ncp);
        const size_t epi = (size_t)ROWS_WARPS * 16 * (p.groups * 32 + 1) * 4;
        const size_t smem = stage > epi ? stage : epi;
        const dim3 grid(row_groups, p.splits);
        cudaError_t le = cudaErrorInvalidValue;
#define SP_ROWS(F, GG) if (sg.dtype == F && p.groups == GG) le = launch_rows_inst<F, GG>(p, grid, smem, st)
        SP_ROWS(T_Q4_K, 1); SP_ROWS(T_Q4_K, 2); SP_ROWS(T_Q4_K, 3);
        SP_ROWS(T_Q6_K, 1); SP_ROWS(T_Q6_K, 2); SP_ROWS(T_Q6_K, 3);
        SP_ROWS(T_Q8_0, 1); SP_ROWS(T_Q8_0, 2); SP_ROWS(T_Q8_0, 3);
#undef SP_ROWS
        if (le != cudaSuccess) return le;
        le = count_launch_and_check();
        if (le != cudaSuccess) return le;
    }
    return cudaSuccess;
}

}  // namespace sp
