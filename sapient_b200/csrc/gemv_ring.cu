// Persistent dequant-GEMV for decode-shaped steps (1-4 activation rows): one CTA per SM streams its share of the weight
// tiles through a shared-memory ring filled by bulk copies (cp.async.bulk + mbarrier), and builds its own copy of the
// activation digits in shared memory from the f32 activations — optionally through the RMSNorm / LayerNorm, SwiGLU or
// GELU that precedes the matrix in the layer. A layer's chain norm -> q|k|v, norm -> gate|up, SwiGLU -> down therefore
// needs no separate producer kernels, and under programmatic dependent launch the ring of the NEXT matrix fills while
// the previous kernel is still running: weights never depend on another kernel, so every CTA requests its first stages
// before the grid-dependency wait.
//
// Arithmetic per tile is that of gemv_imma.cu (exact integer products of weight quants and activation digits on
// mma.sync, block scales applied to the s32 sums); it restates the reference's matmul_nt
// (crates/sapient-backends/cpu/src/kernels/matmul.rs:575-689,862-943,1111-1167), linear_3d + bias
// (forward/common.rs:220-240,556-569), rms_norm / layer_norm (kernels/layernorm.rs:17-105) and silu·up / tanh-GELU
// (kernels/elementwise.rs:120-143).
//
// Work split. The launch's tiles (16 rows x 256 columns, all segments concatenated in [segment][tile row][k tile]
// order, which is also their order in memory) are cut into gridDim.x equal contiguous ranges, so each CTA reads one
// or a few contiguous byte spans whatever the matrix shape — 256 tile rows of o_proj still occupy all 148 SMs. A tile
// row whose k tiles straddle two or more CTAs is finished by the last of them to arrive (each writes its 16 x m partial
// sums to scratch and bumps a counter; the last one adds the parts in CTA order): no CTA waits for another, and the
// order of every f32 addition is fixed, so results do not vary from run to run.
//
// Inside a CTA: warps 0-7 are consumers, warp 8 is the service warp.
//   * ring: `stages` slots of 8 tiles; a slot is filled by ONE bulk copy of up to 8 consecutive tiles (18-35 KB),
//     completing on the slot's `full` mbarrier by byte count; consumer warp w takes tile w of the slot, computes its
//     16 x 8NT partial fragment against the digits in shared memory and leaves it in the first bytes of the tile it has
//     just consumed, then arrives on the slot's `empty` mbarrier (count 8);
//   * the service warp waits for `empty`, adds the slot's fragments (in tile order) into the running sum of the current
//     tile row, re-arms the slot with the next bulk copy, and writes finished rows: digit columns summed, bias,
//     residual, store (or the cross-CTA hand-over above). Consumers never wait for anything but data.
// Every mbarrier wait is bounded; after an expired wait the CTA stops consuming, raises the error flag the host reads
// (imma_take_timeout), waits — bounded again — for its copies in flight and returns.
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "gemv_imma.cuh"
#include "gemv_imma_dev.cuh"
#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu
void imma_note_ring_launch();          // gemv_imma.cu: arms imma_take_timeout
int* imma_timeout_flag();              // gemv_imma.cu: device address of the flag on the current device

// Consumer warps = tiles per ring slot. 15 (16 warps with the service warp: four per scheduler, up to 128 registers per
// thread) for launches that mix weight formats; 23 (24 warps, 80 registers) when every segment has one K-quant format
// and the per-format code fits the smaller register budget: the tile arithmetic is latency-bound per warp, so more
// resident warps are worth more than a deeper ring.
constexpr int RING_CW_MIXED = 15, RING_CW_SINGLE = 23;
constexpr int RING_PART_FLOATS = 96;               // partial block of a shared tile row: 16 x 5 outputs, padded
constexpr int RING_SPIN_LIMIT = 1 << 22;           // try_wait polls (each blocks for a short, implementation-defined time): a second or so
constexpr int RING_SMEM_MAX = 200 * 1024;

__device__ __forceinline__ uint32_t ring_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ring_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ring_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void ring_expect_tx(uint64_t* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(ring_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ring_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ring_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ring_bulk_g2s(void* dst, const void* src, int bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(ring_smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(ring_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = ring_smem_u32(bar);
    for (int spin = 0; spin < RING_SPIN_LIMIT; ++spin) {
        uint32_t ok;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
template <int CW>
__device__ __forceinline__ void ring_bar_consumers() { asm volatile("bar.sync 2, %0;\n" ::"r"(CW * 32) : "memory"); }

// ───────────────────────── activation digits in shared memory ─────────────────────────
// Digits of tile kt, digit column col: a 256-byte record in fragment order [t 0..3][block 0..7][8 B] (gemv_imma.cuh),
// whose sixteen 16-byte slots are permuted so that the eight lanes of a shared-memory load phase (two columns x four t)
// hit eight different bank groups: slot (t, i) lives at 4 t + (i ^ ((t >> 1) | ((col & 1) << 1))).
__device__ __forceinline__ int ring_slot(int t, int i, int col) { return 4 * t + (i ^ ((t >> 1) | ((col & 1) << 1))); }

struct RingDigits {
    int8_t* xq;      // [kt][ncols][256]
    int8_t* rec32;   // [kt][ncols][32]: { a[0..7], 0 x 8, b[0..7], 0 x 8 }, block sums S = a + 64 b
    int8_t* rec16;   // [kt][ncols][32]: { a[0..15], b[0..15] }
    float* cs;       // [kt][8 NT]
    int ncols, ncp, digits;
};

// One warp converts the 256 columns of tile kt of activation row m; lane holds columns 8 lane .. 8 lane + 7 in v.
// Same digit arithmetic as quantize_chunk (gemv_imma.cu), one exponent per 256 columns.
__device__ __forceinline__ void ring_quantize_tile(const float (&v)[8], int lane, int kt, int m, const RingDigits& q) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const int digits = q.digits, P = 8 * digits - 2;
    float up = 0.f, down = 0.f;
    if (amax > 0.f && amax < INFINITY) {
        int e = ilogbf(amax) + 1;
        e = max(e, -100);
        up = scalbnf(1.0f, P - e);
        down = scalbnf(1.0f, e - P);
    }
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
    const int a4 = lane & 3, blk = lane >> 2;
    const int h = a4 >> 1, t0 = 2 * (a4 & 1);
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        const int s16 = sum[d] + __shfl_xor_sync(0xFFFFFFFFu, sum[d], 1);
        const int s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
        if (d < digits) {
            const int col = m * digits + d;
            int8_t* rec = q.xq + ((int64_t)kt * q.ncols + col) * 256;
            // fragment byte (t, blk, 4 h ..) sits in 16-byte slot (t, blk >> 1) at offset 8 (blk & 1) + 4 h
            *reinterpret_cast<uint32_t*>(rec + 16 * ring_slot(t0, blk >> 1, col) + 8 * (blk & 1) + 4 * h) = w0[d];
            *reinterpret_cast<uint32_t*>(rec + 16 * ring_slot(t0 + 1, blk >> 1, col) + 8 * (blk & 1) + 4 * h) = w1[d];
            int8_t* r32 = q.rec32 + ((int64_t)kt * q.ncols + col) * 32;
            int8_t* r16 = q.rec16 + ((int64_t)kt * q.ncols + col) * 32;
            if ((lane & 1) == 0) {
                const int a = ((s16 + 32) & 63) - 32;
                r16[lane >> 1] = (int8_t)a;
                r16[16 + (lane >> 1)] = (int8_t)((s16 - a) >> 6);
            }
            if (a4 == 0) {
                const int a = ((s32 + 32) & 63) - 32;
                r32[blk] = (int8_t)a;
                r32[16 + blk] = (int8_t)((s32 - a) >> 6);
                r32[8 + blk] = 0;
                r32[24 + blk] = 0;
            }
        }
    }
    if (lane == 0) {
        float s = down;
        for (int d = 0; d < digits; ++d) {
            q.cs[kt * q.ncp + m * digits + d] = s;
            s *= 256.f;
        }
    }
}

// Per-lane constants of the B-fragment loads: byte offsets inside one k tile's block of digit records.
template <int NT>
struct RingLane {
    int xoff[NT][4];   // digit words: record of the lane's column + its four 16-byte slots
    int roff[NT];      // digit-sum records
    int own[NT][2];    // activation row that digit column 8 nt + 2 t + e belongs to, or -1 past the live columns
    bool live[NT];
};
template <int NT>
__device__ __forceinline__ void ring_lane_init(RingLane<NT>& L, int g, int t, int ncols, int digits) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
        L.live[nt] = col < ncols;
#pragma unroll
        for (int i = 0; i < 4; ++i) L.xoff[nt][i] = col * 256 + 16 * ring_slot(t, i, col);
        L.roff[nt] = col * 32 + 4 * t;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int c = nt * 8 + 2 * t + e;
            L.own[nt][e] = c < ncols ? (digits == 3 ? c / 3 : c >> 1) : -1;
        }
    }
}
template <int NT, int FMT>
__device__ __forceinline__ void ring_load_b(const RingDigits& q, const RingLane<NT>& L, int kt, int t, int dtype, BFrag<NT>& b) {
    const int8_t* xb = q.xq + (int64_t)kt * q.ncols * 256;
    const int8_t* r32 = q.rec32 + (int64_t)kt * q.ncols * 32;
    const int8_t* r16 = q.rec16 + (int64_t)kt * q.ncols * 32;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if (L.live[nt]) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4*>(xb + L.xoff[nt][i]);
                b.w[nt][4 * i] = v.x; b.w[nt][4 * i + 1] = v.y; b.w[nt][4 * i + 2] = v.z; b.w[nt][4 * i + 3] = v.w;
            }
            const bool q4 = FMT == T_Q4_K || (FMT == 0 && dtype == T_Q4_K), q6 = FMT == T_Q6_K || (FMT == 0 && dtype == T_Q6_K);
            b.ra32[nt] = q4 ? *reinterpret_cast<const uint32_t*>(r32 + L.roff[nt]) : 0u;
            b.rb32[nt] = q4 ? *reinterpret_cast<const uint32_t*>(r32 + L.roff[nt] + 16) : 0u;
            b.ra16[nt] = q6 ? *reinterpret_cast<const uint32_t*>(r16 + L.roff[nt]) : 0u;
            b.rb16[nt] = q6 ? *reinterpret_cast<const uint32_t*>(r16 + L.roff[nt] + 16) : 0u;
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) b.w[nt][i] = 0u;
            b.ra32[nt] = b.rb32[nt] = b.ra16[nt] = b.rb16[nt] = 0u;
        }
        b.cs[nt] = *reinterpret_cast<const float2*>(q.cs + kt * q.ncp + nt * 8 + 2 * t);
    }
}

// ───────────────────────────────── the kernel ─────────────────────────────────
__device__ __forceinline__ int ring_tile_bytes(int dtype) { return dtype == T_Q4_K ? Q4_K_TILE_BYTES : dtype == T_Q6_K ? Q6_K_TILE_BYTES : 4352; }

__device__ __forceinline__ float ring_silu_mul(float g, float u) { return __fmul_rn(g / (1.0f + expf(-g)), u); }
__device__ __forceinline__ float ring_gelu(float t) {
    const float inner = __fmul_rn(0.79788456f, __fadd_rn(t, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, t), t), t)));
    return __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, tanhf(inner)));
}
__device__ __forceinline__ void ring_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Hand-over of one finished tile row by the service warp (not inlined: it is a few hundred instructions that run once
// per tile row, or once per CTA for the shared-row path). v0 / v1: the sums of outputs `lane` and `lane + 32` of the
// row's 16 x m outputs (idx = 16 * activation row + weight row inside the tile row) over this CTA's tiles of the row.
struct RowOut {
    const RingArgs* a;
    int t_begin, t_end, lane;
};
template <int R>
__device__ __noinline__ void ring_row_out(const RowOut& ro, int seg, int row_in_seg, const float (&v)[R]) {
    const RingArgs& a = *ro.a;
    const int lane = ro.lane, KT = a.kt, n_out = 16 * a.m;
    const int64_t T = a.total_tiles;
    const ImmaSeg& sg = a.seg[seg];
    auto finalize = [&](int idx, float val) {
        const int r = idx & 15, mm = idx >> 4;
        const int64_t row = (int64_t)row_in_seg * 16 + r;
        if (idx >= n_out || row >= sg.n) return;
        if (sg.bias) val += sg.bias[row];
        if (seg == 0 && a.res) val += a.res[(int64_t)mm * a.ldres + row];
        sg.y[(int64_t)mm * sg.ldy + row] = val;
    };
    const int rs = a.seg_tile0[seg] + row_in_seg * KT, re = rs + KT;  // the tile row's tiles, launch-wide numbering
    if (ro.t_begin <= rs && re <= ro.t_end) {  // every tile of the row was this CTA's
#pragma unroll
        for (int r = 0; r < R; ++r) finalize(lane + 32 * r, v[r]);
        return;
    }
    // shared with other CTAs: leave the partial sums, count the arrival; the last CTA adds the parts in CTA order
    auto cta_begin = [&](int c) { return (int)(T * c / gridDim.x); };
    auto cta_of = [&](int tile) {
        int c = (int)(((int64_t)tile * gridDim.x) / T);
        while (c + 1 < (int)gridDim.x && cta_begin(c + 1) <= tile) ++c;
        while (c > 0 && cta_begin(c) > tile) --c;
        return c;
    };
    const int slot = (rs <= ro.t_begin && ro.t_begin < re) ? 0 : 1;  // slot 0: the row holding the CTA's first tile
    float* mine = a.fix_part + ((size_t)blockIdx.x * 2 + slot) * RING_PART_FLOATS;
#pragma unroll
    for (int r = 0; r < R; ++r) mine[lane + 32 * r] = v[r];
    __threadfence();
    __syncwarp();
    const int c0 = cta_of(rs), c1 = cta_of(re - 1);
    const int row_id = a.seg_row0[seg] + row_in_seg;
    unsigned prev = 0;
    if (lane == 0) prev = atomicAdd(&a.fix_cnt[row_id], 1u);
    prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
    if (prev != (unsigned)(c1 - c0)) return;
    __threadfence();
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = 0.f;
    for (int c = c0; c <= c1; ++c) {
        const int fb_tile = cta_begin(c);  // that CTA's first tile: inside this row -> its slot 0
        const float* part = a.fix_part + ((size_t)c * 2 + ((rs <= fb_tile && fb_tile < re) ? 0 : 1)) * RING_PART_FLOATS;
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] += __ldcg(part + lane + 32 * r);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) finalize(lane + 32 * r, s[r]);
    if (lane == 0) a.fix_cnt[row_id] = 0u;  // ready for the next launch
}

template <int NT, int CW, int FMT>
__global__ void __launch_bounds__((CW + 1) * 32, 1) gemv_ring_kernel(const __grid_constant__ RingArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float norm_red[CW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + a.off_bar);
    uint64_t* empty = full + RING_MAX_STAGES;
    uint8_t* ring = smem + a.off_stage;
    const int KT = a.kt;
    const int64_t T = a.total_tiles;
    const int t_begin = (int)(T * blockIdx.x / gridDim.x), t_end = (int)(T * (blockIdx.x + 1) / gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) { ring_mbar_init(&full[s], 1); ring_mbar_init(&empty[s], CW); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // the sequence of ring slots: consecutive chunks of up to CW tiles that do not cross a segment boundary
    auto chunk_len = [&](int t, int& s) {
        while (s < a.nseg - 1 && t >= a.seg_tile0[s + 1]) ++s;
        return min(CW, min(t_end, a.seg_tile0[s + 1]) - t);
    };

    if (warp == CW) {
        // ───────────── service warp: producer of the ring, reducer of the fragments, writer of finished rows ─────────────
        int pt = t_begin, ps = 0, pslot = 0;  // producer cursor
        auto issue = [&]() {
            const int len = chunk_len(pt, ps);
            if (lane == 0) {
                const int tb = ring_tile_bytes(a.seg[ps].dtype);
                const uint8_t* src = a.seg[ps].wt + (int64_t)(pt - a.seg_tile0[ps]) * tb;
                ring_expect_tx(&full[pslot], len * tb);
                ring_bulk_g2s(ring + (size_t)pslot * a.stage_bytes, src, len * tb, &full[pslot]);
            }
            pt += len;
            pslot = pslot + 1 == a.stages ? 0 : pslot + 1;
        };
        int issued = 0;
        for (int i = 0; i < a.stages && pt < t_end; ++i) { issue(); ++issued; }
        pdl_wait();      // the residual (and the scratch of shared rows) belong to the previous kernel until here
        pdl_trigger();

        // Consumers hand over, per tile, the 16 x m outputs with the digit columns already added (80 floats at most):
        // lane l of this warp owns outputs l, l + 32, l + 64 (output idx = 16 * activation row + weight row of the tile
        // row); one or two activation rows need only the first.
        constexpr int R = NT == 1 ? 1 : 3;
        float racc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) racc[r] = 0.f;
        const int n_out = 16 * a.m;
        int cur_seg = -1, cur_row = -1;       // tile row being summed: (segment, row inside the segment)
        RowOut ro;
        ro.a = &a; ro.t_begin = t_begin; ro.t_end = t_end; ro.lane = lane;

        bool ok = true;
        int ct = t_begin, cs = 0, cslot = 0;
        uint32_t cpar = 0;
        int retired = 0;
        // position of the next tile inside its segment: (tile row, k tile), kept without divisions
        int nrow = 0, nkt = 0;
        {
            while (cs < a.nseg - 1 && t_begin >= a.seg_tile0[cs + 1]) ++cs;  // the segment the range starts in
            const int local = t_begin - a.seg_tile0[cs];
            nrow = local / KT;
            nkt = local - nrow * KT;
        }
        while (ct < t_end) {
            const int seg_before = cs;
            const int len = chunk_len(ct, cs);
            if (cs != seg_before) { nrow = 0; nkt = 0; }  // chunks never cross a segment: a new one starts at its first tile
            ok = ok && ring_wait(&empty[cslot], cpar);
            if (!ok) break;
            ++retired;
            const int tb = ring_tile_bytes(a.seg[cs].dtype);
            const uint8_t* slot_base = ring + (size_t)cslot * a.stage_bytes;
            // the slot's hand-over values into registers, then the slot is re-armed, then they are summed
            float v[CW][R];
            float guard = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) {
                const float* f = reinterpret_cast<const float*>(slot_base + (size_t)w * tb);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    v[w][r] = (w < len && lane + 32 * r < n_out) ? f[lane + 32 * r] : 0.f;
                    guard += v[w][r];
                }
            }
            asm volatile("" ::"f"(guard) : "memory");  // the loads have returned before the copy may overwrite the slot
            if (pt < t_end) {
                __syncwarp();
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the slot's generic accesses precede the async refill
                issue();
                ++issued;
            }
#pragma unroll
            for (int w = 0; w < CW; ++w) {
                if (w < len) {
                    if (cs != cur_seg || nrow != cur_row) {
                        if (cur_row >= 0) ring_row_out<R>(ro, cur_seg, cur_row, racc);
#pragma unroll
                        for (int r = 0; r < R; ++r) racc[r] = 0.f;
                        cur_seg = cs;
                        cur_row = nrow;
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) racc[r] += v[w][r];
                    if (++nkt == KT) { nkt = 0; ++nrow; }
                }
            }
            ct += len;
            if (++cslot == a.stages) { cslot = 0; cpar ^= 1u; }
        }
        if (ok && cur_row >= 0) ring_row_out<R>(ro, cur_seg, cur_row, racc);
        if (!ok) {
            if (lane == 0) *reinterpret_cast<volatile int*>(a.err) = 1;  // host-mapped flag: a plain store
            // copies still in flight write into this CTA's shared memory: wait for them (bounded) before leaving
            for (int i = retired; i < issued; ++i) {
                const int s = i % a.stages;
                ring_wait(&full[s], (uint32_t)((i / a.stages) & 1));
            }
        }
    } else {
        // ───────────── consumers ─────────────
        pdl_wait();  // the activations are the previous kernel's output
        const int g = lane >> 2, t = lane & 3;
        RingDigits q;
        q.xq = reinterpret_cast<int8_t*>(smem + a.off_xq);
        q.rec32 = reinterpret_cast<int8_t*>(smem + a.off_rec32);
        q.rec16 = reinterpret_cast<int8_t*>(smem + a.off_rec16);
        q.cs = reinterpret_cast<float*>(smem + a.off_cs);
        q.ncols = a.m * a.digits; q.ncp = 8 * NT; q.digits = a.digits;
        // unused digit columns meet zero digits but their scales are read: keep them finite
        for (int i = threadIdx.x; i < KT * 8 * NT; i += CW * 32) q.cs[i] = 0.f;
        ring_bar_consumers<CW>();
        auto block_sum = [&](float v) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            ring_bar_consumers<CW>();
            if (lane == 0) norm_red[warp] = v;
            ring_bar_consumers<CW>();
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < CW; ++w) s += norm_red[w];
            return s;
        };
        for (int mm = 0; mm < a.m; ++mm) {
            const float* row = a.x + (int64_t)mm * a.ldx;
            float mean = 0.f, inv = 1.f;
            if (a.src == RING_SRC_RMS || a.src == RING_SRC_LN) {
                if (a.src == RING_SRC_LN) {
                    float s = 0.f;
                    for (int kt = warp; kt < KT; kt += CW) {
                        float xv[8];
                        ring_load8(row + kt * 256 + lane * 8, xv);
                        s += ((xv[0] + xv[1]) + (xv[2] + xv[3])) + ((xv[4] + xv[5]) + (xv[6] + xv[7]));
                    }
                    mean = block_sum(s) / (float)a.k;
                }
                float ss = 0.f;
                for (int kt = warp; kt < KT; kt += CW) {
                    float xv[8];
                    ring_load8(row + kt * 256 + lane * 8, xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { const float c = xv[i] - mean; ss = fmaf(c, c, ss); }
                }
                inv = 1.0f / sqrtf(block_sum(ss) / (float)a.k + a.eps);
            }
            for (int kt = warp; kt < KT; kt += CW) {
                const int k0 = kt * 256 + lane * 8;
                float v[8];
                ring_load8(row + k0, v);
                if (a.src == RING_SRC_RMS || a.src == RING_SRC_LN) {
                    float wv[8];
                    ring_load8(a.nw + k0, wv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i] - mean, inv), wv[i]);
                    if (a.src == RING_SRC_LN && a.nb) {
                        float bv[8];
                        ring_load8(a.nb + k0, bv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(v[i], bv[i]);
                    }
                } else if (a.src == RING_SRC_SWIGLU) {
                    float u[8];
                    ring_load8(row + a.k + k0, u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = ring_silu_mul(v[i], u[i]);
                } else if (a.src == RING_SRC_GELU) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = ring_gelu(v[i]);
                }
                ring_quantize_tile(v, lane, kt, mm, q);
            }
        }
        ring_bar_consumers<CW>();  // every consumer sees the complete digits
        RingLane<NT> L;
        ring_lane_init<NT>(L, g, t, q.ncols, q.digits);

        bool ok = true;
        int ct = t_begin, cs = 0, slot = 0;
        uint32_t par = 0;
        while (ct < t_end) {
            const int len = chunk_len(ct, cs);
            if (warp < len && ok) {
                ok = ring_wait(&full[slot], par);
                if (ok) {
                    const int dtype = FMT ? FMT : a.seg[cs].dtype, tb = ring_tile_bytes(dtype);
                    const int kt = (ct + warp - a.seg_tile0[cs]) % KT;
                    uint8_t* tile = ring + (size_t)slot * a.stage_bytes + (size_t)warp * tb;
                    float acc[NT][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                    BFrag<NT> b;
                    ring_load_b<NT, FMT>(q, L, kt, t, dtype, b);
                    if (FMT == T_Q4_K || (FMT == 0 && dtype == T_Q4_K)) {
                        Q4Regs r;
                        load_q4_k<false>(tile, lane, r);
                        compute_q4_k<NT>(r, b, lane, acc);
                    } else if (FMT == T_Q6_K || (FMT == 0 && dtype == T_Q6_K)) {
                        Q6Regs r;
                        load_q6_k<false>(tile, lane, r);
                        compute_q6_k<NT>(r, b, lane, acc);
                    } else if (FMT == 0) {
                        Q8Regs r;
                        load_q8_0<false>(tile, lane, r);
                        compute_q8_0<NT>(r, b, acc);
                    }
                    __syncwarp();  // every lane has its tile bytes in registers: the hand-over values may overwrite them
                    // outputs of this tile: for activation row mm the digit columns mm * digits .. are added; lane (g, t)
                    // holds columns 8 nt + 2 t, + 1 of weight rows g (acc[.][0..1]) and g + 8 (acc[.][2..3])
                    float* hand = reinterpret_cast<float*>(tile);
                    for (int mm = 0; mm < a.m; ++mm) {
                        float lo = 0.f, hi = 0.f;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                if (L.own[nt][e] == mm) { lo += acc[nt][e]; hi += acc[nt][2 + e]; }
                        lo += __shfl_xor_sync(0xFFFFFFFFu, lo, 1); lo += __shfl_xor_sync(0xFFFFFFFFu, lo, 2);
                        hi += __shfl_xor_sync(0xFFFFFFFFu, hi, 1); hi += __shfl_xor_sync(0xFFFFFFFFu, hi, 2);
                        if (t == 0) { hand[mm * 16 + g] = lo; hand[mm * 16 + 8 + g] = hi; }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ring_arrive(&empty[slot]);  // also after an expired wait: the service warp must not starve
            ct += len;
            if (++slot == a.stages) { slot = 0; par ^= 1u; }
        }
        if (!ok && lane == 0) *reinterpret_cast<volatile int*>(a.err) = 1;
    }
}

// ───────────────────────────────── host side ─────────────────────────────────
cudaError_t RingScratch::alloc(int max_rows) {
    release();
    const int sms = device_sm_count();
    cudaError_t e = cudaMalloc((void**)&part, (size_t)sms * 2 * RING_PART_FLOATS * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&cnt, (size_t)(max_rows + 4) * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(cnt, 0, (size_t)(max_rows + 4) * sizeof(unsigned));
    if (e == cudaSuccess) { rows_cap = max_rows + 4; ctas_cap = sms; }
    else release();
    return e;
}
void RingScratch::release() {
    if (part) cudaFree(part);
    if (cnt) cudaFree(cnt);
    part = nullptr; cnt = nullptr; rows_cap = 0; ctas_cap = 0;
}

// Fills the work split and the shared-memory layout; false when the launch does not fit this kernel.
bool ring_plan(RingArgs& a, const RingScratch& sc, bool share_sm) {
    (void)share_sm;
    if (a.k <= 0 || a.k % 256 != 0 || a.m < 1 || a.m > RING_MAX_M || a.nseg < 1 || a.nseg > 3 || !sc.part || !sc.cnt) return false;
    a.digits = 3;  // activations to 2^-23 of each block's maximum at every row count this kernel takes
    const int ncols = a.m * a.digits;
    const int nt = ncols <= 8 ? 1 : 2;
    a.kt = a.k / 256;
    int tiles = 0, rows = 0, max_tb = 0;
    bool all_q4 = true, all_q6 = true;
    for (int s = 0; s < a.nseg; ++s) {
        const int dt = a.seg[s].dtype;
        if (dt != T_Q4_K && dt != T_Q6_K && dt != T_Q8_0) return false;
        if (a.seg[s].n <= 0) return false;
        all_q4 = all_q4 && dt == T_Q4_K;
        all_q6 = all_q6 && dt == T_Q6_K;
        a.seg_tile0[s] = tiles;
        a.seg_row0[s] = rows;
        const int r = (a.seg[s].n + 15) / 16;
        rows += r;
        tiles += r * a.kt;
        max_tb = std::max(max_tb, dt == T_Q4_K ? Q4_K_TILE_BYTES : dt == T_Q6_K ? Q6_K_TILE_BYTES : 4352);
    }
    for (int s = a.nseg; s < 4; ++s) { a.seg_tile0[s] = tiles; a.seg_row0[s] = rows; }
    a.total_tiles = tiles;
    if (rows > sc.rows_cap) return false;
    int off = 0;
    a.off_bar = off; off += 2 * RING_MAX_STAGES * 8;
    a.off_flush = off; off += nt * 128 * 4;
    a.off_cs = off; off += a.kt * 8 * nt * 4;
    a.off_rec32 = off; off += a.kt * ncols * 32;
    a.off_rec16 = off; off += a.kt * ncols * 32;
    off = (off + 127) / 128 * 128;
    a.off_xq = off; off += a.kt * ncols * 256;
    off = (off + 127) / 128 * 128;
    a.off_stage = off;
    // the wide single-format instance when its ring still has two slots, else the 15-consumer instance
    const int fmt = all_q4 ? T_Q4_K : all_q6 ? T_Q6_K : 0;
    for (int cw : {fmt && nt == 1 ? RING_CW_SINGLE : RING_CW_MIXED, RING_CW_MIXED}) {
        a.cw = cw;
        a.fmt = cw == RING_CW_SINGLE ? fmt : 0;
        a.stage_bytes = (cw * max_tb + 127) / 128 * 128;
        const int stages = (RING_SMEM_MAX - off) / a.stage_bytes;
        if (stages < 2) continue;
        a.stages = std::min(stages, RING_MAX_STAGES);
        a.smem_total = off + a.stages * a.stage_bytes;
        a.fix_part = sc.part;
        a.fix_cnt = sc.cnt;
        return true;
    }
    return false;
}

template <int NT, int CW, int FMT>
static cudaError_t ring_launch_instance(const RingArgs& a, int grid, cudaStream_t st) {
    static PerDeviceOnce attr;
    cudaError_t e = attr.run([] { return cudaFuncSetAttribute(gemv_ring_kernel<NT, CW, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_SMEM_MAX); });
    if (e != cudaSuccess) return e;
    return launch_pdl(gemv_ring_kernel<NT, CW, FMT>, dim3(grid), dim3((CW + 1) * 32), (size_t)a.smem_total, st, a);
}

cudaError_t launch_gemv_ring(RingArgs& a, cudaStream_t st) {
    const int nt = a.m * a.digits <= 8 ? 1 : 2;
    const int sms = device_sm_count();
    // at least one full ring slot of work per CTA
    const int grid = std::min(sms, std::max(1, a.total_tiles / a.cw));
    a.err = imma_timeout_flag();
    if (!a.err) return cudaErrorInvalidValue;
    cudaError_t e;
    if (nt == 2) e = ring_launch_instance<2, RING_CW_MIXED, 0>(a, grid, st);
    else if (a.cw == RING_CW_SINGLE && a.fmt == T_Q4_K) e = ring_launch_instance<1, RING_CW_SINGLE, T_Q4_K>(a, grid, st);
    else if (a.cw == RING_CW_SINGLE && a.fmt == T_Q6_K) e = ring_launch_instance<1, RING_CW_SINGLE, T_Q6_K>(a, grid, st);
    else e = ring_launch_instance<1, RING_CW_MIXED, 0>(a, grid, st);
    if (e != cudaSuccess) return e;
    return count_launch_and_check();
}

}  // namespace sp
