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

#include "gemv_imma.cuh"
#include "gemv_imma_dev.cuh"
#include "kernels.h"
#include "pdl.cuh"
#include "sp_common.cuh"

namespace sp {

cudaError_t count_launch_and_check();  // kernels.cu
void imma_note_ring_launch();          // gemv_imma.cu: arms imma_take_timeout
int* imma_timeout_flag();              // gemv_imma.cu: device address of the flag on the current device

constexpr int RING_CW = 15;                        // consumer warps = tiles per ring slot (16 warps with the service warp:
                                                   // four per scheduler, 128 registers per thread)
constexpr int RING_THREADS = (RING_CW + 1) * 32;
constexpr int RING_SPIN_LIMIT = 1 << 22;           // try_wait polls (each blocks for a short, implementation-defined time): a second or so
constexpr int RING_SMEM_SHARED_SM = 112 * 1024;    // budget that leaves room for a second CTA on the SM
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
__device__ __forceinline__ void ring_bar_consumers() { asm volatile("bar.sync 2, %0;\n" ::"r"(RING_CW * 32) : "memory"); }

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

template <int NT>
__device__ __forceinline__ void ring_load_b(const RingDigits& q, int kt, int g, int t, BFrag<NT>& b) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
        if (col < q.ncols) {
            const int8_t* rec = q.xq + ((int64_t)kt * q.ncols + col) * 256;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = *reinterpret_cast<const uint4*>(rec + 16 * ring_slot(t, i, col));
                b.w[nt][4 * i] = v.x; b.w[nt][4 * i + 1] = v.y; b.w[nt][4 * i + 2] = v.z; b.w[nt][4 * i + 3] = v.w;
            }
            const int64_t r = ((int64_t)kt * q.ncols + col) * 32 + 4 * t;
            b.ra32[nt] = *reinterpret_cast<const uint32_t*>(q.rec32 + r);
            b.rb32[nt] = *reinterpret_cast<const uint32_t*>(q.rec32 + r + 16);
            b.ra16[nt] = *reinterpret_cast<const uint32_t*>(q.rec16 + r);
            b.rb16[nt] = *reinterpret_cast<const uint32_t*>(q.rec16 + r + 16);
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

template <int NT>
__global__ void __launch_bounds__(RING_THREADS, 1) gemv_ring_kernel(const RingArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float norm_red[RING_CW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + a.off_bar);
    uint64_t* empty = full + RING_MAX_STAGES;
    uint8_t* ring = smem + a.off_stage;
    const int KT = a.kt;
    const int64_t T = a.total_tiles;
    const int t_begin = (int)(T * blockIdx.x / gridDim.x), t_end = (int)(T * (blockIdx.x + 1) / gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) { ring_mbar_init(&full[s], 1); ring_mbar_init(&empty[s], RING_CW); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // the sequence of ring slots: consecutive chunks of up to RING_CW tiles that do not cross a segment boundary
    auto chunk_len = [&](int t, int& s) {
        while (s < a.nseg - 1 && t >= a.seg_tile0[s + 1]) ++s;
        return min(RING_CW, min(t_end, a.seg_tile0[s + 1]) - t);
    };

    if (warp == RING_CW) {
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

        float racc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) racc[nt][0] = racc[nt][1] = racc[nt][2] = racc[nt][3] = 0.f;
        float* fb = reinterpret_cast<float*>(smem + a.off_flush);
        const int first_row_tile = t_begin;  // the CTA's first tile row is the one holding this tile
        int cur_seg = -1, cur_row = -1;       // tile row being summed: (segment, row inside the segment)

        // finished value of output (row r of the tile row, activation row mm): bias, residual, store
        auto finalize = [&](int sgi, int row_in_seg, int idx, float v) {
            const ImmaSeg& sg = a.seg[sgi];
            const int r = idx & 15, mm = idx >> 4;
            const int64_t row = (int64_t)row_in_seg * 16 + r;
            if (row >= sg.n) return;
            if (sg.bias) v += sg.bias[row];
            if (sgi == 0 && a.res) v += a.res[(int64_t)mm * a.ldres + row];
            sg.y[(int64_t)mm * sg.ldy + row] = v;
        };
        auto cta_begin = [&](int c) { return (int)(T * c / gridDim.x); };
        auto cta_of = [&](int tile) {
            int c = (int)(((int64_t)tile * gridDim.x) / T);
            while (c + 1 < (int)gridDim.x && cta_begin(c + 1) <= tile) ++c;
            while (c > 0 && cta_begin(c) > tile) --c;
            return c;
        };
        auto flush = [&]() {
            if (cur_row < 0) return;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) fb[(nt * 4 + e) * 32 + lane] = racc[nt][e];
            __syncwarp();
            const int rs = a.seg_tile0[cur_seg] + cur_row * KT, re = rs + KT;  // the tile row's tiles, launch-wide numbering
            const bool owned = t_begin <= rs && re <= t_end;
            const int n_out = 16 * a.m;
            const int row_id = a.seg_row0[cur_seg] + cur_row;
            bool last = false;
            int c0 = 0, c1 = 0;
            if (!owned) {
                const int slot = (rs <= first_row_tile && first_row_tile < re) ? 0 : 1;
                float* mine = a.fix_part + ((size_t)blockIdx.x * 2 + slot) * 64;
                for (int idx = lane; idx < n_out; idx += 32) {
                    const int r = idx & 15, mm = idx >> 4;
                    float v = 0.f;
                    for (int d = 0; d < a.digits; ++d) {
                        const int col = mm * a.digits + d, nt = col >> 3, cc = col & 7;
                        v += fb[((nt * 4) + (r < 8 ? 0 : 2) + (cc & 1)) * 32 + (r & 7) * 4 + (cc >> 1)];
                    }
                    mine[idx] = v;
                }
                __threadfence();
                __syncwarp();
                c0 = cta_of(rs);
                c1 = cta_of(re - 1);
                unsigned prev = 0;
                if (lane == 0) prev = atomicAdd(&a.fix_cnt[row_id], 1u);
                prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
                last = prev == (unsigned)(c1 - c0);
                if (last) __threadfence();
            }
            if (owned || last) {
                for (int idx = lane; idx < n_out; idx += 32) {
                    float v = 0.f;
                    if (owned) {
                        const int r = idx & 15, mm = idx >> 4;
                        for (int d = 0; d < a.digits; ++d) {
                            const int col = mm * a.digits + d, nt = col >> 3, cc = col & 7;
                            v += fb[((nt * 4) + (r < 8 ? 0 : 2) + (cc & 1)) * 32 + (r & 7) * 4 + (cc >> 1)];
                        }
                    } else {
                        for (int c = c0; c <= c1; ++c) {
                            const int fb_tile = cta_begin(c);  // that CTA's first tile: inside this row -> its slot 0
                            const int slot = (rs <= fb_tile && fb_tile < re) ? 0 : 1;
                            v += __ldcg(a.fix_part + ((size_t)c * 2 + slot) * 64 + idx);
                        }
                    }
                    finalize(cur_seg, cur_row, idx, v);
                }
                if (last && lane == 0) a.fix_cnt[row_id] = 0u;  // ready for the next launch
            }
            __syncwarp();
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) racc[nt][0] = racc[nt][1] = racc[nt][2] = racc[nt][3] = 0.f;
        };

        bool ok = true;
        int ct = t_begin, cs = 0, cslot = 0;
        uint32_t cpar = 0;
        int retired = 0;
        // position of the next tile inside its segment: (tile row, k tile), kept without divisions
        int nrow = 0, nkt = 0;
        {
            int s0 = 0;
            while (s0 < a.nseg - 1 && t_begin >= a.seg_tile0[s0 + 1]) ++s0;
            const int local = t_begin - a.seg_tile0[s0];
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
            auto add_tile = [&](const float4 (&f)[NT]) {
                if (cs != cur_seg || nrow != cur_row) {
                    flush();
                    cur_seg = cs;
                    cur_row = nrow;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    racc[nt][0] += f[nt].x; racc[nt][1] += f[nt].y; racc[nt][2] += f[nt].z; racc[nt][3] += f[nt].w;
                }
                if (++nkt == KT) { nkt = 0; ++nrow; }
            };
            auto rearm = [&]() {
                if (pt < t_end) {
                    __syncwarp();
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the slot's generic accesses precede the async refill
                    issue();
                    ++issued;
                }
            };
            if (NT == 1) {
                // all fragments of the slot into registers first, so that the slot is re-armed before they are summed
                float4 fr[RING_CW][NT];
                float guard = 0.f;
#pragma unroll
                for (int w = 0; w < RING_CW; ++w) {
                    fr[w][0] = w < len ? reinterpret_cast<const float4*>(slot_base + (size_t)w * tb)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
                    guard += fr[w][0].x;
                }
                asm volatile("" ::"f"(guard) : "memory");  // the loads have returned before the copy may overwrite the slot
                rearm();
#pragma unroll
                for (int w = 0; w < RING_CW; ++w)
                    if (w < len) add_tile(fr[w]);
            } else {
                for (int w = 0; w < len; ++w) {
                    float4 f[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) f[nt] = reinterpret_cast<const float4*>(slot_base + (size_t)w * tb)[nt * 32 + lane];
                    add_tile(f);
                }
                rearm();
            }
            ct += len;
            if (++cslot == a.stages) { cslot = 0; cpar ^= 1u; }
        }
        if (ok) flush();
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
        for (int i = threadIdx.x; i < KT * 8 * NT; i += RING_CW * 32) q.cs[i] = 0.f;
        ring_bar_consumers();
        auto block_sum = [&](float v) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            ring_bar_consumers();
            if (lane == 0) norm_red[warp] = v;
            ring_bar_consumers();
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < RING_CW; ++w) s += norm_red[w];
            return s;
        };
        for (int mm = 0; mm < a.m; ++mm) {
            const float* row = a.x + (int64_t)mm * a.ldx;
            float mean = 0.f, inv = 1.f;
            if (a.src == RING_SRC_RMS || a.src == RING_SRC_LN) {
                if (a.src == RING_SRC_LN) {
                    float s = 0.f;
                    for (int kt = warp; kt < KT; kt += RING_CW) {
                        float xv[8];
                        ring_load8(row + kt * 256 + lane * 8, xv);
                        s += ((xv[0] + xv[1]) + (xv[2] + xv[3])) + ((xv[4] + xv[5]) + (xv[6] + xv[7]));
                    }
                    mean = block_sum(s) / (float)a.k;
                }
                float ss = 0.f;
                for (int kt = warp; kt < KT; kt += RING_CW) {
                    float xv[8];
                    ring_load8(row + kt * 256 + lane * 8, xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { const float c = xv[i] - mean; ss = fmaf(c, c, ss); }
                }
                inv = 1.0f / sqrtf(block_sum(ss) / (float)a.k + a.eps);
            }
            for (int kt = warp; kt < KT; kt += RING_CW) {
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
        ring_bar_consumers();  // every consumer sees the complete digits

        bool ok = true;
        int ct = t_begin, cs = 0, slot = 0;
        uint32_t par = 0;
        while (ct < t_end) {
            const int len = chunk_len(ct, cs);
            if (warp < len && ok) {
                ok = ring_wait(&full[slot], par);
                if (ok) {
                    const int dtype = a.seg[cs].dtype, tb = ring_tile_bytes(dtype);
                    const int kt = (ct + warp - a.seg_tile0[cs]) % KT;
                    uint8_t* tile = ring + (size_t)slot * a.stage_bytes + (size_t)warp * tb;
                    float acc[NT][4];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                    BFrag<NT> b;
                    ring_load_b<NT>(q, kt, g, t, b);
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
                    __syncwarp();  // every lane has its tile bytes in registers: the fragment may overwrite them
                    float4* frag = reinterpret_cast<float4*>(tile);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) frag[nt * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
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
    cudaError_t e = cudaMalloc((void**)&part, (size_t)sms * 2 * 64 * sizeof(float));
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
    if (a.k <= 0 || a.k % 256 != 0 || a.m < 1 || a.m > 4 || a.nseg < 1 || a.nseg > 3 || !sc.part || !sc.cnt) return false;
    a.digits = a.m <= 2 ? 3 : 2;
    const int ncols = a.m * a.digits;
    const int nt = ncols <= 8 ? 1 : 2;
    a.kt = a.k / 256;
    int tiles = 0, rows = 0, max_tb = 0;
    for (int s = 0; s < a.nseg; ++s) {
        const int dt = a.seg[s].dtype;
        if (dt != T_Q4_K && dt != T_Q6_K && dt != T_Q8_0) return false;
        if (a.seg[s].n <= 0) return false;
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
    a.stage_bytes = (RING_CW * max_tb + 127) / 128 * 128;
    const int budget = share_sm ? RING_SMEM_SHARED_SM : RING_SMEM_MAX;
    int stages = (budget - off) / a.stage_bytes;
    if (stages < 2) stages = (RING_SMEM_MAX - off) / a.stage_bytes;  // does not fit beside a second CTA: take the SM alone
    if (stages < 2) return false;
    a.stages = std::min(stages, RING_MAX_STAGES);
    a.smem_total = off + a.stages * a.stage_bytes;
    a.fix_part = sc.part;
    a.fix_cnt = sc.cnt;
    return true;
}

static PerDeviceOnce g_ring_attr[2];

cudaError_t launch_gemv_ring(RingArgs& a, cudaStream_t st) {
    const int nt = a.m * a.digits <= 8 ? 1 : 2;
    const int sms = device_sm_count();
    // at least one full ring slot of work per CTA
    int grid = std::min(sms, std::max(1, a.total_tiles / RING_CW));
    a.err = imma_timeout_flag();
    if (!a.err) return cudaErrorInvalidValue;
    cudaError_t e = g_ring_attr[nt - 1].run([nt] {
        return nt == 1 ? cudaFuncSetAttribute(gemv_ring_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_SMEM_MAX)
                       : cudaFuncSetAttribute(gemv_ring_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_SMEM_MAX);
    });
    if (e != cudaSuccess) return e;
    imma_note_ring_launch();
    e = nt == 1 ? launch_pdl(gemv_ring_kernel<1>, dim3(grid), dim3(RING_THREADS), (size_t)a.smem_total, st, a)
                : launch_pdl(gemv_ring_kernel<2>, dim3(grid), dim3(RING_THREADS), (size_t)a.smem_total, st, a);
    if (e != cudaSuccess) return e;
    return count_launch_and_check();
}

}  // namespace sp
