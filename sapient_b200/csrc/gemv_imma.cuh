// Tile-repacked weight layouts and activation digit format of the tensor-core GEMV.
//
// Weights are regrouped at upload into tiles of 16 rows x 256 columns (Q8_0: 16 rows x
// `bpt` 32-blocks), stored tile after tile in [row_tile][k_tile] order, so that one warp
// streams one tile with 16-byte loads where lane (g = lane/4, t = lane%4) finds exactly the
// bytes its mma.sync fragment needs (rows g and g+8; k = 4t..4t+3 and 16+4t..16+4t+3 of
// every 32-column block). No bit of the ggml blocks is changed or dropped; tile sizes
// equal 16 rows of raw blocks (Q4_K 2304 B, Q6_K 3360 B, Q8_0 544 B per 32-block column).
//
//   Q4_K tile: [j 0..3][lane 0..31][16 B] nibble words, then [row 0..15][16 B] block headers.
//     lane's 16 B for j = { rowg.B[32j+4t..], rowg.B[32j+16+4t..], rowg8.B[32j+4t..], rowg8.B[32j+16+4t..] }
//     (B = the block's 128 nibble bytes; low nibbles are sub-block 2j, high nibbles sub-block 2j+1).
//   Q6_K tile: [i 0..5][lane][16 B] then [row][16 B int8 scales] then [row] f16 d.
//     lane's 24 words = for c = (half, p) in 0..3: { qlA_g, qlB_g, qh_g, qlA_g8, qlB_g8, qh_g8 } with
//     qlA = ql[64 half + 16 p + 4t ..], qlB = ql[64 half + 32 + 16 p + 4t ..], qh = qh[32 half + 16 p + 4t ..].
//   Q8_0 tile (bpt blocks): [b 0..bpt-1][lane][16 B] = { rowg.q[4t..], rowg.q[16+4t..], rowg8.q[4t..], rowg8.q[16+4t..] }
//     then [row][bpt] f16 d.
//
// Activations are converted once per GEMV input into D (2 or 3) balanced base-256 int8
// digits per element with one power-of-two scale per 256 (or 32) columns:
//   x ~= 2^(e-P) * (d0 + 256 d1 + 65536 d2),  P = 8 D - 2,  |error| <= 2^(e-P-1), max|x| < 2^e
// so the products with the integer weights are exact in the s32 accumulators of
// mma.sync.m16n8k32.s8 and only the digit truncation (2^-23 resp. 2^-15 of the block
// maximum) separates the result from f32 arithmetic. Column c = m * D + i of the mma's
// N dimension carries digit i of activation row m; the epilogue adds a row's digit columns.
#pragma once
#include <stdint.h>

namespace sp {

constexpr int TILE_ROWS = 16;
constexpr int Q4_K_TILE_BYTES = 16 * 144;  // 2304
constexpr int Q6_K_TILE_BYTES = 16 * 210;  // 3360
constexpr int IMMA_MAX_NT = 4;             // n-tiles of 8 digit columns per launch (<= 16 activation rows)

struct ImmaSeg {
    const uint8_t* wt;  // tiled weights
    const float* bias;  // [n] or null
    float* y;           // output base, element (m, r) at y[m * ldy + r]
    int dtype;
    int n;              // real rows
    int ldy;
    int bpt;            // Q8_0: 32-blocks per tile
};

struct ImmaArgs {
    ImmaSeg seg[3];
    int nseg;
    int k;
    int m;        // activation rows in this launch (<= 8 * NT / digits)
    int digits;   // 2 or 3
    int ncp;      // padded digit columns = 8 * NT
    int eb;       // columns per activation exponent block: 256 or 32
    int kp;       // k rounded up to 256: column stride of xq
    // Digits: xq[col][kp]; inside each 256-column tile the bytes are ordered [t 0..3][block 0..7][8 B], the 8 B
    // of (t, block) being columns 4t..4t+3 and 16+4t..16+4t+3 of that 32-block (one lane's B fragment).
    const int8_t* xq;
    const float* colscale;  // [k / eb][ncp]
    // Digit sums S of every 32-block (xs32d) and 16-block (xs16d) of a tile, split as S = a + 64 b with a in
    // [-32, 31]: records [k / 256][ncp][32 B] = { a[0..7], 0 x 8, b[0..7], 0 x 8 } resp. { a[0..15], b[0..15] }.
    // They feed one extra mma per tile for the Q4_K minimum term and the Q6_K zero point.
    const int8_t* xs32d;
    const int8_t* xs16d;
    const float* res;       // optional residual for segment 0 (may alias its y)
    int ldres;
    // Tensor-parallel column-split matrix (tp != null): segment 0's outputs are not stored to y but pushed, as partial
    // sums tagged with the exchange number, into the receive area of every rank (tp.cuh); tp_row0 = activation row of
    // this launch's row 0.
    int tp_row0;
    int pad_;
    const struct TpDev* tp;
};

}  // namespace sp
