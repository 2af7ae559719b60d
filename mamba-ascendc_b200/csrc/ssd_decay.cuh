// The causal decay weighting shared by the forward and backward tile kernels:
//   v[i,j] <- v[i,j] * exp(cs_i - cs_j)  for j <= i,   0  for j > i        (one 128 x 128 tile)
// done per warp on one 32 x 32 block (rows 32*qr.., columns 32*c..), lane = row.
//
// Blocks above the diagonal are zero.  The diagonal blocks take one exp per
// element, with the select applied to the exponent BEFORE the exp (the masked
// half would overflow, cs decreases along the tile).  Blocks below the diagonal
// use exp(cs_i - cs_j) = exp(cs_i - ref) * exp(ref - cs_j) with ref = cs of the
// block's first row: both exponents are <= 0, so neither factor overflows, and
// the second factor comes from a small table filled once per head
// (ej[qr-1][j] for j < 32*qr), which leaves two multiplies per element.
#pragma once

#include "ssd_tile.cuh"

namespace ssd {

constexpr int kDecayTableFloats = 3 * kTile;

// Called by thread `row` (0..127) when it publishes its row's cs: fills the
// table entries of column `row`.  ref[q] = cs of row 32*(q+1), q = 0..2.
__device__ __forceinline__ void decay_table_fill(float* ej, int row, float cs_row, const float* ref) {
#pragma unroll
    for (int q = 0; q < 3; ++q) {
        if (row < 32 * (q + 1)) ej[q * kTile + row] = __expf(ref[q] - cs_row);
    }
}

// v: the 32 values of row i = 32*qr + lane in columns [32*c, 32*c+32).
__device__ __forceinline__ void decay_block_lower(float* v, int i, int qr, int c, const float* cs_s, const float* ej) {
    if (c > qr) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) v[jj] = 0.f;
    } else if (c == qr) {
        const float csi = cs_s[i];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
            const int j = 32 * c + jj;
            const float e = __expf(j <= i ? csi - cs_s[j] : 0.f);
            v[jj] = j <= i ? v[jj] * e : 0.f;
        }
    } else {
        const float ei = __expf(cs_s[i] - cs_s[32 * qr]);
        const float* t = ej + (qr - 1) * kTile + 32 * c;
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) v[jj] *= ei * t[jj];
    }
}

}  // namespace ssd
