// The causal decay weighting of the tile kernels, exp(cs_i - cs_j) for j <= i and 0 elsewhere on a 128 x 128
// tile, done per warp on one 32 x 32 block with lane = row.  Two forms are in use, both built on a reference
// cs per block of 32 so that no factor can overflow:
//
//  * folded (output kernel, dB/dC kernel; code in those kernels):
//      exp(cs_i - cs_j) = exp(cs_i - c0) * exp(c0 - cs_j),   c0 = cs of the first row of the COLUMN block of j.
//    The second factor (>= 1, bounded by the decay across 32 tokens) is multiplied into the rows of the tile that
//    carries index j when that tile is split for the tensor core, so the accumulator arrives carrying it and the
//    pass multiplies a whole block of a row by the one scalar exp(cs_i - c0), with no table.
//  * table driven (dx kernel, below): one table of 128 entries per head and one exp per thread.
//
// In both, a block whose decay exceeds e^60 (or whose cs increases) takes the exact path: one exp per element,
// with the select applied to the exponent BEFORE the exp.
#pragma once

#include "ssd_tile.cuh"

namespace ssd {

constexpr float kDecayFastLimit = 60.f;

// ---- the table-driven form, for a tile held transposed (rows j, columns i):
//   v[j,i] <- v[j,i] * exp(cs_i - cs_j)  for i >= j,   0  for i < j
// Here exp(cs_i - cs_j) = exp(cs_i - ref) * exp(ref - cs_j) with ref = cs of the first column of the COLUMN
// block, so one table of 128 entries serves every block: ei[i] = exp(cs_i - cs[32*(i/32)]) (exponent <= 0 for
// cs non-increasing), and the row factor is one exp per thread (<= 1 right of the diagonal block; inside it
// bounded by the decay across 32 tokens, with the same exact fallback).
constexpr int kDecayColTableFloats = kTile;

// Entry of row `row`: cs_row = cs of that row, ref = cs of row 32 * (row / 32).
__device__ __forceinline__ float decay_col_table_entry(float cs_row, float ref) {
    return __expf(fminf(cs_row - ref, 80.f));
}

// v: the 32 values of row j = 32*qr + lane in columns [32*c, 32*c+32).
__device__ __forceinline__ void decay_block_upper(float* v, int j, int qr, int c, const float* cs_s, const float* ei) {
    if (c < qr) {
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) v[ii] = 0.f;
        return;
    }
    const float ref = cs_s[32 * c];
    const float* t = ei + 32 * c;
    if (c > qr) {
        const float fj = __expf(fminf(ref - cs_s[j], 80.f));
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) v[ii] *= fj * t[ii];
        return;
    }
    const float span = ref - cs_s[32 * qr + 31];  // decay across the diagonal block (warp-uniform)
    if (span >= 0.f && span < kDecayFastLimit) {
        const float fj = __expf(ref - cs_s[j]);
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) v[ii] = (32 * c + ii >= j) ? v[ii] * (fj * t[ii]) : 0.f;
    } else {
        const float csj = cs_s[j];
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) {
            const int i = 32 * c + ii;
            const float e = __expf(i >= j ? cs_s[i] - csj : 0.f);
            v[ii] = i >= j ? v[ii] * e : 0.f;
        }
    }
}

}  // namespace ssd
