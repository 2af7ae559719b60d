// The causal decay weighting shared by the forward and backward tile kernels:
//   v[i,j] <- v[i,j] * exp(cs_i - cs_j)  for j <= i,   0  for j > i        (one 128 x 128 tile)
// done per warp on one 32 x 32 block (rows 32*qr.., columns 32*c..), lane = row.
//
// Blocks above the diagonal are zero.  Everywhere else
//   exp(cs_i - cs_j) = exp(cs_i - ref) * exp(ref - cs_j),   ref = cs of the first row of the ROW block,
// so the inner loop is a table read and two multiplies, with no exp on its dependency chain (32
// dependent exp chains per thread do not fit the register budget and end up serialised).  The first
// factor is one exp per thread (exponent <= 0 for cs non-increasing).  The second comes from a table
// filled once per head: ej[qr][j] = exp(cs[32*qr] - cs_j) for j < 32*(qr+1).  Below the diagonal block
// its exponent is <= 0; inside the diagonal block it is >= 0 and bounded by the decay across 32 tokens.
// If that decay exceeds e^60 (or cs increases) the diagonal block falls back to one exp per element,
// with the select applied to the exponent BEFORE the exp, so nothing can overflow.
#pragma once

#include "ssd_tile.cuh"

namespace ssd {

// Two layouts: one row of 128 floats per row block, or (COMPACT) the rows stored back to back.
constexpr int kDecayTableFloats = 4 * kTile;
constexpr int kDecayTableFloatsCompact = 32 + 64 + 96 + 128;
template <bool COMPACT>
__device__ __forceinline__ constexpr int decay_table_row(int q) {
    return COMPACT ? 16 * q * (q + 1) : q * kTile;
}
constexpr float kDecayFastLimit = 60.f;

// Called by thread `row` (0..127) when it publishes its row's cs: fills the table entries of column
// `row`.  ref[q] = cs of row 32*q, q = 0..3.
template <bool COMPACT = false>
__device__ __forceinline__ void decay_table_fill(float* ej, int row, float cs_row, const float* ref) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (row < 32 * (q + 1)) ej[decay_table_row<COMPACT>(q) + row] = __expf(fminf(ref[q] - cs_row, 80.f));
    }
}

// v: the W values of row i = 32*qr + lane in columns [32*c + col_off, 32*c + col_off + W)  (W = 32 or 16).
template <bool COMPACT = false, int W = 32>
__device__ __forceinline__ void decay_block_lower(float* v, int i, int qr, int c, const float* cs_s, const float* ej,
                                                  int col_off = 0) {
    if (c > qr) {
#pragma unroll
        for (int jj = 0; jj < W; ++jj) v[jj] = 0.f;
        return;
    }
    const float ref = cs_s[32 * qr];
    const int col0 = 32 * c + col_off;
    const float* t = ej + decay_table_row<COMPACT>(qr) + col0;
    if (c < qr) {
        const float ei = __expf(cs_s[i] - ref);
#pragma unroll
        for (int jj = 0; jj < W; ++jj) v[jj] *= ei * t[jj];
        return;
    }
    const float span = ref - cs_s[32 * qr + 31];  // decay across the diagonal block (warp-uniform)
    if (span >= 0.f && span < kDecayFastLimit) {
        const float ei = __expf(cs_s[i] - ref);
#pragma unroll
        for (int jj = 0; jj < W; ++jj) v[jj] = (col0 + jj <= i) ? v[jj] * (ei * t[jj]) : 0.f;
    } else {
        const float csi = cs_s[i];
#pragma unroll
        for (int jj = 0; jj < W; ++jj) {
            const int j = col0 + jj;
            const float e = __expf(j <= i ? csi - cs_s[j] : 0.f);
            v[jj] = j <= i ? v[jj] * e : 0.f;
        }
    }
}

// ---- the mirrored form, for a tile held transposed (rows j, columns i):
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
