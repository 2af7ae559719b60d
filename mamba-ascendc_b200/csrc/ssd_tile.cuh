// Pieces every SSD tile kernel shares on top of ssd_umma.cuh: the CTA shape and its barriers, the hand-off
// to the issuing warp, fp32 tiles loaded by TMA into operand-tile memory and split in place, and the TMEM
// addressing of the compute warps.
//
// CTA shape of the large kernels: 512 compute threads = 16 warps, one CTA per SM (the state kernel for
// dstate 64 uses 8 compute warps and two CTAs per SM instead).  A token tile has 128 rows; TMEM lane == row.
// Warp w may only touch TMEM lanes [32*(w%4), 32*(w%4)+32), so the four warps w, w+4, w+8, w+12 share rows
// and split the columns four ways (column group = w / 4).
#pragma once

#include "../../include/ssd_b200.h"
#include "ssd_umma.cuh"

namespace ssd {

constexpr int kThreads = 512;              // compute threads (16 warps)
// Launch size: the 16 compute warps plus a fifth warp group whose first warp only issues tensor-core
// instructions; in the persistent kernels its second warp issues every TMA load and store and its third
// publishes the per-head rows (the remaining warps leave at once).  A whole group, because register trading
// (reg_release / reg_acquire) works on groups of four warps: a 17th warp alone would cap every thread at
// 96 registers (five warps on one scheduler share its 512 registers per lane).  The registers traded are the
// CTA's own (640 x 96 at launch): with 112 for the compute groups the fifth group cannot keep more than 32.
constexpr int kLaunchThreadsGroups = kThreads + 128;
constexpr uint32_t kIssuerRegs = 32;    // 96 at launch (640 threads): the issuing group keeps 32 ...
constexpr uint32_t kComputeRegs = 112;  // ... and each of the four computing groups takes 16 more

// Barrier over the 512 compute threads only (named barrier 1); the MMA-issuing warp never joins it.
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// Compute warps -> issuing warp hand-off.  Every compute thread makes its shared-memory writes visible to
// the async proxy and orders its TMEM reads, then one lane per warp arrives (the barrier is initialised
// with a count of 16).  The issuing thread waits on the barrier before it issues.
__device__ __forceinline__ void signal_issuer(uint64_t* bar, int lane) {
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
constexpr int kTile = 128;            // tokens per tile (T)
constexpr uint32_t kSlabBytes = 128 * 128;  // one staged box: 128 rows x 32 floats

// ---------------------------------------------------------------- work items of a persistent CTA
// The persistent kernels walk the (batch, group, token tile) grid, token tile fastest: CTA c takes tiles c,
// c + gridDim.x, ... and, inside a tile, the heads of the group in sequence.  Positions are advanced without
// divisions (three at kernel start), so that the warp that issues the loads has the next coordinates ready
// before the barrier that frees their memory flips.
struct TilePos {
    int b, g, k;
};
struct HeadPos {
    int g, h, tok0;
    int tile_index;  // (batch, head, token tile) index: first row of q / cs over 128, state row over 64
};
struct TileWalk {
    int nchunks, ngroups, nheads, seqlen, heads_per_group, step_k, step_g, step_b;
    __host__ __device__ __forceinline__ TileWalk(const SsdShape& s, int grid)
        : nchunks(s.seqlen / 128), ngroups(s.ngroups), nheads(s.nheads), seqlen(s.seqlen),
          heads_per_group(s.nheads / s.ngroups) {
        step_k = grid % nchunks;
        step_g = (grid / nchunks) % ngroups;
        step_b = grid / (nchunks * ngroups);
    }
    __host__ __device__ __forceinline__ TilePos first(int tile) const {
        TilePos t;
        t.k = tile % nchunks;
        t.g = (tile / nchunks) % ngroups;
        t.b = tile / (nchunks * ngroups);
        return t;
    }
    __host__ __device__ __forceinline__ void advance(TilePos& t) const {  // the CTA's next tile
        t.k += step_k;
        if (t.k >= nchunks) {
            t.k -= nchunks;
            ++t.g;
        }
        t.g += step_g;
        if (t.g >= ngroups) {
            t.g -= ngroups;
            ++t.b;
        }
        t.b += step_b;
    }
    // The head `ahead` heads after head `hi` of tile `t` in the CTA's sequence.
    __host__ __device__ __forceinline__ HeadPos locate(TilePos t, int hi, int ahead) const {
        hi += ahead;
        while (hi >= heads_per_group) {
            hi -= heads_per_group;
            advance(t);
        }
        HeadPos w;
        w.g = t.g;
        w.h = t.g * heads_per_group + hi;
        w.tok0 = t.b * seqlen + t.k * 128;
        w.tile_index = (t.b * nheads + w.h) * nchunks + t.k;
        return w;
    }
};

// ---------------------------------------------------------------- tiles loaded and split in place
// A [rows x 64] fp32 tile occupies exactly the bytes of its bf16 hi tile plus its lo tile.  TMA
// therefore writes the fp32 data straight into the operand tile's own memory -- columns 0..31 where
// the hi tile will be, columns 32..63 where the lo tile will be, both as swizzled 128-byte rows -- and
// the threads split it in place: no staging buffer, and the load can be issued as soon as the tile's
// previous consumer (an MMA) has finished, a whole head ahead of its use.
// `expect` = false: the caller has already announced the bytes of several tiles on `bar` in one go.
__device__ __forceinline__ void tma_tile_3d(uint8_t* tile, uint32_t rows, const CUtensorMap* m, uint64_t* bar, int col0,
                                            int c1, int c2, bool expect = true) {
    if (expect) mbar_arrive_expect_tx(bar, 2u * rows * 128u);
    tma_load_3d(tile, m, bar, col0, c1, c2);
    tma_load_3d(tile + rows * 128u, m, bar, col0 + 32, c1, c2);
}
__device__ __forceinline__ void tma_tile_2d(uint8_t* tile, uint32_t rows, const CUtensorMap* m, uint64_t* bar, int col0,
                                            int c1, bool expect = true) {
    if (expect) mbar_arrive_expect_tx(bar, 2u * rows * 128u);
    tma_load_2d(tile, m, bar, col0, c1);
    tma_load_2d(tile + rows * 128u, m, bar, col0 + 32, c1);
}

// Split such a tile in place.  Four threads share a row (16 floats each); a warp covers 8 rows, warps
// 0 .. rows/8-1 take part and the whole of each must call.  Thread (r, qd) reads floats [16qd, 16qd+16)
// and writes bf16 chunks 2qd, 2qd+1 of the hi and of the lo row; the __syncwarp between the reads and
// the writes is what makes the in-place update safe (a row never leaves its warp).  Lanes of a
// quarter-warp hold 8 different rows, so every 16-byte access is free of bank conflicts.
// `after(r, qd, v)` sees the 16 (scaled) values, e.g. to form row sums.
template <class AfterF>
__device__ __forceinline__ void split_tile_inplace(uint8_t* tile, uint32_t rows, const float* scale, int warp, int lane,
                                                   AfterF after) {
    if (static_cast<uint32_t>(warp) * 8u >= rows) return;
    const uint32_t r = static_cast<uint32_t>(warp) * 8u + (lane & 7);
    const uint32_t qd = static_cast<uint32_t>(lane) >> 3;
    uint8_t* hi = tile;
    uint8_t* lo = tile + rows * 128u;
    const uint8_t* src = (qd >> 1) ? lo : hi;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 f = *reinterpret_cast<const float4*>(src + swz(r, (qd & 1) * 4 + i));
        v[4 * i] = f.x;
        v[4 * i + 1] = f.y;
        v[4 * i + 2] = f.z;
        v[4 * i + 3] = f.w;
    }
    if (scale != nullptr) {
        const float sc = scale[r];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= sc;
    }
    after(r, qd, v);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 h, l;
        split8(v + 8 * i, h, l);
        const uint32_t off = swz(r, 2 * qd + i);
        *reinterpret_cast<uint4*>(hi + off) = h;
        *reinterpret_cast<uint4*>(lo + off) = l;
    }
}
__device__ __forceinline__ void split_tile_inplace(uint8_t* tile, uint32_t rows, const float* scale, int warp,
                                                   int lane) {
    split_tile_inplace(tile, rows, scale, warp, lane, [](uint32_t, uint32_t, const float*) {});
}

// The same with the scale of this thread's row (row 8 * warp + (lane & 7)) already in a register;
// `before(r, qd, v)` sees the 16 values as they landed, before they are scaled.
template <class BeforeF>
__device__ __forceinline__ void split_tile_inplace_scaled(uint8_t* tile, uint32_t rows, float sc, int warp, int lane,
                                                          BeforeF before) {
    if (static_cast<uint32_t>(warp) * 8u >= rows) return;
    const uint32_t r = static_cast<uint32_t>(warp) * 8u + (lane & 7);
    const uint32_t qd = static_cast<uint32_t>(lane) >> 3;
    uint8_t* hi = tile;
    uint8_t* lo = tile + rows * 128u;
    const uint8_t* src = (qd >> 1) ? lo : hi;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 f = *reinterpret_cast<const float4*>(src + swz(r, (qd & 1) * 4 + i));
        v[4 * i] = f.x;
        v[4 * i + 1] = f.y;
        v[4 * i + 2] = f.z;
        v[4 * i + 3] = f.w;
    }
    before(r, qd, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= sc;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 h, l;
        split8(v + 8 * i, h, l);
        const uint32_t off = swz(r, 2 * qd + i);
        *reinterpret_cast<uint4*>(hi + off) = h;
        *reinterpret_cast<uint4*>(lo + off) = l;
    }
}
__device__ __forceinline__ void split_tile_inplace_scaled(uint8_t* tile, uint32_t rows, float sc, int warp, int lane) {
    split_tile_inplace_scaled(tile, rows, sc, warp, lane, [](uint32_t, uint32_t, const float*) {});
}

// Two tiles of the same height at once (the loads of both are in flight together, one warp barrier).
__device__ __forceinline__ void split_two_tiles_inplace(uint8_t* tile_a, const float* scale_a, uint8_t* tile_b,
                                                        const float* scale_b, uint32_t rows, int warp, int lane) {
    if (static_cast<uint32_t>(warp) * 8u >= rows) return;
    const uint32_t r = static_cast<uint32_t>(warp) * 8u + (lane & 7);
    const uint32_t qd = static_cast<uint32_t>(lane) >> 3;
    const uint32_t half = rows * 128u;
    const uint32_t src_off = (qd >> 1) ? half : 0u;
    float va[16], vb[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 fa = *reinterpret_cast<const float4*>(tile_a + src_off + swz(r, (qd & 1) * 4 + i));
        const float4 fb = *reinterpret_cast<const float4*>(tile_b + src_off + swz(r, (qd & 1) * 4 + i));
        va[4 * i] = fa.x;
        va[4 * i + 1] = fa.y;
        va[4 * i + 2] = fa.z;
        va[4 * i + 3] = fa.w;
        vb[4 * i] = fb.x;
        vb[4 * i + 1] = fb.y;
        vb[4 * i + 2] = fb.z;
        vb[4 * i + 3] = fb.w;
    }
    if (scale_a != nullptr) {
        const float sc = scale_a[r];
#pragma unroll
        for (int i = 0; i < 16; ++i) va[i] *= sc;
    }
    if (scale_b != nullptr) {
        const float sc = scale_b[r];
#pragma unroll
        for (int i = 0; i < 16; ++i) vb[i] *= sc;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 h, l;
        const uint32_t off = swz(r, 2 * qd + i);
        split8(va + 8 * i, h, l);
        *reinterpret_cast<uint4*>(tile_a + off) = h;
        *reinterpret_cast<uint4*>(tile_a + half + off) = l;
        split8(vb + 8 * i, h, l);
        *reinterpret_cast<uint4*>(tile_b + off) = h;
        *reinterpret_cast<uint4*>(tile_b + half + off) = l;
    }
}

// TMEM address of (lane quarter of this warp, column).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int warp, uint32_t col) {
    return base + ((static_cast<uint32_t>(warp & 3) * 32u) << 16) + col;
}

// Round a shared-memory pointer up to 1024 bytes by ADDING an offset, so that the compiler still
// knows the result points to shared memory (an integer round trip would turn every later access
// into a generic load / store).
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
    const uint32_t a = smem_u32(p);
    return p + ((1024u - (a & 1023u)) & 1023u);
}

// Numerically plain softplus with torch's threshold (F.softplus: x for x > 20).
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

}  // namespace ssd
