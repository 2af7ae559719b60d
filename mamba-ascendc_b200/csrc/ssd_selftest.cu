// Tile-level check of the tensor-core building blocks: TMA fp32 tile load,
// split-bf16 operand conversion, tcgen05.mma in all four operand-major
// combinations, TMEM read-back.  One CTA, D[128 x n] = A * B^T with K = 128.
#include "ssd_host.h"
#include "ssd_tile.cuh"


namespace ssd {

namespace {

constexpr int kStThreads = 256;
constexpr int kM = 128;
constexpr int kK = 128;

struct SelftestSmem {
    // every tile: 128 rows x 128 columns bf16 (two 64-column blocks) = 32 KB
    static constexpr uint32_t kTile = 128 * 128 * 2;
    static constexpr uint32_t kAHi = 0;
    static constexpr uint32_t kALo = kAHi + kTile;
    static constexpr uint32_t kBHi = kALo + kTile;
    static constexpr uint32_t kBLo = kBHi + kTile;
    static constexpr uint32_t kStage = kBLo + kTile;  // 128 rows x 128 B
    static constexpr uint32_t kBars = kStage + 128 * 128;
    static constexpr uint32_t kTotal = kBars + 64;
};

__global__ void __launch_bounds__(kStThreads, 1)
selftest_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float* d, int n,
                int a_mn, int b_mn, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + SelftestSmem::kBars);
    uint64_t* bar_mma = bar_tma + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 128);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // operand tiles: rows x cols as given in global memory
    const uint32_t a_rows = a_mn ? kK : kM, a_cols = a_mn ? kM : kK;
    const uint32_t b_rows = b_mn ? kK : n, b_cols = b_mn ? n : kK;
    uint32_t phase = 0;
    bool ok = true;
    for (int which = 0; which < 2; ++which) {
        const CUtensorMap* map = which == 0 ? &map_a : &map_b;
        const uint32_t rows = which == 0 ? a_rows : b_rows, cols = which == 0 ? a_cols : b_cols;
        uint8_t* hi = smem + (which == 0 ? SelftestSmem::kAHi : SelftestSmem::kBHi);
        uint8_t* lo = smem + (which == 0 ? SelftestSmem::kALo : SelftestSmem::kBLo);
        for (uint32_t c0 = 0; c0 < cols; c0 += 32) {
            if (tid == 0) {
                mbar_arrive_expect_tx(bar_tma, rows * 128u);
                tma_load_2d(smem + SelftestSmem::kStage, map, bar_tma, c0, 0);
            }
            ok = mbar_wait(bar_tma, phase, status, kStatusTmaTimeout | wait_site(6, 1)) && ok;
            phase ^= 1;
            convert_slab(smem + SelftestSmem::kStage, hi, lo, rows, c0, nullptr, tid, kStThreads);
            __syncthreads();  // staging is reused by the next box
        }
    }
    fence_proxy_async_smem();
    __syncthreads();

    if (tid == 0) {
        tc_fence_after_sync();
        Operand a{smem_u32(smem + SelftestSmem::kAHi), smem_u32(smem + SelftestSmem::kALo), a_rows, a_mn != 0};
        Operand b{smem_u32(smem + SelftestSmem::kBHi), smem_u32(smem + SelftestSmem::kBLo), b_rows, b_mn != 0};
        issue_gemm_split<kK / 16>(tmem, a, 0, b, 0, make_idesc_bf16(kM, n, a_mn != 0, b_mn != 0), false);
        umma_commit(bar_mma);
    }
    ok = mbar_wait(bar_mma, 0, status, kStatusMmaTimeout | wait_site(6, 2)) && ok;
    tc_fence_after_sync();

    // warps 0-3 take the first half of the columns, warps 4-7 the second
    const uint32_t quarter = warp & 3, half = warp >> 2;
    const uint32_t row = quarter * 32 + lane;
    const uint32_t cols_per_half = n / 2;
    for (uint32_t c = 0; c < cols_per_half; c += 32) {
        const uint32_t col = half * cols_per_half + c;
        float v[32];
        tmem_ld32(tmem + ((quarter * 32u) << 16) + col, v);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(d + row * n + col + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// Same product, but with the tiles loaded by TMA straight into operand-tile memory and split in place
// (tma_tile_2d + split_tile_inplace), two 64-column blocks per operand: [hi | lo] pairs per block.
__global__ void __launch_bounds__(kThreads, 1)
selftest_inplace_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float* d,
                        int n, int a_mn, int b_mn, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + SelftestSmem::kBars);
    uint64_t* bar_mma = bar_tma + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 128);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t a_rows = a_mn ? kK : kM, a_cols = a_mn ? kM : kK;
    const uint32_t b_rows = b_mn ? kK : n, b_cols = b_mn ? n : kK;
    uint8_t* a_tile = smem + SelftestSmem::kAHi;  // 64 KB: up to two [128 x 64] blocks of (hi, lo)
    uint8_t* b_tile = smem + SelftestSmem::kBHi;
    uint32_t phase = 0;
    bool ok = true;
    for (int which = 0; which < 2; ++which) {
        const CUtensorMap* map = which == 0 ? &map_a : &map_b;
        const uint32_t rows = which == 0 ? a_rows : b_rows, cols = which == 0 ? a_cols : b_cols;
        uint8_t* tile = which == 0 ? a_tile : b_tile;
        for (uint32_t cb = 0; cb < cols / 64; ++cb) {
            uint8_t* blk = tile + cb * 2 * rows * 128;
            if (tid == 0) tma_tile_2d(blk, rows, map, bar_tma, 64 * cb, 0);
            ok = mbar_wait(bar_tma, phase, status, kStatusTmaTimeout | wait_site(6, 3)) && ok;
            phase ^= 1;
            split_tile_inplace(blk, rows, nullptr, warp, lane);
        }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after_sync();
        Operand a{smem_u32(a_tile), smem_u32(a_tile) + a_rows * 128, a_rows, a_mn != 0, 2 * a_rows * 128};
        Operand b{smem_u32(b_tile), smem_u32(b_tile) + b_rows * 128, b_rows, b_mn != 0, 2 * b_rows * 128};
        issue_gemm_split<kK / 16>(tmem, a, 0, b, 0, make_idesc_bf16(kM, n, a_mn != 0, b_mn != 0), false);
        umma_commit(bar_mma);
    }
    ok = mbar_wait(bar_mma, 0, status, kStatusMmaTimeout | wait_site(6, 4)) && ok;
    tc_fence_after_sync();
    const int row = (warp & 3) * 32 + lane;
    const int cols_per_warp = n / 4;
    for (int c = 0; c < cols_per_warp; c += 16) {
        const int col = (warp >> 2) * cols_per_warp + c;
        float v[16];
        tmem_ld16(tmem_addr(tmem, warp, col), v);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(d + row * n + col + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// Same product with A held in tensor memory: the fp32 A tile lands in shared memory, each thread splits
// 32 contraction elements of its row into packed bf16 (hi, lo) pairs and writes them to TMEM
// (tcgen05.st); the MMAs then read A from TMEM and only B from shared memory.  A must be K-major.
__global__ void __launch_bounds__(kThreads, 1)
selftest_tmem_a_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float* d,
                       int n, int b_mn, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + SelftestSmem::kBars);
    uint64_t* bar_mma = bar_tma + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_d = tmem, tm_ahi = tmem + 128, tm_alo = tmem + 192;  // D [n], A hi [64], A lo [64]
    const uint32_t b_rows = b_mn ? kK : n, b_cols = b_mn ? n : kK;
    uint8_t* a_tile = smem + SelftestSmem::kAHi;  // fp32 A: two [128 x 64] column blocks of 64 KB in total
    uint8_t* b_tile = smem + SelftestSmem::kBHi;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t cb = 0; cb < kK / 64; ++cb) {
        if (tid == 0) tma_tile_2d(a_tile + cb * 2 * kM * 128, kM, &map_a, bar_tma, 64 * cb, 0);
        ok = mbar_wait(bar_tma, phase, status, kStatusTmaTimeout | wait_site(6, 5)) && ok;
        phase ^= 1;
    }
    for (uint32_t cb = 0; cb < b_cols / 64; ++cb) {
        uint8_t* blk = b_tile + cb * 2 * b_rows * 128;
        if (tid == 0) tma_tile_2d(blk, b_rows, &map_b, bar_tma, 64 * cb, 0);
        ok = mbar_wait(bar_tma, phase, status, kStatusTmaTimeout | wait_site(6, 6)) && ok;
        phase ^= 1;
        split_tile_inplace(blk, b_rows, nullptr, warp, lane);
    }
    {
        // thread: row of its TMEM lane quarter, contraction elements [32*kq, 32*kq + 32)
        const uint32_t row = (warp & 3) * 32 + lane, kq = warp >> 2;
        const uint8_t* src = a_tile + (kq >> 1) * 2 * kM * 128 + (kq & 1) * kM * 128;
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 f = *reinterpret_cast<const float4*>(src + swz(row, c));
            const float v[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float a = v[2 * e], b = v[2 * e + 1];
                const uint32_t h = pack_bf16x2(a, b);
                hi[2 * c + e] = h;
                lo[2 * c + e] = pack_bf16x2(a - __uint_as_float(h << 16), b - __uint_as_float(h & 0xFFFF0000u));
            }
        }
        tmem_st16(tmem_addr(tm_ahi, warp, 16 * kq), hi);
        tmem_st16(tmem_addr(tm_alo, warp, 16 * kq), lo);
        tmem_st_wait();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
        tc_fence_after_sync();
        Operand b{smem_u32(b_tile), smem_u32(b_tile) + b_rows * 128, b_rows, b_mn != 0, 2 * b_rows * 128};
        issue_gemm_split_ta<kK / 16>(tm_d, tm_ahi, tm_alo, b, 0, make_idesc_bf16(kM, n, false, b_mn != 0), false);
        umma_commit(bar_mma);
    }
    ok = mbar_wait(bar_mma, 0, status, kStatusMmaTimeout | wait_site(6, 7)) && ok;
    tc_fence_after_sync();
    const int row = (warp & 3) * 32 + lane;
    const int cols_per_warp = n / 4;
    for (int c = 0; c < cols_per_warp; c += 16) {
        const int col = (warp >> 2) * cols_per_warp + c;
        float v[16];
        tmem_ld16(tmem_addr(tm_d, warp, col), v);
        tmem_ld_wait();
        if (ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(d + row * n + col + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

// A bounded wait that is left to run out: one warp waits on an mbarrier on which nobody ever arrives, with
// no copy and no tensor-core instruction in flight.  After `polls` polls the wait gives up, records
// kStatusTmaTimeout in the status word and the kernel returns normally -- the path every tile kernel takes
// when a load or a product does not complete.
__global__ void __launch_bounds__(32, 1) wait_expiry_kernel(int* status, uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    if (threadIdx.x == 0) mbar_wait(&bar, 0, status, kStatusTmaTimeout, polls);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_selftest_umma(const float* a, const float* b, float* d, int n, int a_mn, int b_mn, int inplace,
                                 int* status, ssd_stream_t stream) {
    using namespace ssd;
    if (!a || !b || !d || !status) return SSD_ERR_NULL;
    if (n != 64 && n != 128) return SSD_ERR_UNSUPPORTED;
    CUtensorMap map_a, map_b;
    int rc = a_mn ? make_tmap_f32_2d(&map_a, a, kK, kM, kK) : make_tmap_f32_2d(&map_a, a, kM, kK, kM);
    if (rc != SSD_OK) return rc;
    rc = b_mn ? make_tmap_f32_2d(&map_b, b, kK, n, kK) : make_tmap_f32_2d(&map_b, b, n, kK, n);
    if (rc != SSD_OK) return rc;
    const size_t smem = SelftestSmem::kTotal + 1024;
    cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (inplace == 2) {
        if (a_mn) return SSD_ERR_UNSUPPORTED;
        cudaFuncSetAttribute(selftest_tmem_a_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
        selftest_tmem_a_kernel<<<1, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, d, n,
                                                                                              b_mn, status);
    } else if (inplace) {
        cudaFuncSetAttribute(selftest_inplace_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
        selftest_inplace_kernel<<<1, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, d, n, a_mn,
                                                                                               b_mn, status);
    } else {
        selftest_kernel<<<1, kStThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, d, n, a_mn,
                                                                                         b_mn, status);
    }
    return launch_status();
}

extern "C" int ssd_selftest_wait_expiry(int* status, int polls, ssd_stream_t stream) {
    using namespace ssd;
    if (!status) return SSD_ERR_NULL;
    if (polls < 1 || polls > 65536) return SSD_ERR_UNSUPPORTED;  // at most a few tens of milliseconds
    wait_expiry_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, static_cast<uint32_t>(polls));
    return launch_status();
}

// Host-side check of the persistent kernels' position arithmetic (TileWalk, ssd_tile.cuh): the first `count`
// heads of CTA `cta` of a grid of `grid` CTAs, each as (group, head, first token, tile index), found the way the
// kernels find them: from the CTA's first tile by `locate` with a growing look-ahead for the even entries and by
// `advance` plus a look-ahead of at most two for the odd ones.
extern "C" int ssd_selftest_tile_walk(const SsdShape* shape, int grid, int cta, int count, int* out) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!out || grid <= 0 || cta < 0 || cta >= grid || count < 0) return SSD_ERR_SHAPE;
    const TileWalk walk(*shape, grid);
    const TilePos first = walk.first(cta);
    TilePos cur = first;
    int hi = 0;
    for (int it = 0; it < count; ++it) {
        const HeadPos w = (it & 1) ? walk.locate(cur, hi, 0) : walk.locate(first, 0, it);
        out[4 * it] = w.g;
        out[4 * it + 1] = w.h;
        out[4 * it + 2] = w.tok0;
        out[4 * it + 3] = w.tile_index;
        if (++hi == walk.heads_per_group) {
            hi = 0;
            walk.advance(cur);
        }
    }
    return SSD_OK;
}

