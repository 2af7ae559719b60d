// Per-tile state contraction  S[p,n] = sum_t (w_t * X[t,p]) * M[t,n]  for every head of one (batch, group,
// tile), on tcgen05 with split-bf16 operands.
//
//   mode 0 (forward):  X = x,    M = B, w_t = q_t * exp(cs_last - cs_t)  -> chunk state U_k
//   mode 1 (backward): X = dout, M = C, w_t = exp(cs_t)                   -> local dS_k
//
// Two heads of the group are stacked along the MMA's M dimension (2 x P = 128), so one instruction group
// yields both heads' [P,N] blocks; M (B or C) is shared by all heads of the group and split once per CTA.
// Both operands are MN-major: the contraction index t runs along the rows of the token-major tiles
// exactly as they arrive from global memory.  Tiles are loaded by TMA straight into operand-tile memory
// and split in place; the finished states are staged in the dead pair buffer and written by TMA.
//
// The kernel is small on purpose: 8 compute warps plus the issuing warp group, one pair buffer, under
// 100 KB of shared memory with dstate 64, so TWO CTAs share an SM.  Inside a CTA the phases of a head pair
// are serial (load, split, product, write-out); the overlap comes from the other CTA on the SM being in a
// different phase, which also hides each CTA's start-up and load latency.
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

constexpr int kCsWarps = 8;                        // compute warps
constexpr int kCsThreads = kCsWarps * 32;
constexpr int kCsLaunch = kCsThreads + 128;        // plus the issuing warp group
constexpr uint32_t kCsIssuerRegs = 32;             // 80 at launch (2 x 384 threads per SM); the issuing group keeps 32 ...
constexpr uint32_t kCsComputeRegs = 104;           // ... and the two computing groups take 24 more each

__device__ __forceinline__ void cs_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int N>
struct ChunkStateSmem {
    static constexpr uint32_t kXTile = kTile * 128 * 2;           // one head: [128 x 64] hi | lo
    static constexpr uint32_t kPair = 2 * kXTile;                 // two heads
    static constexpr uint32_t kMTile = kTile * 128 * 2 * (N / 64);  // [128 x N]: N/64 blocks of hi | lo
    static constexpr uint32_t kX = 0;                             // the pair buffer
    static constexpr uint32_t kM = kX + kPair;
    static constexpr uint32_t kScale = kM + kMTile;               // float[2 sets][2 heads][128]
    static constexpr uint32_t kBars = kScale + 4 * kTile * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};
// two CTAs per SM with dstate 64 (each CTA also takes 1 KB of system shared memory)
static_assert(2 * (ChunkStateSmem<64>::kTotal + 1024) <= 233472, "two state CTAs do not fit one SM");

template <int N>
__global__ void __launch_bounds__(kCsLaunch, (N == 64 ? 2 : 1))
chunk_state_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_m,
                   const __grid_constant__ CUtensorMap map_st, const float* __restrict__ q,
                   const float* __restrict__ cs, SsdShape s, int mode, int* status) {
    using L = ChunkStateSmem<N>;
    constexpr int kBlocks = N / 64;
    extern __shared__ __align__(1024) uint8_t smem[];
    float* scale = reinterpret_cast<float*>(smem + L::kScale);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_x = bars;       // pair buffer has landed
    uint64_t* full_m = bars + 1;   // group operand has landed
    uint64_t* bar_mma = bars + 2;  // product done
    uint64_t* bar_rdy = bars + 3;  // pair split (and accumulator free)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;
    const int h_first = g * heads_per_group;
    const int npairs = (heads_per_group + 1) / 2;

    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need the declared alignment
        if (tid == 0) atomicCAS(status, 0, kStatusSmemAlign);
        return;
    }

    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below, so that no warp is ever
    // left waiting on a barrier that departed warps will not reach.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 3; ++i) mbar_init(&bars[i], 1);
        mbar_init(bar_rdy, kCsWarps);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, N);  // one accumulator [128 x N]
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (tmem_slot[1] != 0) {
        if (warp == 0) tmem_dealloc(tmem, N);
        return;
    }
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;

    // ---- warp 8: issues every tensor-core instruction of the CTA
    if (warp >= kCsWarps) {
        reg_release<kCsIssuerRegs>();  // this warp group hands most of its registers to the computing groups
        if (warp == kCsWarps && lane == 0) {
            const uint32_t sm = smem_u32(smem + L::kM), sx = smem_u32(smem + L::kX);
            const Operand m{sm, sm + kHalf, kTile, true, 2 * kHalf};
            const Operand a{sx, sx + kHalf, kTile, true, 2 * kHalf};  // column blocks = the two heads
            const uint32_t idesc = make_idesc_bf16(128, N, true, true);
            uint32_t pr = 0;
            for (int pair = 0; pair < npairs; ++pair) {
                mbar_wait(bar_rdy, pr, status, kStatusMmaTimeout | wait_site(1, 1));
                pr ^= 1;
                tc_fence_after_sync();
                issue_gemm_split<kTile / 16>(tmem, a, 0, m, 0, idesc, false);
                umma_commit(bar_mma);
            }
        }
        return;
    }
    reg_acquire<kCsComputeRegs>();

    uint8_t* buf = smem + L::kX;
    auto heads_in = [&](int pair) { return (2 * pair + 1 < heads_per_group) ? 2 : 1; };
    auto load_pair = [&](int pair) {
        const int nh = heads_in(pair);
        mbar_arrive_expect_tx(full_x, nh * L::kXTile);
        for (int hh = 0; hh < nh; ++hh)
            tma_tile_3d(buf + hh * L::kXTile, kTile, &map_x, full_x, 0, h_first + 2 * pair + hh, tok0, false);
    };
    if (tid == 0) {
        mbar_arrive_expect_tx(full_m, L::kMTile);
        for (int cb = 0; cb < kBlocks; ++cb)
            tma_tile_3d(smem + L::kM + cb * 2 * kHalf, kTile, &map_m, full_m, 64 * cb, g, tok0, false);
        load_pair(0);
    }

    // per-row weights: one thread per (head of the pair, row); raw (q, cs, cs_last) are fetched one pair
    // ahead into registers and published into the set of that pair's parity
    const int w_hh = tid >> 7, w_t = tid & 127;
    float w_q = 0.f, w_cs = 0.f, w_last = 0.f;
    auto fetch_rows = [&](int pair) {
        if (w_hh < heads_in(pair)) {
            const size_t row = (static_cast<size_t>(b) * s.nheads + h_first + 2 * pair + w_hh) * s.seqlen + k * kTile;
            w_cs = cs[row + w_t];
            w_last = cs[row + kTile - 1];
            w_q = q[row + w_t];
        }
    };
    auto publish_rows = [&](int pair) {
        scale[((pair & 1) * 2 + w_hh) * kTile + w_t] = mode == 0 ? w_q * expf(w_last - w_cs) : expf(w_cs);
    };
    fetch_rows(0);
    publish_rows(0);
    if (npairs > 1) fetch_rows(1);

    ok = mbar_wait(full_m, 0, status, kStatusTmaTimeout | wait_site(1, 2)) && ok;
    for (int cb = 0; cb < kBlocks; ++cb) {
        split_tile_inplace(smem + L::kM + cb * 2 * kHalf, kTile, nullptr, warp, lane);
        split_tile_inplace(smem + L::kM + cb * 2 * kHalf, kTile, nullptr, warp + kCsWarps, lane);
    }
    cs_sync();  // weights of the first pair are visible

    uint32_t px = 0, pm = 0;
    constexpr int kIoThread = 128;  // issues the state stores and the next pair's load
    constexpr uint32_t kOutSlab = 64 * 128;
    for (int pair = 0; pair < npairs; ++pair) {
        const int h0 = h_first + 2 * pair;
        const int nh = heads_in(pair);
        ok = mbar_wait(full_x, px, status, kStatusTmaTimeout | wait_site(1, 3)) && ok;
        px ^= 1;
        {
            const float* sc = scale + (pair & 1) * 2 * kTile;
            if (nh == 2) {  // both heads of the pair at once, per row group
                split_two_tiles_inplace(buf, sc, buf + L::kXTile, sc + kTile, kTile, warp, lane);
                split_two_tiles_inplace(buf, sc, buf + L::kXTile, sc + kTile, kTile, warp + kCsWarps, lane);
            } else {
                split_tile_inplace(buf, kTile, sc, warp, lane);
                split_tile_inplace(buf, kTile, sc, warp + kCsWarps, lane);
            }
        }
        signal_issuer(bar_rdy, lane);
        if (pair + 1 < npairs) publish_rows(pair + 1);  // other set
        if (pair + 2 < npairs) fetch_rows(pair + 2);
        ok = mbar_wait(bar_mma, pm, status, kStatusMmaTimeout | wait_site(1, 4)) && ok;
        pm ^= 1;
        tc_fence_after_sync();

        // epilogue: TMEM row = hh * 64 + p.  The pair buffer is dead now; the fp32 states are staged there as
        // swizzled [64 rows x 32 floats] slabs (index hh * N/32 + c) and written out by TMA in full lines.
        {
            const int row = (warp & 3) * 32 + lane;
            const int hh = row >> 6, p = row & 63;
            const int half = warp >> 2;  // this warp's half of the N columns
#pragma unroll
            for (int c32 = 0; c32 < N / 64; ++c32) {
                const int col0 = half * (N / 2) + 32 * c32;
                float v[32];
                tmem_ld32(tmem_addr(tmem, warp, col0), v);
                tmem_ld_wait();
                uint8_t* slab = buf + (hh * (N / 32) + col0 / 32) * kOutSlab;
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(slab + swz(p, i >> 2)) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cs_sync();  // staged states complete; next pair's weights visible; accumulator free
        if (tid == kIoThread) {
            if (ok) {
                for (int hh = 0; hh < nh; ++hh) {
                    const int row0 = static_cast<int>(((static_cast<size_t>(b) * s.nheads + h0 + hh) * nchunks + k) * 64);
                    for (int c = 0; c < N / 32; ++c)
                        tma_store_2d(&map_st, buf + (hh * (N / 32) + c) * kOutSlab, 32 * c, row0);
                }
                tma_store_commit();
            }
            tma_store_wait_read();  // then the buffer can take the next pair
            if (pair + 1 < npairs) load_pair(pair + 1);
        }
    }
    if (tid == kIoThread) tma_store_wait_all();
    cs_sync();
    if (warp == 0) tmem_dealloc(tmem, N);
}

// ---- dstate 128: two CTAs of the small kernel do not fit one SM, so this shape keeps the 16-warp form: two
// pair buffers and two accumulators, so the product of pair p runs while the compute warps split pair p+1
// and write out pair p-1.
template <int N>
struct ChunkStateWideSmem {
    static constexpr uint32_t kXTile = kTile * 128 * 2;           // one head: [128 x 64] hi | lo
    static constexpr uint32_t kPair = 2 * kXTile;                 // two heads
    static constexpr uint32_t kMTile = kTile * 128 * 2 * (N / 64);  // [128 x N]: N/64 blocks of hi | lo
    static constexpr uint32_t kX = 0;                             // two pair buffers
    static constexpr uint32_t kM = kX + 2 * kPair;
    static constexpr uint32_t kScale = kM + kMTile;               // float[2 buffers][2 heads][128]
    static constexpr uint32_t kBars = kScale + 4 * kTile * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};
static_assert(ChunkStateWideSmem<128>::kTotal + 1024 <= 232448, "wide state kernel exceeds the shared memory of one SM");

template <int N>
__global__ void __launch_bounds__(kLaunchThreadsGroups, 1)
chunk_state_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_m,
                   const __grid_constant__ CUtensorMap map_st, const float* __restrict__ q,
                   const float* __restrict__ cs, SsdShape s, int mode, int* status) {
    using L = ChunkStateWideSmem<N>;
    constexpr int kBlocks = N / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* scale = reinterpret_cast<float*>(smem + L::kScale);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_x = bars;       // [2] pair buffer has landed
    uint64_t* full_m = bars + 2;   // group operand has landed
    uint64_t* bar_mma = bars + 3;  // [2] product done, by pair parity
    uint64_t* bar_rdy = bars + 5;  // [2] pair split (and its accumulator free), by pair parity
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;
    const int h_first = g * heads_per_group;
    const int npairs = (heads_per_group + 1) / 2;


    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below, so that no warp is ever
    // left waiting on a barrier that departed warps will not reach.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
        mbar_init(&bar_rdy[0], kThreads / 32);
        mbar_init(&bar_rdy[1], kThreads / 32);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 2 * N);  // two accumulators [128 x N], by pair parity
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (tmem_slot[1] != 0) {
        if (warp == 0) tmem_dealloc(tmem, 2 * N);
        return;
    }
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;

    // ---- warp 16: issues every tensor-core instruction of the CTA
    if (warp >= kThreads / 32) {
        reg_release<kIssuerRegs>();  // this warp group hands most of its registers to the computing groups
        if (warp == kThreads / 32 && lane == 0) {
            const uint32_t sm = smem_u32(smem + L::kM);
            const Operand m{sm, sm + kHalf, kTile, true, 2 * kHalf};
            const uint32_t idesc = make_idesc_bf16(128, N, true, true);
            uint32_t pr = 0;  // one parity bit per buffer
            for (int pair = 0; pair < npairs; ++pair) {
                const int pb = pair & 1;
                const uint32_t sx = smem_u32(smem + L::kX + pb * L::kPair);
                const Operand a{sx, sx + kHalf, kTile, true, 2 * kHalf};  // column blocks = the two heads
                mbar_wait(&bar_rdy[pb], (pr >> pb) & 1u, status, kStatusMmaTimeout | wait_site(1, 5));
                pr ^= 1u << pb;
                tc_fence_after_sync();
                issue_gemm_split<kTile / 16>(tmem + pb * N, a, 0, m, 0, idesc, false);
                umma_commit(&bar_mma[pb]);
            }
        }
        return;
    }
    reg_acquire<kComputeRegs>();

    auto pair_buf = [&](int pair) { return smem + L::kX + (pair & 1) * L::kPair; };
    auto heads_in = [&](int pair) { return (2 * pair + 1 < heads_per_group) ? 2 : 1; };
    auto load_pair = [&](int pair) {
        const int nh = heads_in(pair);
        mbar_arrive_expect_tx(&full_x[pair & 1], nh * L::kXTile);
        for (int hh = 0; hh < nh; ++hh)
            tma_tile_3d(pair_buf(pair) + hh * L::kXTile, kTile, &map_x, &full_x[pair & 1], 0, h_first + 2 * pair + hh,
                        tok0, false);
    };
    if (tid == 0) {
        mbar_arrive_expect_tx(full_m, L::kMTile);
        for (int cb = 0; cb < kBlocks; ++cb)
            tma_tile_3d(smem + L::kM + cb * 2 * kHalf, kTile, &map_m, full_m, 64 * cb, g, tok0, false);
        load_pair(0);
        if (npairs > 1) load_pair(1);
    }

    // per-row weights: raw (q, cs, cs_last) of a pair are fetched one pair ahead into registers
    const int w_hh = tid >> 7, w_t = tid & 127;
    float w_q = 0.f, w_cs = 0.f, w_last = 0.f;
    auto fetch_rows = [&](int pair) {
        if (w_hh < heads_in(pair)) {
            const size_t row = (static_cast<size_t>(b) * s.nheads + h_first + 2 * pair + w_hh) * s.seqlen + k * kTile;
            w_cs = cs[row + w_t];
            w_last = cs[row + kTile - 1];
            w_q = q[row + w_t];
        }
    };
    auto publish_rows = [&](int pair) {
        if (w_hh < 2) scale[((pair & 1) * 2 + w_hh) * kTile + w_t] = mode == 0 ? w_q * expf(w_last - w_cs) : expf(w_cs);
    };
    fetch_rows(0);
    publish_rows(0);
    if (npairs > 1) fetch_rows(1);

    ok = mbar_wait(full_m, 0, status, kStatusTmaTimeout | wait_site(1, 6)) && ok;
    for (int cb = 0; cb < kBlocks; ++cb) split_tile_inplace(smem + L::kM + cb * 2 * kHalf, kTile, nullptr, warp, lane);
    cta_sync();  // weights of the first pair are visible

    uint32_t px = 0, pm = 0;  // one parity bit per buffer
    constexpr int kIoThread = 256;  // issues the state stores
    constexpr uint32_t kOutSlab = 64 * 128;

    // Pair ready for the tensor core: tiles split in place (scaled by the row weights).
    auto split_pair = [&](int pair) {
        const int pb = pair & 1;
        uint8_t* buf = pair_buf(pair);
        ok = mbar_wait(&full_x[pb], (px >> pb) & 1u, status, kStatusTmaTimeout | wait_site(1, 7)) && ok;
        px ^= 1u << pb;
        for (int hh = 0; hh < heads_in(pair); ++hh)
            split_tile_inplace(buf + hh * L::kXTile, kTile, scale + (pb * 2 + hh) * kTile, warp, lane);
        signal_issuer(&bar_rdy[pb], lane);
    };
    // Pair finished: TMEM row = hh * 64 + p.  The pair buffer is dead now; the fp32 states are staged there as
    // swizzled [64 rows x 32 floats] slabs (index hh * N/32 + c) and written out by TMA in full lines.
    auto write_pair = [&](int pair) {
        const int pb = pair & 1;
        const int h0 = h_first + 2 * pair;
        const int nh = heads_in(pair);
        uint8_t* buf = pair_buf(pair);
        ok = mbar_wait(&bar_mma[pb], (pm >> pb) & 1u, status, kStatusMmaTimeout | wait_site(1, 8)) && ok;
        pm ^= 1u << pb;
        tc_fence_after_sync();
        {
            const int row = (warp & 3) * 32 + lane;
            const int hh = row >> 6, p = row & 63;
            constexpr int kColsPerWarp = N / 4;
            const int col0 = (warp >> 2) * kColsPerWarp;
            float v[kColsPerWarp];
            if constexpr (kColsPerWarp == 32) {
                tmem_ld32(tmem_addr(tmem + pb * N, warp, col0), v);
            } else {
                tmem_ld16(tmem_addr(tmem + pb * N, warp, col0), v);
            }
            tmem_ld_wait();
            uint8_t* slab = buf + (hh * (N / 32) + col0 / 32) * kOutSlab;
#pragma unroll
            for (int i = 0; i < kColsPerWarp; i += 4)
                *reinterpret_cast<float4*>(slab + swz(p, ((col0 & 31) + i) >> 2)) =
                    make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();  // staged states complete; weights published before this are visible
        if (tid == kIoThread) {
            if (ok) {
                for (int hh = 0; hh < nh; ++hh) {
                    const int row0 = static_cast<int>(((static_cast<size_t>(b) * s.nheads + h0 + hh) * nchunks + k) * 64);
                    for (int c = 0; c < N / 32; ++c)
                        tma_store_2d(&map_st, buf + (hh * (N / 32) + c) * kOutSlab, 32 * c, row0);
                }
                tma_store_commit();
            }
            tma_store_wait_read();  // then the buffer can take pair + 2
            if (pair + 2 < npairs) load_pair(pair + 2);
        }
    };

    // Pipeline: split(p) -> [tensor core: product p] ; meanwhile write(p - 1).  The weights of pair p + 1 are
    // published before the barrier inside write(p - 1) (or the one below for the first pair).
    for (int pair = 0; pair < npairs; ++pair) {
        split_pair(pair);
        if (pair + 1 < npairs) publish_rows(pair + 1);  // other buffer's weights
        if (pair + 2 < npairs) fetch_rows(pair + 2);
        if (pair > 0) {
            write_pair(pair - 1);
        } else if (npairs > 1) {
            cta_sync();  // weights of the second pair are visible
        }
    }
    write_pair(npairs - 1);
    if (tid == kIoThread) tma_store_wait_all();
    cta_sync();
    if (warp == 0) tmem_dealloc(tmem, 2 * N);
}

template <int N>
int launch_chunk_state(const SsdShape& s, const float* x, const float* m, const float* q, const float* cs,
                       float* states, int mode, int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_m, map_st;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc != SSD_OK) return rc;
    rc = make_tmap_f32_tokens(&map_m, m, tokens, s.ngroups, s.dstate, kTile);
    if (rc != SSD_OK) return rc;
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    rc = make_tmap_f32_2d(&map_st, states, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
    if constexpr (N == 64) {
        const size_t smem = ChunkStateSmem<N>::kTotal;
        static std::atomic<uint64_t> smem_set{0};
        rc = set_max_smem_once(reinterpret_cast<const void*>(chunk_state_kernel<N>), smem, smem_set);
        if (rc != SSD_OK) return rc;
        chunk_state_kernel<N><<<grid, kCsLaunch, smem, stream>>>(map_x, map_m, map_st, q, cs, s, mode, status);
    } else {
        const size_t smem = ChunkStateWideSmem<N>::kTotal + 1024;
        static std::atomic<uint64_t> smem_set{0};
        rc = set_max_smem_once(reinterpret_cast<const void*>(chunk_state_wide_kernel<N>), smem, smem_set);
        if (rc != SSD_OK) return rc;
        chunk_state_wide_kernel<N><<<grid, kLaunchThreadsGroups, smem, stream>>>(map_x, map_m, map_st, q, cs, s, mode,
                                                                                 status);
    }
    return launch_status();
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_state(const SsdShape* shape, const float* x, const float* m, const float* q, const float* cs,
                               float* states, int mode, int* status, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!x || !m || !q || !cs || !states || !status) return SSD_ERR_NULL;
    if (mode != 0 && mode != 1) return SSD_ERR_UNSUPPORTED;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    return shape->dstate == 64 ? launch_chunk_state<64>(*shape, x, m, q, cs, states, mode, status, st)
                               : launch_chunk_state<128>(*shape, x, m, q, cs, states, mode, status, st);
}
