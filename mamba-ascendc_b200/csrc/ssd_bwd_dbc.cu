// Backward kernel for dB and dC.  One persistent CTA per SM walks its share of the (batch, group, tile of
// 128 tokens) work items.  Four roles: 16 compute warps; one warp that only issues tensor-core instructions;
// one producer warp that issues every TMA load and store; one warp that publishes each head's rows (cs, q).
// The compute warps meet at a CTA barrier once per tile only (when the finished gradients are staged): inside a tile
// every hand-off is an mbarrier, so a warp with little to do in one phase runs ahead into the next head's
// split while the others finish.  The gradient of the group is accumulated over its heads inside the CTA, so
// each output element is written once by one CTA (no atomics, fixed order).
// Per head h (xdt = q .* x, S = state at the start of the tile, dU = gradient of the state after the tile):
//
//   D0[i,j]  = sum_p dout[i,p] * xdt[j,p]                    tcgen05, N = 128  (A = dout from tensor memory)
//   T[i,n]   = sum_p dout[i,p] * S[p,n]                      tcgen05   (state-to-output term of dC; A = dout again)
//   V[j,n]   = sum_p xdt[j,p]  * dU[p,n]                     tcgen05   (chunk-state term of dB)
//   dCB[i,j] += D0[i,j] * exp(cs_i - cs_j)  for j <= i                 TMEM -> fp32 registers, fixed head order
//   regC    += exp(cs_i) .* T ;  regB += exp(cs_last - cs_j) .* V      fp32 registers, fixed head order
//
// and once per tile, with dCB summed over the heads of the group (B and C are the group's, so the sum
// commutes with the products; the reference sums dCB over heads too, mamba2_ssd_prepare_dcb/design.md:15-18):
//
//   accC = dCB   * B                                         tcgen05   (dCB as bf16 hi/lo tile, read K-major)
//   accB = dCB^T * C                                         tcgen05   (the SAME tile read MN-major)
//
// dC = accC + regC, dB = accB + regB.  Every fp32 tile is loaded by TMA straight into its
// operand tile's memory and split in place (dout goes from there to tensor memory: it is an A operand only).
// There are two (dout, xdt) regions, used by head parity; a region is free as soon as D0, T and V of its head
// exist, so loads run two heads ahead.  D0 is handed to the tensor core as soon as dout and xdt are ready, while
// S and dU (one buffer: requested when the previous head's T and V are done) still arrive.  The last head's
// region takes the dCB tile of the group; the finished gradients are staged in the same memory and written
// by TMA while the next tile's first head is already being worked on.
#include "ssd_decay.cuh"
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

struct BwdDbcSmem {
    static constexpr int N = 64;
    static constexpr uint32_t kPTile = kTile * 128 * 2;  // [128 x 64] hi | lo (= the fp32 tile)
    static constexpr uint32_t kTHalf = kTile * 128 * 2;  // [128 x 128] one of hi / lo
    static constexpr uint32_t kSTile = 64 * 128 * 2;     // [64 x 64] hi | lo
    // two regions by head parity: dout tile + xdt tile, later that head's dCB tile (hi half, lo half);
    // at the very end region 0 stages the fp32 dC / dB slabs
    static constexpr uint32_t kRegion = 2 * kPTile;
    static constexpr uint32_t kG = 0;
    static constexpr uint32_t kX = kG + kPTile;
    static constexpr uint32_t kDHi = 0;
    static constexpr uint32_t kDLo = kDHi + kTHalf;
    static constexpr uint32_t kS = 2 * kRegion;
    static constexpr uint32_t kU = kS + kSTile;
    static constexpr uint32_t kB = kU + kSTile;
    static constexpr uint32_t kC = kB + kPTile;
    // the rows of two heads (by head parity): cs[128], q[128], the head's (batch, head, tile) index
    static constexpr uint32_t kRowSetFloats = 2 * kTile + 4;
    static constexpr uint32_t kRows = kC + kPTile;
    static constexpr uint32_t kRed = kRows + 2 * kRowSetFloats * 4;  // float[2][8] partial sums
    static constexpr uint32_t kBars = kRed + 64;
    static constexpr uint32_t kTotal = kBars + 128;
};
// No slack for re-aligning the base: the dynamic shared memory is declared 1024-byte aligned (and checked).
static_assert(BwdDbcSmem::kTotal <= 232448, "dB/dC kernel exceeds the shared memory of one SM");

__global__ void __launch_bounds__(kLaunchThreadsGroups, 1)
bwd_dbc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_dout,
               const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_du,
               const __grid_constant__ CUtensorMap map_db, const __grid_constant__ CUtensorMap map_dc,
               const float* __restrict__ q, const float* __restrict__ cs, float* __restrict__ g_last, SsdShape s,
               int* status) {
    using L = BwdDbcSmem;
    constexpr int N = L::N;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    float* rows = reinterpret_cast<float*>(smem + L::kRows);    // [2] row sets
    float* red = reinterpret_cast<float*>(smem + L::kRed);      // [2][8] partial sums of sum(dU .* S)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_gx = bars;        // [2] dout and x tiles have landed (by head parity)
    uint64_t* full_su = bars + 2;    // S and dU tiles have landed
    uint64_t* full_bc = bars + 3;    // B and C tiles have landed
    uint64_t* bar_d0 = bars + 4;     // D0 done
    uint64_t* bar_tv = bars + 5;     // T and V done
    uint64_t* bar_g2 = bars + 6;     // dCB products done
    uint64_t* bar_rdy1 = bars + 7;   // S and dU tiles split (and the T, V accumulators read)
    uint64_t* bar_rdy2 = bars + 8;   // dCB tile complete
    uint64_t* rows_ready = bars + 9;  // [2] the rows of a head are published (by head parity)
    uint64_t* rows_free = bars + 11;  // [2] every compute warp has finished with it
    uint64_t* bar_rdy0 = bars + 13;   // dout and xdt tiles split (and the D0 accumulator read)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    // Work list of this CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the (batch, group, token
    // tile) grid, token tile fastest; the heads of all its tiles form one flat sequence of iterations,
    // so the loads, splits and products of a tile's first head overlap the previous tile's last head.
    const int num_tiles = s.batch * s.ngroups * nchunks;
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                         static_cast<int>(gridDim.x);
    const int total = my_tiles * heads_per_group;
    const TileWalk walk(s, static_cast<int>(gridDim.x));
    using Where = HeadPos;
    auto first_tile = [&]() { return walk.first(static_cast<int>(blockIdx.x)); };
    auto advance = [&](TilePos& t) { walk.advance(t); };
    auto locate = [&](const TilePos& t, int hi, int ahead) { return walk.locate(t, hi, ahead); };

    if ((smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled tiles need the declared alignment
        if (tid == 0) atomicCAS(status, 0, kStatusSmemAlign);
        return;
    }

    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below, so that no warp is ever
    // left waiting on a barrier that departed warps will not reach.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
        mbar_init(bar_rdy0, kThreads / 32);
        mbar_init(bar_rdy1, kThreads / 32);
        mbar_init(bar_rdy2, kThreads / 32);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&rows_ready[i], 32);
            mbar_init(&rows_free[i], kThreads / 32);
        }
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (tmem_slot[1] != 0) {
        if (warp == 0) tmem_dealloc(tmem, 512);
        return;
    }
    // D0 [128], T [64], V [64], accC main | correction [128], accB [64]; dout as an A operand (row in lane, two
    // bf16 contraction elements per column): hi [32] | lo [32]
    const uint32_t tm_d0 = tmem, tm_t = tmem + 128, tm_v = tmem + 192, tm_accc = tmem + 256, tm_accb = tmem + 384;
    const uint32_t tm_ghi = tmem + 448, tm_glo = tmem + 480;
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;  // hi -> lo distance of a [128 x 64] tile
    constexpr uint32_t kSHalf = 64 * 128;

    // ---- warp 16: issues every tensor-core instruction of the CTA.  Its warp group hands most of its
    // registers to the four computing groups.
    if (warp >= kThreads / 32) {
        reg_release<kIssuerRegs>();
        if (warp == kThreads / 32 && lane == 0) {
            const uint32_t ss = smem_u32(smem + L::kS), su = smem_u32(smem + L::kU), sb = smem_u32(smem + L::kB),
                           sc = smem_u32(smem + L::kC);
            const Operand st{ss, ss + kSHalf, 64, true};
            const Operand du{su, su + kSHalf, 64, true};
            const Operand bm{sb, sb + kHalf, kTile, true};
            const Operand cm{sc, sc + kHalf, kTile, true};
            uint32_t p0 = 0, p1 = 0, p2 = 0;
            int hi = 0;
            for (int it = 0; it < total; ++it) {
                const uint32_t r0 = smem_u32(smem) + (it & 1) * L::kRegion;
                const Operand xd{r0 + L::kX, r0 + L::kX + kHalf, kTile, false};
                const Operand dcb{r0 + L::kDHi, r0 + L::kDLo, kTile, false};
                const Operand dcbt{r0 + L::kDHi, r0 + L::kDLo, kTile, true};
                mbar_wait(bar_rdy0, p0, status, kStatusMmaTimeout | wait_site(5, 15));
                p0 ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<64 / 16>(tm_d0, tm_ghi, tm_glo, xd, 0, make_idesc_bf16(128, 128, false, false), false);
                umma_commit(bar_d0);  // D0 runs while S and dU arrive and are split
                mbar_wait(bar_rdy1, p1, status, kStatusMmaTimeout | wait_site(5, 1));
                p1 ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<64 / 16>(tm_t, tm_ghi, tm_glo, st, 0, make_idesc_bf16(128, N, false, true), false);
                issue_gemm_split<64 / 16>(tm_v, xd, 0, du, 0, make_idesc_bf16(128, N, false, true), false);
                umma_commit(bar_tv);  // the last readers of this head's dout / xdt, S and dU tiles
                if (hi == heads_per_group - 1) {  // the group's dCB tile is complete: one product pair per tile
                    mbar_wait(bar_rdy2, p2, status, kStatusMmaTimeout | wait_site(5, 2));
                    p2 ^= 1;
                    tc_fence_after_sync();
                    issue_gemm_split_wide<kTile / 16>(tm_accc, dcb, bm, make_idesc_bf16(128, 2 * N, false, true),
                                                      make_idesc_bf16(128, N, false, true), false);
                    issue_gemm_split<kTile / 16>(tm_accb, dcbt, 0, cm, 0, make_idesc_bf16(128, N, true, true), false);
                    umma_commit(bar_g2);
                }
                if (++hi == heads_per_group) hi = 0;
            }
        }
        // ---- warp 17: the producer.  Lane 0 issues every TMA load as soon as the memory it lands in is free (it
        // waits on the same barriers of finished products as the compute warps) and every store of a finished
        // tile.  The coordinates of the next loads are ready BEFORE the wait, so a load leaves within a few
        // cycles of the product that frees its memory.
        if (warp == kThreads / 32 + 1) {
            auto load_gx = [&](int it, const Where& w) {
                uint8_t* r = smem + (it & 1) * L::kRegion;
                uint64_t* bar = &full_gx[it & 1];
                mbar_arrive_expect_tx(bar, 2 * L::kPTile);
                tma_tile_3d(r + L::kG, kTile, &map_dout, bar, 0, w.h, w.tok0, false);
                tma_tile_3d(r + L::kX, kTile, &map_x, bar, 0, w.h, w.tok0, false);
            };
            auto load_su = [&](const Where& w) {
                mbar_arrive_expect_tx(full_su, 2 * L::kSTile);
                tma_tile_2d(smem + L::kS, 64, &map_s, full_su, 0, w.tile_index * 64, false);
                tma_tile_2d(smem + L::kU, 64, &map_du, full_su, 0, w.tile_index * 64, false);
            };
            auto load_bc = [&](int g, int tok0) {
                mbar_arrive_expect_tx(full_bc, 2 * L::kPTile);
                tma_tile_3d(smem + L::kB, kTile, &map_b, full_bc, 0, g, tok0, false);
                tma_tile_3d(smem + L::kC, kTile, &map_c, full_bc, 0, g, tok0, false);
            };
            // Finished tile of group g at token tok0, staged by the compute warps in the region of the tile's
            // last head, iteration `j` (named barrier 4 says so).
            auto store_tile = [&](int j, int g, int tok0) {
                asm volatile("bar.sync 4, 544;" ::: "memory");
                if (lane == 0 && *reinterpret_cast<volatile int*>(status) == 0) {
                    const uint8_t* stage = smem + (j & 1) * L::kRegion;
                    tma_store_3d(&map_dc, stage, 0, g, tok0);
                    tma_store_3d(&map_dc, stage + kSlabBytes, 32, g, tok0);
                    tma_store_3d(&map_db, stage + 2 * kSlabBytes, 0, g, tok0);
                    tma_store_3d(&map_db, stage + 3 * kSlabBytes, 32, g, tok0);
                    tma_store_commit();
                }
            };
            TilePos cur = first_tile();
            int hi = 0, prev_g = 0, prev_tok0 = 0;
            if (lane == 0) {
                const Where w0 = locate(cur, 0, 0);
                load_bc(w0.g, w0.tok0);
                load_gx(0, w0);
                load_su(w0);
                if (total > 1) load_gx(1, locate(cur, 0, 1));
            }
            uint32_t p_tv = 0, p_g2 = 0;
            for (int it = 0; it < total; ++it) {
                const bool last_of_tile = hi == heads_per_group - 1;
                if (it > 0 && hi == 0) {
                    // the previous tile's group products are done with B and C and with the dCB tile, in whose
                    // place the compute warps now stage the gradients
                    const Where w0 = locate(cur, 0, 0), w1 = locate(cur, 0, 1);
                    mbar_wait(bar_g2, p_g2, status, kStatusMmaTimeout | wait_site(5, 11));
                    p_g2 ^= 1;
                    tc_fence_after_sync();
                    if (lane == 0) load_bc(w0.g, w0.tok0);
                    store_tile(it - 1, prev_g, prev_tok0);
                    if (lane == 0 && it + 1 < total) {  // the next head's dout / x tiles, once the store has read
                        tma_store_wait_read();
                        load_gx(it + 1, w1);
                    }
                }
                const Where w1 = locate(cur, hi, 1), w2 = locate(cur, hi, 2);
                // T and V are the last readers of this head's dout / xdt, S and dU tiles
                mbar_wait(bar_tv, p_tv, status, kStatusMmaTimeout | wait_site(5, 12));
                p_tv ^= 1;
                tc_fence_after_sync();
                if (lane == 0) {
                    if (it + 1 < total) load_su(w1);
                    // this head's region is free (unless it takes the group's dCB tile): the head after next
                    if (!last_of_tile && it + 2 < total) load_gx(it + 2, w2);
                }
                if (++hi == heads_per_group) {
                    hi = 0;
                    prev_g = cur.g;
                    prev_tok0 = cur.b * s.seqlen + cur.k * kTile;
                    advance(cur);
                }
            }
            if (total > 0) {
                store_tile(total - 1, prev_g, prev_tok0);
                if (lane == 0) tma_store_wait_all();
            }
        }
        // ---- warp 18 publishes the rows (cs, q, tile index) of the head after next as soon as every compute
        // warp has finished with the head that used the set's memory; the values are fetched before the wait.
        if (warp == kThreads / 32 + 2) {
            TilePos cur = first_tile();
            int hi = 0;
            float c[4], qv[4];
            auto fetch = [&](const Where& w) {
                const size_t o = static_cast<size_t>(w.tile_index) * kTile;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    c[j] = cs[o + 32 * j + lane];
                    qv[j] = q[o + 32 * j + lane];
                }
            };
            auto publish = [&](int it, const Where& w) {
                float* set = rows + (it & 1) * L::kRowSetFloats;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    set[32 * j + lane] = c[j];
                    set[kTile + 32 * j + lane] = qv[j];
                }
                if (lane == 0) set[2 * kTile] = __int_as_float(w.tile_index);
                mbar_arrive(&rows_ready[it & 1]);
            };
            for (int it = 0; it < 2 && it < total; ++it) {
                const Where w = locate(cur, 0, it);
                fetch(w);
                publish(it, w);
            }
            for (int it = 0; it + 2 < total; ++it) {
                const Where w = locate(cur, hi, 2);
                fetch(w);
                mbar_wait(&rows_free[it & 1], (it >> 1) & 1u, status, kStatusMmaTimeout | wait_site(5, 13));
                publish(it + 2, w);
                if (++hi == heads_per_group) {
                    hi = 0;
                    advance(cur);
                }
            }
        }
        return;
    }

    reg_acquire<kComputeRegs>();

    const int t_row = (warp & 3) * 32 + lane;  // this thread's row of the accumulators (TMEM lane)
    const int qr = warp & 3;                   // its block of 32 rows
    const int cg = warp >> 2;                  // its block of 32 columns of D0, 16 columns of T and V

    uint32_t p_gx = 0 /* one parity bit per region */, p_su = 0, p_bc = 0, d0_parity = 0, tv_parity = 0, g2_parity = 0;
    // S (warps 0-7) and dU (warps 8-15) are split side by side.  On the way the warps of S also form
    //   g_last[k] = exp(cs_last,k) * sum_{p,n} dU_k[p,n] S_k[p,n],
    // the gradient of this tile's total decay through the state recurrence
    // (mamba2_ssd_state_passing_bwd/design.md:49-58), because both tiles pass through this kernel anyway:
    // the thread that holds 16 values of S reads the same 16 of dU, four at a time, before dU is split --
    // the warps of dU start their in-place split once the warps of S have read it (named barrier 3; the
    // warps of S cannot reach the next head's arrival before the warps of dU have left this head's wait,
    // because the next S tile is loaded only after products that need every warp's hand-off).
    auto split_s = [&](int it) {  // warps 0-7: S split, products with dU
        if (warp < 8) {
            ok = mbar_wait(full_su, p_su, status, kStatusTmaTimeout | wait_site(5, 3)) && ok;
            const uint8_t* tu = smem + L::kU;
            float dot = 0.f;
            split_tile_inplace(smem + L::kS, 64, nullptr, warp, lane, [&](uint32_t r, uint32_t qd, const float* v) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 u = *reinterpret_cast<const float4*>(tu + (qd >> 1) * kSHalf + swz(r, (qd & 1) * 4 + i));
                    dot = fmaf(v[4 * i], u.x, fmaf(v[4 * i + 1], u.y, fmaf(v[4 * i + 2], u.z, fmaf(v[4 * i + 3], u.w, dot))));
                }
                asm volatile("bar.arrive 3, 512;" ::: "memory");  // dU has been read by this warp
            });
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
            if (lane == 0) red[(it & 1) * 8 + warp] = dot;  // partial sums of sum(dU .* S), by head parity
        }
    };
    auto split_u = [&]() {  // warps 8-15: dU split, once the warps of S have read it
        if (warp >= 8) {
            ok = mbar_wait(full_su, p_su, status, kStatusTmaTimeout | wait_site(5, 3)) && ok;
            asm volatile("bar.sync 3, 512;" ::: "memory");
            split_tile_inplace(smem + L::kU, 64, nullptr, warp - 8, lane);
        }
        p_su ^= 1;
    };
    auto split_bc = [&]() {
        ok = mbar_wait(full_bc, p_bc, status, kStatusTmaTimeout | wait_site(5, 4)) && ok;
        p_bc ^= 1;
        split_tile_inplace(smem + L::kB, kTile, nullptr, warp, lane);
        split_tile_inplace(smem + L::kC, kTile, nullptr, warp, lane);
    };

    // per-thread slice of the state terms: row t, 16 columns
    float reg_c[16], reg_b[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) reg_c[i] = reg_b[i] = 0.f;

    // Finished tile: dC (slabs 0, 1) and dB (slabs 2, 3) are staged in `stage` (the region of the tile's last
    // head, whose dCB products are done); the producer warp writes them out by TMA once every compute warp has
    // passed the barrier.  The CTA barrier also separates the reads of the accumulator columns here from the
    // stores of the new tile's dCB sum into the same columns by other warps.
    auto write_tile = [&](uint8_t* stage) {
        // dC first, then dB, 8 columns (16 transient registers) at a time
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float a[8], x[8];
            tmem_ld8(tmem_addr(tm_accc, warp, cg * 16 + 8 * half), a);
            tmem_ld8(tmem_addr(tm_accc, warp, N + cg * 16 + 8 * half), x);
            tmem_ld_wait();
            uint8_t* slab_c = stage + (cg >> 1) * kSlabBytes;
#pragma unroll
            for (int i = 0; i < 8; i += 4)
                *reinterpret_cast<float4*>(slab_c + swz(t_row, (cg & 1) * 4 + 2 * half + (i >> 2))) = make_float4(
                    a[i] + x[i] + reg_c[8 * half + i], a[i + 1] + x[i + 1] + reg_c[8 * half + i + 1],
                    a[i + 2] + x[i + 2] + reg_c[8 * half + i + 2], a[i + 3] + x[i + 3] + reg_c[8 * half + i + 3]);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float a[8];
            tmem_ld8(tmem_addr(tm_accb, warp, cg * 16 + 8 * half), a);
            tmem_ld_wait();
            uint8_t* slab_b = stage + (2 + (cg >> 1)) * kSlabBytes;
#pragma unroll
            for (int i = 0; i < 8; i += 4)
                *reinterpret_cast<float4*>(slab_b + swz(t_row, (cg & 1) * 4 + 2 * half + (i >> 2))) = make_float4(
                    a[i] + reg_b[8 * half + i], a[i + 1] + reg_b[8 * half + i + 1], a[i + 2] + reg_b[8 * half + i + 2],
                    a[i + 3] + reg_b[8 * half + i + 3]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) reg_c[i] = reg_b[i] = 0.f;
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        asm volatile("bar.arrive 4, 544;" ::: "memory");
    };

    // dCB of the group is summed over its heads in fp32 in the columns of accC, which are idle between the
    // write-out of the previous tile (before the first head's pass) and this tile's group products: every
    // thread keeps its 32 entries of row t there (read - add - write back; only the blocks left of and on the
    // diagonal), since 32 more accumulator registers per thread do not fit.
    int hi = 0;
    for (int it = 0; it < total; ++it) {
        uint8_t* region = smem + (it & 1) * L::kRegion;
        const bool first_of_tile = hi == 0;
        const bool last_of_tile = hi == heads_per_group - 1;
        const bool new_tile = it > 0 && first_of_tile;
        // ---- this head's rows (the producer warp published them a head ago) and the scalars this thread
        // derives from them.  The causal decay exp(cs_i - cs_j), j <= i, is factored per block of 32 columns
        // with the block's first cs as reference:  exp(cs_i - c0) * exp(c0 - cs_j).  The second factor (>= 1,
        // bounded by the decay across 32 tokens) is folded into the rows of the xdt tile when it is split, so
        // that D0 leaves the tensor core carrying it and the decay pass multiplies a whole block of a row by
        // ONE scalar, with no table and no shared-memory read; V, which is formed from the same xdt tile,
        // gives the factor back in its own row scale.  A block whose decay exceeds the fast limit (or whose
        // cs increases) is left unscaled and takes one exp per element, exponent selected before the exp.
        ok = mbar_wait(&rows_ready[it & 1], (it >> 1) & 1u, status, kStatusMmaTimeout | wait_site(5, 14)) && ok;
        const float* cs_s = rows + (it & 1) * L::kRowSetFloats;
        float fx;  // scale of the xdt row this thread splits: q, and the folded factor of its block of 32 rows
        {
            const float b0 = cs_s[32 * cg];  // rows 8 * warp .. 8 * warp + 7 lie in block warp / 4 = cg
            const float span = b0 - cs_s[32 * cg + 31];
            const int split_row = warp * 8 + (lane & 7);
            fx = cs_s[kTile + split_row];
            if (span >= 0.f && span < kDecayFastLimit) fx *= __expf(b0 - cs_s[split_row]);
        }

        // ---- the dout and xdt tiles landed, in this head's region, two heads ago: D0 can start at once.  S and
        // dU were requested only when the previous head's T and V were done; they arrive, and are split, while
        // D0 runs.
        ok = mbar_wait(&full_gx[it & 1], (p_gx >> (it & 1)) & 1u, status, kStatusTmaTimeout | wait_site(5, 5)) && ok;
        p_gx ^= 1u << (it & 1);
        {  // dout is an A operand only (of D0 and T): from the fp32 tile as it landed to tensor memory, row t in
           // lane t, this warp's 16 of the 64 contraction elements -- no shared-memory operand tile, and the
           // products read it without touching shared memory
            const uint8_t* src = region + L::kG + (cg >> 1) * kHalf;
            float v[16];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float4 f = *reinterpret_cast<const float4*>(src + swz(t_row, (cg & 1) * 4 + c));
                v[4 * c] = f.x;
                v[4 * c + 1] = f.y;
                v[4 * c + 2] = f.z;
                v[4 * c + 3] = f.w;
            }
            uint32_t ghi[8], glo[8];
            split16_packed(v, ghi, glo);
            tmem_st8(tmem_addr(tm_ghi, warp, 8 * cg), ghi);
            tmem_st8(tmem_addr(tm_glo, warp, 8 * cg), glo);
            tmem_st_wait();
        }
        split_tile_inplace_scaled(region + L::kX, kTile, fx, warp, lane);
        signal_issuer(bar_rdy0, lane);
        split_s(it);
        split_u();
        signal_issuer(bar_rdy1, lane);
        // First head of a new tile: when the previous tile's group products are done its gradients are staged
        // in the other region (the previous head's, which held the dCB tile) for the producer warp to write out.
        if (new_tile) {
            ok = mbar_wait(bar_g2, g2_parity, status, kStatusMmaTimeout | wait_site(5, 6)) && ok;
            g2_parity ^= 1;
            tc_fence_after_sync();
            write_tile(smem + ((it + 1) & 1) * L::kRegion);
        }
        // the scalars of the decay pass (column block cg) and of the state terms, while the products run
        const float c0 = cs_s[32 * cg];
        const float span_c = c0 - cs_s[32 * cg + 31];
        const bool fast_c = span_c >= 0.f && span_c < kDecayFastLimit;
        const float csi = cs_s[t_row];
        const float ei = __expf(fminf(csi - c0, 80.f));
        const float clast = cs_s[kTile - 1];
        const float q0 = cs_s[32 * qr];
        const float span_q = q0 - cs_s[32 * qr + 31];
        const float e_out = expf(csi);
        const float e_end = expf(span_q >= 0.f && span_q < kDecayFastLimit ? clast - q0 : clast - csi);
        ok = mbar_wait(bar_d0, d0_parity, status, kStatusMmaTimeout | wait_site(5, 7)) && ok;
        d0_parity ^= 1;
        tc_fence_after_sync();
        // D0 exists, so every warp has handed its split tiles over, the warps of S their partial sums included:
        // one thread of a warp with no share of the decay pass adds them in a fixed order.
        if (g_last != nullptr && tid == 384 && ok) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += red[(it & 1) * 8 + w];
            g_last[__float_as_int(cs_s[2 * kTile])] = expf(clast) * sum;
        }

        // ---- this head's dCB block into the group sum, and the state terms
        {
            // T and V are the last readers of this head's dout / xdt, S and dU tiles.  In the last head of a
            // tile the finished dCB tile overwrites that region, so there the wait comes before the pass.
            if (last_of_tile) {
                ok = mbar_wait(bar_tv, tv_parity, status, kStatusMmaTimeout | wait_site(5, 8)) && ok;
                tv_parity ^= 1;
                tc_fence_after_sync();
            }
            if (cg <= qr) {  // in two halves of 16 columns (register budget)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t col = 32 * cg + 16 * half;
                    float v[16], acc[16];
                    tmem_ld16(tmem_addr(tm_d0, warp, col), v);
                    if (!first_of_tile) tmem_ld16(tmem_addr(tm_accc, warp, col), acc);
                    tmem_ld_wait();
                    if (fast_c) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            v[jj] = (cg < qr || static_cast<int>(col) + jj <= t_row) ? v[jj] * ei : 0.f;
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const int j = static_cast<int>(col) + jj;
                            const float e = __expf(j <= t_row ? csi - cs_s[j] : 0.f);
                            v[jj] = j <= t_row ? v[jj] * e : 0.f;
                        }
                    }
                    if (!first_of_tile) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) v[jj] += acc[jj];
                    }
                    if (!last_of_tile) {
                        tmem_st16(tmem_addr(tm_accc, warp, col), reinterpret_cast<const uint32_t*>(v));
                    } else {  // the group's dCB block is complete: bf16 hi/lo into this head's dead region
                        store_split8(region + L::kDHi, region + L::kDLo, kTile, t_row, col, v);
                        store_split8(region + L::kDHi, region + L::kDLo, kTile, t_row, col + 8, v + 8);
                    }
                }
                if (!last_of_tile) tmem_st_wait();
            } else if (last_of_tile) {  // right of the diagonal: zeros
                float z[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) z[jj] = 0.f;
#pragma unroll
                for (int jj = 0; jj < 32; jj += 8)
                    store_split8(region + L::kDHi, region + L::kDLo, kTile, t_row, 32 * cg + jj, z);
            }
            // this warp has finished with the head's rows
            __syncwarp();
            if (lane == 0) mbar_arrive(&rows_free[it & 1]);
            if (!last_of_tile) {
                ok = mbar_wait(bar_tv, tv_parity, status, kStatusMmaTimeout | wait_site(5, 9)) && ok;
                tv_parity ^= 1;
                tc_fence_after_sync();
            }
            float tv[16], vv[16];
            tmem_ld16(tmem_addr(tm_t, warp, cg * 16), tv);
            tmem_ld16(tmem_addr(tm_v, warp, cg * 16), vv);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                reg_c[i] += e_out * tv[i];
                reg_b[i] += e_end * vv[i];
            }
        }
        if (last_of_tile) {
            // ---- this tile's B and C; then the group products can run
            split_bc();
            signal_issuer(bar_rdy2, lane);
        }

        if (++hi == heads_per_group) hi = 0;
    }
    // the last dCB products, the last tile
    if (total > 0) {
        ok = mbar_wait(bar_g2, g2_parity, status, kStatusMmaTimeout | wait_site(5, 10)) && ok;
        tc_fence_after_sync();
        write_tile(smem + ((total + 1) & 1) * L::kRegion);
    }
    tc_fence_before_sync();
    cta_sync();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_dbc_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                                 const float* dout, const float* states_start, const float* dstates, const float* q,
                                 const float* cs, float* dB, float* dC, float* g_last, int* status,
                                 ssd_stream_t stream) {
    using namespace ssd;
    const int rc0 = ssd_check_shape(shape);
    if (rc0 != SSD_OK) return rc0;
    if (!x || !bm || !cm || !dout || !states_start || !dstates || !q || !cs || !dB || !dC || !status)
        return SSD_ERR_NULL;
    const SsdShape& s = *shape;
    if (s.dstate != 64) return SSD_ERR_UNSUPPORTED;
    CUtensorMap map_x, map_b, map_c, map_dout, map_s, map_du, map_db, map_dc;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_b, bm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_c, cm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dout, dout, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_db, dB, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dc, dC, tokens, s.ngroups, s.dstate, kTile);
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_s, states_start, state_rows, s.dstate, 64);
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_du, dstates, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    const size_t smem = BwdDbcSmem::kTotal;
    static std::atomic<uint64_t> smem_set{0};
    rc = set_max_smem_once(reinterpret_cast<const void*>(bwd_dbc_kernel), smem, smem_set);
    if (rc != SSD_OK) return rc;
    const int tiles = (s.seqlen / kTile) * s.ngroups * s.batch;
    const int sms = sm_count();
    if (sms <= 0) return SSD_ERR_LAUNCH;
    const dim3 grid(tiles < sms ? tiles : sms);  // persistent: one CTA per SM walks its share of the tiles
    bwd_dbc_kernel<<<grid, kLaunchThreadsGroups, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        map_x, map_b, map_c, map_dout, map_s, map_du, map_db, map_dc, q, cs, g_last, s, status);
    return launch_status();
}
