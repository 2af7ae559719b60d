// Backward kernel for dB and dC.  One persistent CTA per SM walks its share of the (batch, group, tile of
// 128 tokens) work items; 16 compute warps plus one warp that only issues tensor-core instructions; the gradient of the group is accumulated over its
// heads inside the CTA, so each output element is written once by one CTA (no atomics, fixed order).
// Per head h (xdt = q .* x, S = state at the start of the tile, dU = gradient of the state after the tile):
//
//   D0[i,j]  = sum_p dout[i,p] * xdt[j,p]                    tcgen05, N = 128
//   T[i,n]   = sum_p dout[i,p] * S[p,n]                      tcgen05   (state-to-output term of dC)
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
// operand tile's memory and split in place.  There are two (dout, xdt) regions, used by head parity; a
// region is free as soon as D0, T and V of its head exist, so loads run two heads ahead.  The last head's
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
    static constexpr uint32_t kRows = kC + kPTile;  // cs[128], q[128], decay table
    static constexpr uint32_t kRed = kRows + (2 * kTile + kDecayTableFloatsCompact) * 4;  // float[8] partial sums
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
    float* cs_s = reinterpret_cast<float*>(smem + L::kRows);  // [128]
    float* q_s = cs_s + kTile;                                // [128]
    float* ej_s = cs_s + 2 * kTile;                           // decay table, see ssd_decay.cuh
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_gx = bars;        // [2] dout and x tiles have landed (by head parity)
    uint64_t* full_su = bars + 2;    // S and dU tiles have landed
    uint64_t* full_bc = bars + 3;    // B and C tiles have landed
    uint64_t* bar_d0 = bars + 4;     // D0 done
    uint64_t* bar_tv = bars + 5;     // T and V done
    uint64_t* bar_g2 = bars + 6;     // dCB products done
    uint64_t* bar_rdy1 = bars + 7;   // dout, xdt, S, dU tiles split
    uint64_t* bar_rdy2 = bars + 8;   // dCB tile complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);

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
    struct Where {
        int g, h, tok0, srow;
        size_t row0;
    };
    auto where = [&](int it) {
        const int tile = blockIdx.x + (it / heads_per_group) * gridDim.x;
        const int k = tile % nchunks, g = (tile / nchunks) % s.ngroups, b = tile / (nchunks * s.ngroups);
        Where w;
        w.g = g;
        w.h = g * heads_per_group + it % heads_per_group;
        w.tok0 = b * s.seqlen + k * kTile;
        w.srow = ((b * s.nheads + w.h) * nchunks + k) * 64;
        w.row0 = (static_cast<size_t>(b) * s.nheads + w.h) * s.seqlen + k * kTile;
        return w;
    };

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
        mbar_init(bar_rdy1, kThreads / 32);
        mbar_init(bar_rdy2, kThreads / 32);
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
    // D0 [128], T [64], V [64], accC main | correction [128], accB main | correction [128]
    const uint32_t tm_d0 = tmem, tm_t = tmem + 128, tm_v = tmem + 192, tm_accc = tmem + 256, tm_accb = tmem + 384;
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
            uint32_t p1 = 0, p2 = 0;
            int hi = 0;
            for (int it = 0; it < total; ++it) {
                const uint32_t r0 = smem_u32(smem) + (it & 1) * L::kRegion;
                const Operand gy{r0 + L::kG, r0 + L::kG + kHalf, kTile, false};
                const Operand xd{r0 + L::kX, r0 + L::kX + kHalf, kTile, false};
                const Operand dcb{r0 + L::kDHi, r0 + L::kDLo, kTile, false};
                const Operand dcbt{r0 + L::kDHi, r0 + L::kDLo, kTile, true};
                mbar_wait(bar_rdy1, p1, status, kStatusMmaTimeout | wait_site(5, 1));
                p1 ^= 1;
                tc_fence_after_sync();
                issue_gemm_split<64 / 16>(tm_d0, gy, 0, xd, 0, make_idesc_bf16(128, 128, false, false), false);
                umma_commit(bar_d0);  // the decay pass can start on D0 ...
                issue_gemm_split<64 / 16>(tm_t, gy, 0, st, 0, make_idesc_bf16(128, N, false, true), false);
                issue_gemm_split<64 / 16>(tm_v, xd, 0, du, 0, make_idesc_bf16(128, N, false, true), false);
                umma_commit(bar_tv);  // ... but may overwrite the dout / xdt tiles only after T and V
                if (hi == heads_per_group - 1) {  // the group's dCB tile is complete: one product pair per tile
                    mbar_wait(bar_rdy2, p2, status, kStatusMmaTimeout | wait_site(5, 2));
                    p2 ^= 1;
                    tc_fence_after_sync();
                    issue_gemm_split_wide<kTile / 16>(tm_accc, dcb, bm, make_idesc_bf16(128, 2 * N, false, true),
                                                      make_idesc_bf16(128, N, false, true), false);
                    issue_gemm_split_wide<kTile / 16>(tm_accb, dcbt, cm, make_idesc_bf16(128, 2 * N, true, true),
                                                      make_idesc_bf16(128, N, true, true), false);
                    umma_commit(bar_g2);
                }
                if (++hi == heads_per_group) hi = 0;
            }
        }
        return;
    }

    reg_acquire<kComputeRegs>();

    // ---- loads.  One thread issues them; each lands in its operand tile's own memory.
    auto load_gx = [&](int it) {
        const Where w = where(it);
        uint8_t* r = smem + (it & 1) * L::kRegion;
        uint64_t* bar = &full_gx[it & 1];
        mbar_arrive_expect_tx(bar, 2 * L::kPTile);
        tma_tile_3d(r + L::kG, kTile, &map_dout, bar, 0, w.h, w.tok0, false);
        tma_tile_3d(r + L::kX, kTile, &map_x, bar, 0, w.h, w.tok0, false);
    };
    auto load_su = [&](int it) {
        const Where w = where(it);
        mbar_arrive_expect_tx(full_su, 2 * L::kSTile);
        tma_tile_2d(smem + L::kS, 64, &map_s, full_su, 0, w.srow, false);
        tma_tile_2d(smem + L::kU, 64, &map_du, full_su, 0, w.srow, false);
    };
    auto load_bc = [&](int it) {
        const Where w = where(it);
        mbar_arrive_expect_tx(full_bc, 2 * L::kPTile);
        tma_tile_3d(smem + L::kB, kTile, &map_b, full_bc, 0, w.g, w.tok0, false);
        tma_tile_3d(smem + L::kC, kTile, &map_c, full_bc, 0, w.g, w.tok0, false);
    };
    if (tid == 0) {
        load_bc(0);
        load_gx(0);
        load_su(0);
        if (total > 1) load_gx(1);
    }

    // rows (cs, q) and the decay references cs[0], cs[32], cs[64], cs[96] are fetched one head ahead
    float r_cs = 0.f, r_q = 0.f, r_ref[4] = {0.f, 0.f, 0.f, 0.f};
    auto fetch_rows = [&](int it) {
        const size_t o = where(it).row0;
        r_cs = cs[o + tid];
        r_q = q[o + tid];
#pragma unroll
        for (int i = 0; i < 4; ++i) r_ref[i] = cs[o + 32 * i];
    };
    if (tid < kTile) fetch_rows(0);

    uint32_t p_gx = 0 /* one parity bit per region */, p_su = 0, p_bc = 0, d0_parity = 0, tv_parity = 0, g2_parity = 0;
    // S (warps 0-7) and dU (warps 8-15) are split side by side.  On the way the warps of S also form
    //   g_last[k] = exp(cs_last,k) * sum_{p,n} dU_k[p,n] S_k[p,n],
    // the gradient of this tile's total decay through the state recurrence
    // (mamba2_ssd_state_passing_bwd/design.md:49-58), because both tiles pass through this kernel anyway:
    // the thread that holds 16 values of S reads the same 16 of dU, four at a time, before dU is split --
    // the warps of dU start their in-place split once the warps of S have read it (named barrier 3).
    auto split_s = [&]() {  // warps 0-7: S split, products with dU
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
            if (lane == 0) cs_s[(L::kRed - L::kRows) / 4 + warp] = dot;  // partial sums of sum(dU .* S), warps 0-7
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
    // The 8 partial sums of the head whose rows are still published, added in a fixed order by the thread that
    // owns the tile's last row (it reads before it publishes the next head's row).
    auto write_g_last = [&]() {
        if (g_last != nullptr && tid == kTile - 1 && ok) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += cs_s[(L::kRed - L::kRows) / 4 + w];
            g_last[__float_as_uint(cs_s[(L::kRed - L::kRows) / 4 + 8])] = expf(cs_s[kTile - 1]) * sum;
        }
    };
    auto split_bc = [&]() {
        ok = mbar_wait(full_bc, p_bc, status, kStatusTmaTimeout | wait_site(5, 4)) && ok;
        p_bc ^= 1;
        split_tile_inplace(smem + L::kB, kTile, nullptr, warp, lane);
        split_tile_inplace(smem + L::kC, kTile, nullptr, warp, lane);
    };
    split_s();  // first head
    split_u();

    // per-thread slice of the state terms: row t, 16 columns
    const int t_row = (warp & 3) * 32 + lane;
    const int cg = warp >> 2;
    float reg_c[16], reg_b[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) reg_c[i] = reg_b[i] = 0.f;

    // Finished tile: dC (slabs 0, 1) and dB (slabs 2, 3) are staged in `stage` (a region whose dCB
    // products are done) and written by TMA.  The caller waits for the store to have read `stage`
    // before anything else lands there.
    auto write_tile = [&](uint8_t* stage, const Where& w) {
        {  // dC first, then dB: 32 transient registers at a time
            float ac[16], ax[16];
            tmem_ld16(tmem_addr(tm_accc, warp, cg * 16), ac);
            tmem_ld16(tmem_addr(tm_accc, warp, N + cg * 16), ax);
            tmem_ld_wait();
            uint8_t* slab_c = stage + (cg >> 1) * kSlabBytes;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(slab_c + swz(t_row, (cg & 1) * 4 + (i >> 2))) =
                    make_float4(ac[i] + ax[i] + reg_c[i], ac[i + 1] + ax[i + 1] + reg_c[i + 1],
                                ac[i + 2] + ax[i + 2] + reg_c[i + 2], ac[i + 3] + ax[i + 3] + reg_c[i + 3]);
        }
        {
            float ab[16], ay[16];
            tmem_ld16(tmem_addr(tm_accb, warp, cg * 16), ab);
            tmem_ld16(tmem_addr(tm_accb, warp, N + cg * 16), ay);
            tmem_ld_wait();
            uint8_t* slab_b = stage + (2 + (cg >> 1)) * kSlabBytes;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(slab_b + swz(t_row, (cg & 1) * 4 + (i >> 2))) =
                    make_float4(ab[i] + ay[i] + reg_b[i], ab[i + 1] + ay[i + 1] + reg_b[i + 1],
                                ab[i + 2] + ay[i + 2] + reg_b[i + 2], ab[i + 3] + ay[i + 3] + reg_b[i + 3]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) reg_c[i] = reg_b[i] = 0.f;
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid == 0 && ok) {
            tma_store_3d(&map_dc, stage, 0, w.g, w.tok0);
            tma_store_3d(&map_dc, stage + kSlabBytes, 32, w.g, w.tok0);
            tma_store_3d(&map_db, stage + 2 * kSlabBytes, 0, w.g, w.tok0);
            tma_store_3d(&map_db, stage + 3 * kSlabBytes, 32, w.g, w.tok0);
            tma_store_commit();
        }
    };

    // dCB of the group is summed over its heads in fp32 in the columns of accC, which are idle between the
    // write-out of the previous tile (before the first head's pass) and this tile's group products: every
    // thread keeps its 32 entries of row t there (read - add - write back; only the blocks left of and on the
    // diagonal), since 32 more accumulator registers per thread do not fit.
    int hi = 0;
    for (int it = 0; it < total; ++it) {
        uint8_t* region = smem + (it & 1) * L::kRegion;
        uint8_t* other = smem + ((it + 1) & 1) * L::kRegion;
        const bool first_of_tile = hi == 0;
        const bool last_of_tile = hi == heads_per_group - 1;
        const bool new_tile = it > 0 && first_of_tile;
        // every warp has left the previous head's decay pass: its rows may be replaced
        if (it > 0) {
            cta_sync();
            write_g_last();
        }
        if (tid < kTile) {
            cs_s[tid] = r_cs;
            // (batch, head, tile) index of the head being published, for the thread that will write its g_last
            if (tid == kTile - 1)
                cs_s[(L::kRed - L::kRows) / 4 + 8] = __uint_as_float(static_cast<uint32_t>(where(it).row0 / kTile));
            q_s[tid] = r_q;
            decay_table_fill<true>(ej_s, tid, r_cs, r_ref);
            if (it + 1 < total) fetch_rows(it + 1);
        }
        cta_sync();

        // ---- dout and xdt tiles of this head: they landed, in this head's region, two heads ago; split in
        // place (S and dU of this head were split one head earlier)
        // S and dU of this head: their load was issued when the previous head's T and V were done and has been
        // flying under the row publication.  The warps of S go first, so that the warps of dU, which split the
        // dout and xdt tiles before they turn to dU, never wait for them.
        if (it > 0) split_s();
        ok = mbar_wait(&full_gx[it & 1], (p_gx >> (it & 1)) & 1u, status, kStatusTmaTimeout | wait_site(5, 5)) && ok;
        p_gx ^= 1u << (it & 1);
        split_tile_inplace(region + L::kG, kTile, nullptr, warp, lane);
        split_tile_inplace(region + L::kX, kTile, q_s, warp, lane);
        if (it > 0) split_u();
        signal_issuer(bar_rdy1, lane);
        // First head of a new tile: the previous tile's group products read the other region, and B and C.
        // When they are done the tile's gradients go out through the other region and this tile's B and C are
        // fetched; the dout / x tiles of the next head land in the other region once the store has read it.
        if (new_tile) {
            ok = mbar_wait(bar_g2, g2_parity, status, kStatusMmaTimeout | wait_site(5, 6)) && ok;
            g2_parity ^= 1;
            tc_fence_after_sync();
            write_tile(other, where(it - 1));
            if (tid == 0) {
                load_bc(it);
                if (it + 1 < total) {  // the next head's dout / x tiles take the other region once the store has read it
                    tma_store_wait_read();
                    load_gx(it + 1);
                }
            }
        }
        ok = mbar_wait(bar_d0, d0_parity, status, kStatusMmaTimeout | wait_site(5, 7)) && ok;
        d0_parity ^= 1;
        tc_fence_after_sync();

        // ---- this head's dCB block into the group sum, and the state terms
        {
            const int qr = warp & 3;
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
                    decay_block_lower<true, 16>(v, t_row, qr, cg, cs_s, ej_s, 16 * half);
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
            if (!last_of_tile) {
                ok = mbar_wait(bar_tv, tv_parity, status, kStatusMmaTimeout | wait_site(5, 9)) && ok;
                tv_parity ^= 1;
                tc_fence_after_sync();
            }
            if (tid == 0) {
                if (it + 1 < total) load_su(it + 1);
                // this head's region is free (unless it takes the group's dCB tile): the head after next
                if (!last_of_tile && it + 2 < total) load_gx(it + 2);
            }
            float tv[16], vv[16];
            tmem_ld16(tmem_addr(tm_t, warp, cg * 16), tv);
            tmem_ld16(tmem_addr(tm_v, warp, cg * 16), vv);
            tmem_ld_wait();
            const float e_out = expf(cs_s[t_row]);
            const float e_end = expf(cs_s[kTile - 1] - cs_s[t_row]);
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
        write_tile(smem + ((total + 1) & 1) * L::kRegion, where(total - 1));
        write_g_last();
    }
    if (tid == 0) tma_store_wait_all();
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
