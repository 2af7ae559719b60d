// Forward output kernel.  One persistent CTA per SM walks its share of the (batch, group, tile of 128 tokens)
// work items, heads of the group in sequence.  16 compute warps; one warp that only issues tensor-core
// instructions; one producer warp that issues every TMA load and store; one warp that publishes each head's
// rows (cs, q).  Every hand-off inside the loop is an mbarrier (no CTA-wide barrier), so a warp that is done
// with a phase runs ahead.  The next tile's C and B land and are prepared while the current tile's last head
// computes.
//
//   CB      = C * B^T                                   once per group        [T,T]   (tcgen05)
//   W_h     = tril(CB .* exp(cs_i - cs_j))              per head, TMEM -> registers -> TMEM (A operand, bf16 hi/lo)
//   out_h   = W_h * (q .* x_h)  +  exp(cs_t) .* (C * S_h^T)                   [T,P]   (two tcgen05 products)
//
// S_h is the state at the start of the tile (from the state-passing kernel).  C, B, x and S are loaded by
// TMA straight into their operand tiles' memory and split into bf16 hi/lo in place; W is built from the CB
// accumulator in TMEM and reuses the dead B tile.  With dstate 64 the x and S tiles are double buffered,
// so the next head's loads are in flight while this head computes.  The state product is issued as soon
// as S is split and runs under the W pass; the output tile is staged in the dead x tile and written by TMA.
#include "ssd_decay.cuh"
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

template <int N>
struct ChunkScanSmem {
    static constexpr int kBuf = N == 64 ? 3 : 1;                      // x / S tile buffers (a ring)
    static constexpr int kOffBuf = N == 64 ? 2 : 1;                   // C*S accumulators
    static constexpr uint32_t kCTile = kTile * 128 * 2 * (N / 64);    // [128 x N]: N/64 blocks of (hi | lo)
    static constexpr uint32_t kXTile = kTile * 128 * 2;               // [128 x 64] (hi | lo)
    static constexpr uint32_t kSTile = 64 * 128 * 2 * (N / 64);       // [64 x N]
    static constexpr uint32_t kC = 0;
    static constexpr uint32_t kB = kC + kCTile;
    static constexpr uint32_t kX = kB + kCTile;
    static constexpr uint32_t kS = kX + kBuf * kXTile;
    static constexpr uint32_t kRows = kS + kBuf * kSTile;
    static constexpr uint32_t kRowSet = 2 * kTile;              // cs[128], q[128]
    static constexpr uint32_t kBars = kRows + 3 * kRowSet * 4;  // three row sets in rotation
    static constexpr uint32_t kTotal = kBars + 256;
};
static_assert(ChunkScanSmem<64>::kTotal + 1024 <= 232448 && ChunkScanSmem<128>::kTotal + 1024 <= 232448,
              "output kernel exceeds the shared memory of one SM");

template <int N>
__global__ void __launch_bounds__(kLaunchThreadsGroups, 1)
chunk_scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_s,
                  const __grid_constant__ CUtensorMap map_out, const float* __restrict__ q,
                  const float* __restrict__ cs, SsdShape s, int* status) {
    using L = ChunkScanSmem<N>;
    constexpr int NB = L::kBuf;
    constexpr int NOFF = L::kOffBuf;
    constexpr int kBlocks = N / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* rows = reinterpret_cast<float*>(smem + L::kRows);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_x = bars;          // [3] x tile has landed
    uint64_t* full_s = bars + 3;      // [3] S tile has landed
    uint64_t* full_c = bars + 6;      // C and B tiles have landed
    uint64_t* bar_cb = bars + 7;      // CB done
    uint64_t* bar_y = bars + 8;       // both products of a head done
    uint64_t* bar_rcb = bars + 9;     // C in tensor memory, B tile split
    // S tile split (and accumulators free), one barrier per iteration parity.  The S tile of iteration it + 1 is
    // prepared -- and its arrivals made -- during iteration it, before the issuing thread is known to have seen
    // the completion of iteration it's own phase; with a single barrier a delayed issuing thread could find
    // two phases completed, read the parity as "not yet" and wait for ever.  Arrivals on one of the two
    // barriers are two iterations apart, and the later one needs the products of the iteration between them.
    auto bar_rs = [&](int it) { return bars + 10 + 3 * (it & 1); };  // bars[10] and bars[13]
    uint64_t* bar_rw = bars + 11;     // W and x ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    uint64_t* rows_ready = bars + 14;  // [3] the rows of an iteration are published (set it % 3)
    uint64_t* rows_free = bars + 17;   // [3] every compute warp has finished with them
    // both products of a head done, once more per S buffer for the producer warp: the compute warps may finish
    // two heads while it is busy with a store, and a waiter that misses two completions of one barrier reads
    // the parity as "not yet" for ever; the next completion on a buffer's barrier needs the S tile that the
    // producer loads after this one
    uint64_t* bar_yp = bars + 23;      // [3]
    uint64_t* staged = bars + 20;      // [3] the output tile is staged in x buffer it % NB (an mbarrier per buffer:
                                       //     the compute warps may run up to two heads ahead of the producer warp)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    // Work list of this CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the (batch, group, token tile)
    // grid, token tile fastest; the heads of all its tiles form one flat sequence of iterations.
    const int num_tiles = s.batch * s.ngroups * nchunks;
    const int my_tiles = (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                         static_cast<int>(gridDim.x);
    const int total = my_tiles * heads_per_group;
    const TileWalk walk(s, static_cast<int>(gridDim.x));

    if (total <= 0) return;  // no work item for this CTA: leave before anything is allocated
    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below, so that no warp is ever
    // left waiting on a barrier that departed warps will not reach.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 9; ++i) mbar_init(&bars[i], 1);
        for (int i = 0; i < 3; ++i) mbar_init(&bar_yp[i], 1);
        for (int i = 9; i < 12; ++i) mbar_init(&bars[i], kThreads / 32);
        mbar_init(&bars[13], kThreads / 32);
        for (int i = 0; i < 3; ++i) {
            mbar_init(&rows_ready[i], 32);
            mbar_init(&rows_free[i], kThreads / 32);
            mbar_init(&staged[i], kThreads / 32);
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
    // CB [128], W*x accumulator [64], W as an A operand: hi [64] and lo [64] columns (row t in lane t, two
    // bf16 contraction elements per column), C*S accumulator [64] (two of them, by iteration parity, when the
    // x / S tiles have a ring of buffers), C as an A operand for both of its products: hi [N/2] and lo [N/2] columns
    const uint32_t tm_cb = tmem, tm_diag = tmem + 128, tm_whi = tmem + 192, tm_wlo = tmem + 256;
    auto tm_off = [&](int it) { return tmem + 320u + static_cast<uint32_t>(it % NOFF) * 64u; };
    const uint32_t tm_chi = tmem + 320 + NOFF * 64, tm_clo = tm_chi + N / 2;
    static_assert(320 + NOFF * 64 + N <= 512, "tensor memory columns");
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;       // hi -> lo distance inside a 128-row block
    constexpr uint32_t kSHalf = 64 * 128;         // the same for a 64-row block

    // ---- warp 16: issues every tensor-core instruction of the CTA
    if (warp >= kThreads / 32) {
        reg_release<kIssuerRegs>();  // this warp group hands most of its registers to the computing groups
        if (warp == kThreads / 32 && lane == 0) {
            const Operand bm{smem_u32(smem + L::kB), smem_u32(smem + L::kB) + kHalf, kTile, false, 2 * kHalf};
            uint32_t pcb = 0, ps = 0, pw = 0;  // ps: one parity bit per S-ready barrier
            int hi = 0;
            for (int it = 0; it < total; ++it) {
                if (hi == 0) {  // a new tile: its C is in tensor memory, its B is split
                    mbar_wait(bar_rcb, pcb, status, kStatusMmaTimeout | wait_site(3, 1));
                    pcb ^= 1;
                    tc_fence_after_sync();
                    issue_gemm_split_ta<N / 16>(tm_cb, tm_chi, tm_clo, bm, 0, make_idesc_bf16(128, 128, false, false),
                                                false);
                    umma_commit(bar_cb);
                }
                const uint32_t xb = smem_u32(smem + L::kX + (it % NB) * L::kXTile);
                const uint32_t sb = smem_u32(smem + L::kS + (it % NB) * L::kSTile);
                const Operand x{xb, xb + kHalf, kTile, true};
                const Operand st{sb, sb + kSHalf, 64, false, 2 * kSHalf};
                mbar_wait(bar_rs(it), (ps >> (it & 1)) & 1u, status, kStatusMmaTimeout | wait_site(3, 2));
                ps ^= 1u << (it & 1);
                tc_fence_after_sync();
                issue_gemm_split_ta<N / 16>(tm_off(it), tm_chi, tm_clo, st, 0, make_idesc_bf16(128, 64, false, false), false);
                mbar_wait(bar_rw, pw, status, kStatusMmaTimeout | wait_site(3, 3));
                pw ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<kTile / 16>(tm_diag, tm_whi, tm_wlo, x, 0, make_idesc_bf16(128, 64, false, true), false);
                umma_commit(bar_y);
                umma_commit(&bar_yp[it % NB]);
                if (++hi == heads_per_group) hi = 0;
            }
        }
        // ---- warp 17: the producer.  Lane 0 issues every TMA load as soon as the memory it lands in is free (it
        // waits on the same barriers of finished products as the compute warps) and every store of an output
        // tile; the coordinates of the next loads are ready before the wait.
        if (warp == kThreads / 32 + 1) {
            auto load_x = [&](int it, const HeadPos& w) {
                tma_tile_3d(smem + L::kX + (it % NB) * L::kXTile, kTile, &map_x, &full_x[it % NB], 0, w.h, w.tok0);
            };
            auto load_s = [&](int it, const HeadPos& w) {
                mbar_arrive_expect_tx(&full_s[it % NB], L::kSTile);
                for (int cb = 0; cb < kBlocks; ++cb)
                    tma_tile_2d(smem + L::kS + (it % NB) * L::kSTile + cb * 2 * kSHalf, 64, &map_s, &full_s[it % NB],
                                64 * cb, w.tile_index * 64, false);
            };
            auto load_cb = [&](const HeadPos& w) {  // C and B of a tile
                mbar_arrive_expect_tx(full_c, 2 * L::kCTile);
                for (int cb = 0; cb < kBlocks; ++cb) {
                    tma_tile_3d(smem + L::kC + cb * 2 * kHalf, kTile, &map_c, full_c, 64 * cb, w.g, w.tok0, false);
                    tma_tile_3d(smem + L::kB + cb * 2 * kHalf, kTile, &map_b, full_c, 64 * cb, w.g, w.tok0, false);
                }
            };
            TilePos cur = walk.first(static_cast<int>(blockIdx.x));
            int hi = 0;
            if (lane == 0) {
                load_cb(walk.locate(cur, 0, 0));
                for (int it = 0; it < NB && it < total; ++it) {
                    const HeadPos w = walk.locate(cur, 0, it);
                    load_s(it, w);
                    load_x(it, w);
                }
            }
            uint32_t pcb = 0;
            for (int it = 0; it < total; ++it) {
                const HeadPos w0 = walk.locate(cur, hi, 0), wn = walk.locate(cur, hi, NB);
                if (hi == 0) {
                    // CB of this tile exists: B has been read and C is in tensor memory, the next tile's may land
                    const HeadPos wt = walk.locate(cur, 0, heads_per_group);
                    mbar_wait(bar_cb, pcb, status, kStatusMmaTimeout | wait_site(3, 9));
                    pcb ^= 1;
                    tc_fence_after_sync();
                    if (lane == 0 && it + heads_per_group < total) load_cb(wt);
                }
                // both products of this head are done: the S buffer is free again
                mbar_wait(&bar_yp[it % NB], static_cast<uint32_t>(it / NB) & 1u, status,
                          kStatusMmaTimeout | wait_site(3, 10));
                tc_fence_after_sync();
                if (lane == 0 && it + NB < total) load_s(it + NB, wn);
                // the compute warps have staged the output tile in this head's (dead) x tile
                mbar_wait(&staged[it % NB], static_cast<uint32_t>(it / NB) & 1u, status,
                          kStatusMmaTimeout | wait_site(3, 14));
                if (lane == 0) {
                    if (*reinterpret_cast<volatile int*>(status) == 0) {
                        const uint8_t* stage = smem + L::kX + (it % NB) * L::kXTile;
                        tma_store_3d(&map_out, stage, 0, w0.h, w0.tok0);
                        tma_store_3d(&map_out, stage + kHalf, 32, w0.h, w0.tok0);
                        tma_store_commit();
                    }
                    if (it + NB < total) {  // then the buffer can take the next x tile that maps to it
                        tma_store_wait_read();
                        load_x(it + NB, wn);
                    }
                }
                if (++hi == heads_per_group) {
                    hi = 0;
                    walk.advance(cur);
                }
            }
            if (lane == 0) tma_store_wait_all();
        }
        // ---- warp 18 publishes the rows (cs, q) of iteration it + 3 into set it % 3 as soon as every compute
        // warp has finished with iteration it; the values are fetched before the wait.
        if (warp == kThreads / 32 + 2) {
            TilePos cur = walk.first(static_cast<int>(blockIdx.x));
            int hi = 0;
            float c[4], qv[4];
            auto fetch = [&](const HeadPos& w) {
                const size_t o = static_cast<size_t>(w.tile_index) * kTile;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    c[j] = cs[o + 32 * j + lane];
                    qv[j] = q[o + 32 * j + lane];
                }
            };
            auto publish = [&](int it) {
                float* set = rows + (it % 3) * L::kRowSet;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    set[32 * j + lane] = c[j];
                    set[kTile + 32 * j + lane] = qv[j];
                }
                mbar_arrive(&rows_ready[it % 3]);
            };
            for (int it = 0; it < 3 && it < total; ++it) {
                fetch(walk.locate(cur, 0, it));
                publish(it);
            }
            for (int it = 0; it + 3 < total; ++it) {
                fetch(walk.locate(cur, hi, 3));
                mbar_wait(&rows_free[it % 3], static_cast<uint32_t>(it / 3) & 1u, status,
                          kStatusMmaTimeout | wait_site(3, 11));
                publish(it + 3);
                if (++hi == heads_per_group) {
                    hi = 0;
                    walk.advance(cur);
                }
            }
        }
        return;
    }
    reg_acquire<kComputeRegs>();

    auto x_tile = [&](int it) { return smem + L::kX + (it % NB) * L::kXTile; };
    auto s_tile = [&](int it) { return smem + L::kS + (it % NB) * L::kSTile; };
    auto row_set = [&](int it) { return rows + (it % 3) * L::kRowSet; };

    uint32_t p_c = 0, p_cb = 0;
    // A tile's B is split in place; its C goes to tensor memory (row t in lane t): the thread of row t takes
    // 32 of its N entries from the fp32 tile as it landed (columns 0-31 of a 64-column block sit in the
    // block's first half, 32-63 in its second).  C may only be replaced when the previous tile's state
    // products are done.
    auto split_b = [&]() {
        ok = mbar_wait(full_c, p_c, status, kStatusTmaTimeout | wait_site(3, 4)) && ok;
        p_c ^= 1;
        for (int cb = 0; cb < kBlocks; ++cb) split_tile_inplace(smem + L::kB + cb * 2 * kHalf, kTile, nullptr, warp, lane);
    };
    auto c_to_tmem = [&]() {
        if ((warp >> 2) < N / 32) {
            const uint32_t row = (warp & 3) * 32 + lane, kq = warp >> 2;
            const uint8_t* src = smem + L::kC + (kq >> 1) * 2 * kHalf + (kq & 1) * kHalf;
            float v[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 f = *reinterpret_cast<const float4*>(src + swz(row, c));
                v[4 * c] = f.x;
                v[4 * c + 1] = f.y;
                v[4 * c + 2] = f.z;
                v[4 * c + 3] = f.w;
            }
            uint32_t chi[16], clo[16];
            split32_packed(v, chi, clo);
            tmem_st16(tmem_addr(tm_chi, warp, 16 * kq), chi);
            tmem_st16(tmem_addr(tm_clo, warp, 16 * kq), clo);
            tmem_st_wait();
        }
        signal_issuer(bar_rcb, lane);
    };
    split_b();
    c_to_tmem();

    uint32_t px = 0, ps = 0, y_parity = 0;  // one parity bit per ring slot
    const int t_row = (warp & 3) * 32 + lane;
    const int cg = warp >> 2;  // 32-column chunk of the W pass, 16-column group of the accumulators

    // S and x tiles of an iteration, split in place.  The state product starts as soon as S is split.
    auto prepare_s = [&](int it) {
        const int bi = it % NB;
        ok = mbar_wait(&full_s[bi], (ps >> bi) & 1u, status, kStatusTmaTimeout | wait_site(3, 5)) && ok;
        ps ^= 1u << bi;
        for (int cb = 0; cb < kBlocks; ++cb) split_tile_inplace(s_tile(it) + cb * 2 * kSHalf, 64, nullptr, warp, lane);
        signal_issuer(bar_rs(it), lane);
    };
    auto prepare_x = [&](int it) {
        const int bi = it % NB;
        ok = mbar_wait(&full_x[bi], (px >> bi) & 1u, status, kStatusTmaTimeout | wait_site(3, 6)) && ok;
        px ^= 1u << bi;
        // The causal decay exp(cs_i - cs_j), j <= i, is factored per block of 32 columns with the block's first
        // cs as reference: exp(cs_i - c0) * exp(c0 - cs_j).  The second factor (>= 1, bounded by the decay across
        // 32 tokens) is folded, with q, into the rows of the x tile here, so that the W pass multiplies a whole
        // block of a row by ONE scalar, with no table.  A block whose decay exceeds the fast limit (or whose cs
        // increases) is left unscaled and takes one exp per element in the pass.
        ok = mbar_wait(&rows_ready[it % 3], static_cast<uint32_t>(it / 3) & 1u, status,
                       kStatusMmaTimeout | wait_site(3, 12)) && ok;
        const float* set = row_set(it);
        const float b0 = set[32 * cg];  // rows 8 * warp .. 8 * warp + 7 lie in block warp / 4 = cg
        const float span = b0 - set[32 * cg + 31];
        const int split_row = warp * 8 + (lane & 7);
        float fx = set[kTile + split_row];
        if (span >= 0.f && span < kDecayFastLimit) fx *= __expf(b0 - set[split_row]);
        split_tile_inplace_scaled(x_tile(it), kTile, fx, warp, lane);
    };
    // With a ring of buffers an iteration's tiles are prepared while the tensor core works on the one before it
    // (and their loads were issued two iterations earlier); with one buffer S is prepared before the W pass and x after it (its load flies during the pass).
    prepare_s(0);
    if (NB > 1) prepare_x(0);
    int hi = 0;
    for (int it = 0; it < total; ++it) {
        const float* cs_s = row_set(it);
        const bool last_of_tile = hi == heads_per_group - 1;
        const bool more_tiles = it + 1 < total;
        if (hi == 0) {
            ok = mbar_wait(bar_cb, p_cb, status, kStatusMmaTimeout | wait_site(3, 7)) && ok;  // CB of this tile
            p_cb ^= 1;
            tc_fence_after_sync();
        }
        if (NB == 1 && it > 0) prepare_s(it);

        // ---- W from CB (the previous products are complete, so W's columns are free)
        {
            const int qr = warp & 3;
            float v[32];
            if (cg <= qr) {
                tmem_ld32(tmem_addr(tm_cb, warp, 32 * cg), v);
                // this row's factor for its block of 32 columns (see prepare_x); with one buffer the rows of this
                // iteration are waited for here first
                if (NB == 1)
                    ok = mbar_wait(&rows_ready[it % 3], static_cast<uint32_t>(it / 3) & 1u, status,
                                   kStatusMmaTimeout | wait_site(3, 13)) && ok;
                const float c0 = cs_s[32 * cg];
                const float span = c0 - cs_s[32 * cg + 31];
                const float csi = cs_s[t_row];
                tmem_ld_wait();
                if (span >= 0.f && span < kDecayFastLimit) {
                    const float ei = __expf(fminf(csi - c0, 80.f));
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) v[jj] = (cg < qr || 32 * cg + jj <= t_row) ? v[jj] * ei : 0.f;
                } else {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int j = 32 * cg + jj;
                        const float e = __expf(j <= t_row ? csi - cs_s[j] : 0.f);
                        v[jj] = j <= t_row ? v[jj] * e : 0.f;
                    }
                }
            } else {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) v[jj] = 0.f;
            }
            // W never touches shared memory: each thread writes its 32 entries of row t to tensor memory
            uint32_t whi[16], wlo[16];
            split32_packed(v, whi, wlo);
            tmem_st16(tmem_addr(tm_whi, warp, 16 * cg), whi);
            tmem_st16(tmem_addr(tm_wlo, warp, 16 * cg), wlo);
            tmem_st_wait();
        }
        if (NB == 1) prepare_x(it);
        signal_issuer(bar_rw, lane);  // W and x of this iteration are ready

        // ---- while the tensor core works: the next iteration's tiles (they sit in the other buffers) and,
        //      at the end of a tile, the next tile's B
        if (NB > 1 && more_tiles) {
            prepare_s(it + 1);
            prepare_x(it + 1);
        }
        if (last_of_tile && more_tiles) split_b();

        ok = mbar_wait(bar_y, y_parity, status, kStatusMmaTimeout | wait_site(3, 8)) && ok;
        y_parity ^= 1;
        tc_fence_after_sync();
        // this tile's state products are done: the next tile's C replaces it, and its CB runs under the epilogue
        if (last_of_tile && more_tiles) c_to_tmem();

        // ---- epilogue: out[t, p] = diag + exp(cs_t) * off, staged in this iteration's (dead) x tile
        {
            const float e = expf(cs_s[t_row]);
            float d[16], o[16];
            tmem_ld16(tmem_addr(tm_diag, warp, cg * 16), d);
            tmem_ld16(tmem_addr(tm_off(it), warp, cg * 16), o);
            tmem_ld_wait();
            uint8_t* slab = x_tile(it) + (cg >> 1) * kHalf;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(slab + swz(t_row, (cg & 1) * 4 + (i >> 2))) =
                    make_float4(d[i] + e * o[i], d[i + 1] + e * o[i + 1], d[i + 2] + e * o[i + 2], d[i + 3] + e * o[i + 3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&rows_free[it % 3]);  // this warp has finished with the iteration's rows
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&staged[it % NB]);  // the producer warp writes the staged tile out
        if (++hi == heads_per_group) hi = 0;
    }
    tc_fence_before_sync();
    cta_sync();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int N>
int launch_chunk_scan(const SsdShape& s, const float* x, const float* bm, const float* cm, const float* states,
                      const float* q, const float* cs, float* out, int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_b, map_c, map_s, map_out;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc != SSD_OK) return rc;
    rc = make_tmap_f32_tokens(&map_b, bm, tokens, s.ngroups, s.dstate, kTile);
    if (rc != SSD_OK) return rc;
    rc = make_tmap_f32_tokens(&map_c, cm, tokens, s.ngroups, s.dstate, kTile);
    if (rc != SSD_OK) return rc;
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    rc = make_tmap_f32_2d(&map_s, states, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    rc = make_tmap_f32_tokens(&map_out, out, tokens, s.nheads, s.headdim, kTile);
    if (rc != SSD_OK) return rc;
    const size_t smem = ChunkScanSmem<N>::kTotal + 1024;
    static std::atomic<uint64_t> smem_set{0};  // one per instantiation
    rc = set_max_smem_once(reinterpret_cast<const void*>(chunk_scan_kernel<N>), smem, smem_set);
    if (rc != SSD_OK) return rc;
    const int tiles = (s.seqlen / kTile) * s.ngroups * s.batch;
    const int sms = sm_count();
    if (sms <= 0) return SSD_ERR_LAUNCH;
    const dim3 grid(tiles < sms ? tiles : sms);  // persistent: one CTA per SM walks its share of the tiles
    chunk_scan_kernel<N><<<grid, kLaunchThreadsGroups, smem, stream>>>(map_x, map_b, map_c, map_s, map_out, q, cs, s, status);
    return launch_status();
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_scan_fwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                                  const float* states_start, const float* q, const float* cs, float* out, int* status,
                                  ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!x || !bm || !cm || !states_start || !q || !cs || !out || !status) return SSD_ERR_NULL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    return shape->dstate == 64 ? launch_chunk_scan<64>(*shape, x, bm, cm, states_start, q, cs, out, status, st)
                               : launch_chunk_scan<128>(*shape, x, bm, cm, states_start, q, cs, out, status, st);
}
