// Backward kernel for dx and the whole dt stage.  One CTA per (batch, group, tile of 128 tokens), heads
// of the group in sequence; 16 compute warps plus one warp that only issues tensor-core instructions.
//
//   CB^T     = B * C^T                                        once per group   (tcgen05, A = B from TMEM)
//   W_h^T    = triu(CB^T .* exp(cs_i - cs_j))   [rows j]       TMEM -> registers -> TMEM (A operand, bf16 hi/lo)
//   D1[j,p]  = sum_i W_h[i,j] * dout[i,p]                      (A = W^T from TMEM, never in shared memory)
//   D2[t,p]  = sum_n B[t,n]  * dU_h[p,n]                       dU = d loss / d (state after this tile)
//   dxdt     = D1 + exp(cs_last - cs_t) .* D2 ;  dx = q_t .* dxdt
//
// and, per row t, the gradient with respect to the cumulative decay cs_t:
//
//   g_cs[t] = sum_p dout*out  -  q_t * sum_p x*D1  -  q_t * decay_t * sum_p x*D2
//   g_cs[T-1] += sum_t q_t * decay_t * sum_p x*D2  +  g_last            (g_last from the state scan)
//
// (the first term equals rowsum(dW.*W) plus the state-to-output term because out = W*xdt + exp(cs)*C*S;
// the second is colsum(dW.*W); the third is the chunk-state weight).  A reverse in-tile cumulative sum
// of g_cs gives gw_t, then  ddt_t = (sum_p dxdt*x + A_h*gw_t) * softplus'(dt_t)  and the partial
// dA = sum_t gw_t*q_t.  All reductions are fixed-order; the dt stage runs in fp64 on warps 12-15 while
// the other warps already build the next head's W tile.
//
// Every fp32 tile is loaded by TMA straight into its operand tile's memory and split in place; the
// dout tile is double buffered, so all loads of head h+1 are in flight while head h computes.
#include "ssd_decay.cuh"
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

// dstate N = 64 only
struct BwdDxSmem {
    static constexpr int N = 64;
    static constexpr uint32_t kPTile = kTile * 128 * 2;  // [128 x 64] hi + lo (= the fp32 tile)
    static constexpr uint32_t kUTile = 64 * 128 * 2;     // dU [64 x 64] hi + lo
    static constexpr uint32_t kB = 0;               // fp32 B as it landed (it goes to tensor memory), then the x tiles
    static constexpr uint32_t kG0 = kB + kPTile;    // dout of even heads, then their fp32 dx slabs
    static constexpr uint32_t kG1 = kG0 + kPTile;   // C (for CB only), then dout / dx of odd heads
    static constexpr uint32_t kO = kG1 + kPTile;    // fp32 forward output tile
    static constexpr uint32_t kU = kO + kPTile;
    static constexpr uint32_t kRows = kU + kUTile;
    // float rows: 2 x (cs[128], q[128], decay table[128]); go[2][4][128]; pa[2][4][128]; pb[2][4][128] (by head
    // parity); double scratch[160]
    static constexpr uint32_t kRowSet = 2 * kTile + kDecayColTableFloats;
    static constexpr uint32_t kRowFloats = 2 * kRowSet + 24 * kTile + 320;
    static constexpr uint32_t kBars = kRows + kRowFloats * 4;
    static constexpr uint32_t kTotal = kBars + 128;
};
static_assert(BwdDxSmem::kTotal + 1024 <= 232448, "dx kernel exceeds the shared memory of one SM");
static_assert((BwdDxSmem::kRows + (2 * BwdDxSmem::kRowSet + 24 * kTile) * 4) % 8 == 0, "double scratch alignment");

// SKIP: the D skip connection's share of dx, D .* dy, is added in the epilogue (dy is what this kernel is
// given as dout; the thread reads its 16 values again from global memory, where the tile load of a moment
// ago has left them in L2).  d_mode 1: D[H], 2: D[H,P].
template <bool SKIP>
__global__ void __launch_bounds__(kLaunchThreadsGroups, 1)
bwd_dx_kernel(const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
              const __grid_constant__ CUtensorMap map_dout, const __grid_constant__ CUtensorMap map_out,
              const __grid_constant__ CUtensorMap map_du, const __grid_constant__ CUtensorMap map_dx,
              const __grid_constant__ CUtensorMap map_x, const float* __restrict__ q, const float* __restrict__ cs,
              const float* __restrict__ dt, const float* __restrict__ dt_bias, const float* __restrict__ A,
              const float* __restrict__ g_last, float* __restrict__ ddt_t, double* __restrict__ dA_part,
              const float* __restrict__ dy_raw, const float* __restrict__ dskip, int d_mode, SsdShape s, int* status) {
    using L = BwdDxSmem;
    constexpr int N = L::N;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* rows = reinterpret_cast<float*>(smem + L::kRows);
    float* go_p = rows + 2 * L::kRowSet;   // [2][4][128] partial sum_p dout*out, per head parity
    float* pa_p = go_p + 8 * kTile;        // [2][4][128] partial sum_p x*D1, per head parity
    float* pb_p = pa_p + 8 * kTile;        // [2][4][128] partial sum_p x*D2, per head parity
    double* red_d = reinterpret_cast<double*>(pb_p + 8 * kTile);  // [160] scratch of the dt stage
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_g = bars;           // [2] dout tile of even / odd heads has landed (odd: also C)
    uint64_t* full_o = bars + 2;       // forward output tile has landed
    uint64_t* full_u = bars + 3;       // dU tile has landed
    uint64_t* full_b = bars + 4;       // B tile has landed
    uint64_t* bar_cb = bars + 5;       // CB done
    uint64_t* bar_d2 = bars + 6;       // D2 done
    uint64_t* bar_d1 = bars + 7;       // D1 done
    uint64_t* bar_rcb = bars + 8;      // C and B tiles split
    uint64_t* bar_ra = bars + 9;       // dU tile split (and D2 accumulator free)
    uint64_t* bar_rb = bars + 10;      // W and dout tiles ready (and D1 accumulator free)
    uint64_t* full_x = bars + 11;      // x tile has landed (in the B tile's memory, dead once B is in TMEM)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;
    const int h_first = g * heads_per_group;
    const bool softplus = (s.flags & SSD_FLAG_DT_SOFTPLUS) != 0;


    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below, so that no warp is ever
    // left waiting on a barrier that departed warps will not reach.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 8; ++i) mbar_init(&bars[i], 1);
        for (int i = 8; i < 11; ++i) mbar_init(&bars[i], kThreads / 32);
        mbar_init(full_x, 1);
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
    // CB^T [128], D1 [64], D2 [64]; A operands (row in lane, two bf16 contraction elements per column):
    // B hi [32] | lo [32] for CB^T and D2, W^T hi [64] | lo [64] for D1
    const uint32_t tm_cb = tmem, tm_d1 = tmem + 128, tm_d2 = tmem + 192, tm_bhi = tmem + 256, tm_blo = tmem + 288;
    const uint32_t tm_whi = tmem + 320, tm_wlo = tmem + 384;
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;  // hi -> lo distance of a [128 x 64] tile

    // ---- warp 16: issues every tensor-core instruction of the CTA
    if (warp >= kThreads / 32) {
        reg_release<kIssuerRegs>();  // this warp group hands most of its registers to the computing groups
        if (warp == kThreads / 32 && lane == 0) {
            const Operand c{smem_u32(smem + L::kG1), smem_u32(smem + L::kG1) + kHalf, kTile, false};
            const Operand du{smem_u32(smem + L::kU), smem_u32(smem + L::kU) + 64 * 128, 64, false};
            mbar_wait(bar_rcb, 0, status, kStatusMmaTimeout | wait_site(4, 1));
            tc_fence_after_sync();
            issue_gemm_split_ta<N / 16>(tm_cb, tm_bhi, tm_blo, c, 0, make_idesc_bf16(128, 128, false, false), false);
            umma_commit(bar_cb);
            uint32_t pa = 0, pb = 0;
            for (int hi = 0; hi < heads_per_group; ++hi) {
                const uint32_t gbase = smem_u32(smem + ((hi & 1) ? L::kG1 : L::kG0));
                const Operand gy{gbase, gbase + kHalf, kTile, true};
                mbar_wait(bar_ra, pa, status, kStatusMmaTimeout | wait_site(4, 2));
                pa ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<N / 16>(tm_d2, tm_bhi, tm_blo, du, 0, make_idesc_bf16(128, 64, false, false), false);
                umma_commit(bar_d2);
                mbar_wait(bar_rb, pb, status, kStatusMmaTimeout | wait_site(4, 3));
                pb ^= 1;
                tc_fence_after_sync();
                // every warp has consumed the forward-output tile of this head: the next head's may land
                if (hi + 1 < heads_per_group)
                    tma_tile_3d(smem + L::kO, kTile, &map_out, full_o, 0, h_first + hi + 1, tok0);
                issue_gemm_split_ta<kTile / 16>(tm_d1, tm_whi, tm_wlo, gy, 0, make_idesc_bf16(128, 64, false, true), false);
                umma_commit(bar_d1);
            }
        }
        return;
    }
    reg_acquire<kComputeRegs>();

    // ---- loads.  One thread issues them; each lands in its operand tile's own memory.
    auto srow_of = [&](int h) { return ((b * s.nheads + h) * nchunks + k) * 64; };
    auto g_tile = [&](int hi) { return smem + ((hi & 1) ? L::kG1 : L::kG0); };
    if (tid == 0) {
        tma_tile_3d(smem + L::kB, kTile, &map_b, full_b, 0, g, tok0);
        tma_tile_3d(smem + L::kG1, kTile, &map_c, &full_g[1], 0, g, tok0);
        tma_tile_3d(smem + L::kG0, kTile, &map_dout, &full_g[0], 0, h_first, tok0);
        tma_tile_3d(smem + L::kO, kTile, &map_out, full_o, 0, h_first, tok0);
        tma_tile_2d(smem + L::kU, 64, &map_du, full_u, 0, srow_of(h_first));
    }

    // rows (cs, q, decay references, dt) and per-head scalars are fetched one head ahead into registers
    float r_cs = 0.f, r_q = 0.f, r_dt = 0.f, r_ref = 0.f /* cs of the first row of this row's block of 32 */, r_a = 0.f, r_gl = 0.f;
    auto fetch_rows = [&](int h) {
        const size_t bh = static_cast<size_t>(b) * s.nheads + h;
        const size_t o = bh * s.seqlen + k * kTile;
        if (tid < kTile) {  // warps 0-3 publish the rows
            r_cs = cs[o + tid];
            r_q = q[o + tid];
            r_ref = cs[o + (tid & ~31)];
        } else if (tid >= 384) {  // warps 12-15 run the dt stage
            r_dt = dt[(static_cast<size_t>(tok0) + (tid - 384)) * s.nheads + h] + (dt_bias ? dt_bias[h] : 0.f);
            r_a = A[h];
            r_gl = g_last[bh * nchunks + k];
        }
    };
    auto publish_rows = [&](int set) {
        if (tid < kTile) {
            float* cs_w = rows + set * L::kRowSet;
            cs_w[tid] = r_cs;
            cs_w[kTile + tid] = r_q;
            cs_w[2 * kTile + tid] = decay_col_table_entry(r_cs, r_ref);
        }
    };
    fetch_rows(h_first);

    uint32_t pg = 0 /* one parity bit per dout buffer */, po = 0, pu = 0, px = 0, d1_parity = 0, d2_parity = 0;
    ok = mbar_wait(full_b, 0, status, kStatusTmaTimeout | wait_site(4, 4)) && ok;
    // B is an A operand only (of CB^T = B * C^T and D2 = B * dU^T): it goes to tensor memory (row t in lane t)
    // from the fp32 tile as it landed and never needs a shared-memory operand tile
    if (warp < 8) {
        const uint32_t row = (warp & 3) * 32 + lane, kq = warp >> 2;
        const uint8_t* src = smem + L::kB + kq * kHalf;
        float v[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 f = *reinterpret_cast<const float4*>(src + swz(row, c));
            v[4 * c] = f.x;
            v[4 * c + 1] = f.y;
            v[4 * c + 2] = f.z;
            v[4 * c + 3] = f.w;
        }
        uint32_t bhi[16], blo[16];
        split32_packed(v, bhi, blo);
        tmem_st16(tmem_addr(tm_bhi, warp, 16 * kq), bhi);
        tmem_st16(tmem_addr(tm_blo, warp, 16 * kq), blo);
        tmem_st_wait();
    }
    ok = mbar_wait(&full_g[1], (pg >> 1) & 1u, status, kStatusTmaTimeout | wait_site(4, 5)) && ok;  // C
    pg ^= 2u;
    split_tile_inplace(smem + L::kG1, kTile, nullptr, warp, lane);
    signal_issuer(bar_rcb, lane);
    publish_rows(0);
    ok = mbar_wait(full_u, pu, status, kStatusTmaTimeout | wait_site(4, 6)) && ok;  // dU of the first head
    pu ^= 1;
    split_tile_inplace(smem + L::kU, 64, nullptr, warp, lane);
    ok = mbar_wait(bar_cb, 0, status, kStatusMmaTimeout | wait_site(4, 7)) && ok;  // CB^T ready; the C tile is dead
    tc_fence_after_sync();
    if (tid == 0) {
        if (heads_per_group > 1) tma_tile_3d(smem + L::kG1, kTile, &map_dout, &full_g[1], 0, h_first + 1, tok0);
        tma_tile_3d(smem + L::kB, kTile, &map_x, full_x, 0, h_first, tok0);  // B is in TMEM: x takes its memory
    }
    cta_sync();  // rows of the first head are visible

    const int t_row = (warp & 3) * 32 + lane;
    const int cg = warp >> 2;  // 32-column chunk of the W pass, 16-column group of the accumulators
    constexpr int kIoThread = 256;  // issues the dx stores (not one of the dt-stage threads)
    // ---- the dt stage of head `hp` of the group (warps 12-15, whose share of the W pass is the lightest; one
    // thread per row, own barrier), in fp64 so that the long sums feeding dA add no rounding error of their
    // own.  It is run one head late, after the hand-off of the next head's W and dout tiles, so that it fills
    // the wait for that head's D1 product instead of delaying the hand-off.
    float pv_dt = 0.f, pv_a = 0.f, pv_gl = 0.f, pv_q = 0.f, pv_at = 0.f, pv_bt = 0.f;
    double pv_go = 0.0;
    auto dt_stage = [&](int hp) {
        const int t = tid - 384;
        const int h = h_first + hp;
        const size_t bh = static_cast<size_t>(b) * s.nheads + h;
        const int w4 = warp - 12;
        const float qt = pv_q;
        const float a_t = pv_at, b_t = pv_bt;
        double gcs = pv_go - static_cast<double>(qt) * (static_cast<double>(a_t) + b_t);
        // In-warp pieces first, ONE barrier, then every thread combines them in a fixed order:
        //   extra  = sum_t q_t b_t + g_last   (belongs to the last row, hence to every suffix sum)
        //   gw_t   = (suffix sum of gcs inside the warp) + (totals of the later warps) + extra
        //   dA     = sum_t gw_t q_t
        double s_qb = static_cast<double>(qt) * b_t, s_q = qt;
        double sfx = gcs;  // reverse inclusive scan inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const double dn = __shfl_down_sync(0xffffffffu, sfx, d);
            if (lane + d < 32) sfx += dn;
            s_qb += __shfl_xor_sync(0xffffffffu, s_qb, d);
            s_q += __shfl_xor_sync(0xffffffffu, s_q, d);
        }
        double s_sq = sfx * qt;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) s_sq += __shfl_xor_sync(0xffffffffu, s_sq, d);
        if (lane == 0) {
            red_d[w4] = s_qb;
            red_d[4 + w4] = sfx;  // warp total of gcs
            red_d[8 + w4] = s_sq;
            red_d[12 + w4] = s_q;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        const double extra = (red_d[0] + red_d[1]) + (red_d[2] + red_d[3]) + pv_gl;
        double later = 0.0;
        for (int w = 3; w > w4; --w) later += red_d[4 + w];
        const double gw = sfx + later + extra;
        const double dq = static_cast<double>(a_t) + b_t + static_cast<double>(pv_a) * gw;
        // d q / d dt: softplus' (sigmoid) times the clamp's pass-through mask (dt_min <= value <= dt_max)
        // (softplus is positive: with the default limits (0, inf) its value is not needed again)
        float deriv = softplus ? (pv_dt > 20.f ? 1.f : sigmoid_f(pv_dt)) : 1.f;
        if (!softplus || s.dt_min > 0.f || s.dt_max < 3.0e38f) {
            const float pre = softplus ? softplus_f(pv_dt) : pv_dt;
            if (!(pre >= s.dt_min && pre <= s.dt_max)) deriv = 0.f;
        }
        // a padding token takes no step (its q is forced to zero in the forward pass), so neither dt nor
        // dt_bias receives a gradient from it
        if (s.valid_len > 0 && k * kTile + t >= s.valid_len) deriv = 0.f;
        if (ok) ddt_t[bh * s.seqlen + k * kTile + t] = static_cast<float>(dq * deriv);
        if (t == 0 && ok) {
            double acc = 0.0, lat = extra;  // warps from the last to the first: lat = extra + later totals
            for (int w = 3; w >= 0; --w) {
                acc += red_d[8 + w] + lat * red_d[12 + w];
                lat += red_d[4 + w];
            }
            dA_part[bh * nchunks + k] = acc;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");  // scratch is reused by the next head
    };
    for (int hi = 0; hi < heads_per_group; ++hi) {
        const int h = h_first + hi;
        const int gb = hi & 1;
        const float* cs_s = rows + gb * L::kRowSet;
        const float* q_s = cs_s + kTile;
        const float* ej_s = cs_s + 2 * kTile;
        const float cur_dt = r_dt, cur_a = r_a, cur_gl = r_gl;
        if (hi + 1 < heads_per_group) fetch_rows(h + 1);
        signal_issuer(bar_ra, lane);  // this head's dU tile is split (done one head earlier)

        // ---- W^T from CB^T (the previous head's D1 is complete, so W^T's columns are free).  Row j of this
        //      thread, column block wc: the blocks left of the diagonal are zero, so the warps of column
        //      group 3 (which also run the dt stage) take column block 0, the lightest.
        //      A block left of the diagonal is zero for every head of the group and only its own warp ever
        //      writes it: it is written for the first head and left alone after.
        if (3 - cg >= (warp & 3) || hi == 0) {
            const int qr = warp & 3, wc = 3 - cg;
            float v[32];
            if (wc >= qr) {
                tmem_ld32(tmem_addr(tm_cb, warp, 32 * wc), v);
                tmem_ld_wait();
            }
            decay_block_upper(v, t_row, qr, wc, cs_s, ej_s);
            uint32_t whi[16], wlo[16];
            split32_packed(v, whi, wlo);
            tmem_st16(tmem_addr(tm_whi, warp, 16 * wc), whi);
            tmem_st16(tmem_addr(tm_wlo, warp, 16 * wc), wlo);
            tmem_st_wait();
        }

        // ---- dout tile split in place + row sums of dout*out
        ok = mbar_wait(&full_g[gb], (pg >> gb) & 1u, status, kStatusTmaTimeout | wait_site(4, 8)) && ok;
        pg ^= 1u << gb;
        ok = mbar_wait(full_o, po, status, kStatusTmaTimeout | wait_site(4, 9)) && ok;
        po ^= 1;
        {
            const uint8_t* ot = smem + L::kO;
            split_tile_inplace(g_tile(hi), kTile, nullptr, warp, lane, [&](uint32_t r, uint32_t qd, const float* v) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 o = *reinterpret_cast<const float4*>(ot + (qd >> 1) * kHalf + swz(r, (qd & 1) * 4 + i));
                    acc += v[4 * i] * o.x + v[4 * i + 1] * o.y + v[4 * i + 2] * o.z + v[4 * i + 3] * o.w;
                }
                go_p[(gb * 4 + qd) * kTile + r] = acc;
            });
        }
        signal_issuer(bar_rb, lane);
        // The previous head's dx left its dout tile's memory by a TMA store; once the store has read it, the tile
        // of the head after this one lands there.  Waiting for that read right after issuing the store kept this
        // thread's warp ~1400 cycles behind the others on the way to the hand-off above; here the wait is over
        // before it starts, and the tile still has a whole head to arrive.
        if (tid == kIoThread && hi > 0 && hi + 1 < heads_per_group) {
            tma_store_wait_read();
            tma_tile_3d(g_tile(hi + 1), kTile, &map_dout, &full_g[gb ^ 1], 0, h + 1, tok0);
        }
        if (warp >= 12 && hi > 0) dt_stage(hi - 1);
        float4 dyv[4];
        if constexpr (SKIP) {  // this thread's 16 values of dy, in flight under the products
            const float4* src = reinterpret_cast<const float4*>(
                dy_raw + (static_cast<size_t>(tok0 + t_row) * s.nheads + h) * 64 + cg * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) dyv[i] = __ldg(src + i);
        }
        ok = mbar_wait(bar_d2, d2_parity, status, kStatusMmaTimeout | wait_site(4, 10)) && ok;
        d2_parity ^= 1;
        // D2 no longer reads the dU tile: the next head's may land
        if (tid == 0 && hi + 1 < heads_per_group) tma_tile_2d(smem + L::kU, 64, &map_du, full_u, 0, srow_of(h + 1));
        ok = mbar_wait(bar_d1, d1_parity, status, kStatusMmaTimeout | wait_site(4, 11)) && ok;
        d1_parity ^= 1;
        tc_fence_after_sync();

        // ---- epilogue part 1: dx (staged in this head's dout tile, which D1 no longer reads) and the
        //      per-row dot products with x
        const float cs_last = cs_s[kTile - 1];
        ok = mbar_wait(full_x, px, status, kStatusTmaTimeout | wait_site(4, 12)) && ok;
        px ^= 1;
        {
            const float decay = expf(cs_last - cs_s[t_row]);
            const float qt = q_s[t_row];
            float d1[16], d2[16];
            tmem_ld16(tmem_addr(tm_d1, warp, cg * 16), d1);
            tmem_ld16(tmem_addr(tm_d2, warp, cg * 16), d2);
            tmem_ld_wait();
            uint8_t* slab = g_tile(hi) + (cg >> 1) * kHalf;  // columns 0..31 or 32..63
            const uint8_t* xs = smem + L::kB + (cg >> 1) * kHalf;
            float pa = 0.f, pb = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + swz(t_row, (cg & 1) * 4 + c4));
                const float* a = d1 + 4 * c4;
                const float* bb = d2 + 4 * c4;
                pa += xv.x * a[0] + xv.y * a[1] + xv.z * a[2] + xv.w * a[3];
                pb += xv.x * bb[0] + xv.y * bb[1] + xv.z * bb[2] + xv.w * bb[3];
                float4 o = make_float4(qt * (a[0] + decay * bb[0]), qt * (a[1] + decay * bb[1]),
                                       qt * (a[2] + decay * bb[2]), qt * (a[3] + decay * bb[3]));
                if constexpr (SKIP) {
                    float4 dv;
                    if (d_mode == 2) {
                        dv = __ldg(reinterpret_cast<const float4*>(dskip + h * 64 + cg * 16 + 4 * c4));
                    } else {
                        const float d1v = __ldg(dskip + h);
                        dv = make_float4(d1v, d1v, d1v, d1v);
                    }
                    o.x = fmaf(dv.x, dyv[c4].x, o.x);
                    o.y = fmaf(dv.y, dyv[c4].y, o.y);
                    o.z = fmaf(dv.z, dyv[c4].z, o.z);
                    o.w = fmaf(dv.w, dyv[c4].w, o.w);
                }
                *reinterpret_cast<float4*>(slab + swz(t_row, (cg & 1) * 4 + c4)) = o;
            }
            pa_p[(gb * 4 + cg) * kTile + t_row] = pa;
            pb_p[(gb * 4 + cg) * kTile + t_row] = pb;
        }
        if (hi + 1 < heads_per_group) {
            publish_rows(gb ^ 1);  // next head's rows, other buffer
            ok = mbar_wait(full_u, pu, status, kStatusTmaTimeout | wait_site(4, 13)) && ok;  // next head's dU tile
            pu ^= 1;
            split_tile_inplace(smem + L::kU, 64, nullptr, warp, lane);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid == kIoThread && ok) {  // the dout tile of head hi + 2 follows once the store has read the memory: see above
            tma_store_3d(&map_dx, g_tile(hi), 0, h, tok0);
            tma_store_3d(&map_dx, g_tile(hi) + kHalf, 32, h, tok0);
            tma_store_commit();
        }
        // everyone has read x: the next head's x tile may land in its place
        if (tid == 0 && hi + 1 < heads_per_group) tma_tile_3d(smem + L::kB, kTile, &map_x, full_x, 0, h + 1, tok0);

        // the dt stage of this head runs later, under the next head's D1 product.  Its inputs are gathered into
        // registers now, while no product competes for shared memory (under a product each of these reads
        // costs several times as much, and the stage would outlast the product it hides behind)
        if (warp >= 12) {
            const int t = tid - 384;
            const float* go_h = go_p + gb * 4 * kTile;
            const float* pa_h = pa_p + gb * 4 * kTile;
            const float* pb_h = pb_p + gb * 4 * kTile;
            pv_dt = cur_dt;
            pv_a = cur_a;
            pv_gl = cur_gl;
            pv_q = q_s[t];
            pv_at = (pa_h[t] + pa_h[kTile + t]) + (pa_h[2 * kTile + t] + pa_h[3 * kTile + t]);
            pv_bt = expf(cs_last - cs_s[t]) *
                    ((pb_h[t] + pb_h[kTile + t]) + (pb_h[2 * kTile + t] + pb_h[3 * kTile + t]));
            pv_go = (static_cast<double>(go_h[t]) + go_h[kTile + t]) +
                    (static_cast<double>(go_h[2 * kTile + t]) + go_h[3 * kTile + t]);
        }
    }
    if (warp >= 12) dt_stage(heads_per_group - 1);
    if (tid == kIoThread) tma_store_wait_all();
    cta_sync();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_dx_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                                const float* dout, const float* out, const float* dstates, const float* q,
                                const float* cs, const float* dt, const float* dt_bias, const float* A, const float* g_last,
                                float* dx,
                                float* ddt_t, double* dA_partial, const float* D, int d_mode, int* status,
                                ssd_stream_t stream) {
    using namespace ssd;
    const int rc0 = ssd_check_shape(shape);
    if (rc0 != SSD_OK) return rc0;
    if (!x || !bm || !cm || !dout || !out || !dstates || !q || !cs || !dt || !A || !g_last || !dx || !ddt_t ||
        !dA_partial || !status)
        return SSD_ERR_NULL;
    const SsdShape& s = *shape;
    if (s.dstate != 64) return SSD_ERR_UNSUPPORTED;
    if (d_mode < 0 || d_mode > 2) return SSD_ERR_SHAPE;
    if (d_mode != 0 && !D) return SSD_ERR_NULL;
    CUtensorMap map_b, map_c, map_dout, map_out, map_du, map_dx, map_x;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_b, bm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_c, cm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dout, dout, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_out, out, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dx, dx, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_du, dstates, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    const size_t smem = BwdDxSmem::kTotal + 1024;
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (d_mode == 0) {
        static std::atomic<uint64_t> smem_set{0};
        rc = set_max_smem_once(reinterpret_cast<const void*>(bwd_dx_kernel<false>), smem, smem_set);
        if (rc != SSD_OK) return rc;
        bwd_dx_kernel<false><<<grid, kLaunchThreadsGroups, smem, st>>>(
            map_b, map_c, map_dout, map_out, map_du, map_dx, map_x, q, cs, dt, dt_bias, A, g_last, ddt_t, dA_partial,
            nullptr, nullptr, 0, s, status);
    } else {
        static std::atomic<uint64_t> smem_set{0};
        rc = set_max_smem_once(reinterpret_cast<const void*>(bwd_dx_kernel<true>), smem, smem_set);
        if (rc != SSD_OK) return rc;
        bwd_dx_kernel<true><<<grid, kLaunchThreadsGroups, smem, st>>>(
            map_b, map_c, map_dout, map_out, map_du, map_dx, map_x, q, cs, dt, dt_bias, A, g_last, ddt_t, dA_partial,
            dout, D, d_mode, s, status);
    }
    return launch_status();
}
