// Forward output kernel.  One CTA per (batch, group, tile of 128 tokens), heads of the group in sequence;
// 16 compute warps plus one warp that only issues tensor-core instructions.
//
//   CB      = C * B^T                                   once per group        [T,T]   (tcgen05)
//   W_h     = tril(CB .* exp(cs_i - cs_j))              per head, TMEM -> registers -> split bf16 tile
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

PROF_DECL(scan)

namespace ssd {

namespace {

template <int N>
struct ChunkScanSmem {
    static constexpr int kBuf = N == 64 ? 2 : 1;                      // x / S tile buffers
    static constexpr uint32_t kCTile = kTile * 128 * 2 * (N / 64);    // [128 x N]: N/64 blocks of (hi | lo)
    static constexpr uint32_t kWTile = kTile * 128 * 2;               // [128 x 128], one of hi/lo
    static constexpr uint32_t kXTile = kTile * 128 * 2;               // [128 x 64] (hi | lo)
    static constexpr uint32_t kSTile = 64 * 128 * 2 * (N / 64);       // [64 x N]
    static constexpr uint32_t kBW = kCTile > 2 * kWTile ? kCTile : 2 * kWTile;
    static constexpr uint32_t kC = 0;
    static constexpr uint32_t kB = kC + kCTile;  // B first, later W (hi tile, lo tile)
    static constexpr uint32_t kWHi = kB;
    static constexpr uint32_t kWLo = kWHi + kWTile;
    static constexpr uint32_t kX = kB + kBW;
    static constexpr uint32_t kS = kX + kBuf * kXTile;
    static constexpr uint32_t kRows = kS + kBuf * kSTile;
    static constexpr uint32_t kRowSet = 2 * kTile + kDecayTableFloats;  // cs[128], q[128], decay table
    static constexpr uint32_t kBars = kRows + 3 * kRowSet * 4;  // three row sets in rotation
    static constexpr uint32_t kTotal = kBars + 128;
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
    constexpr int kBlocks = N / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* rows = reinterpret_cast<float*>(smem + L::kRows);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_x = bars;          // [2] x tile has landed
    uint64_t* full_s = bars + 2;      // [2] S tile has landed
    uint64_t* full_c = bars + 4;      // C and B tiles have landed
    uint64_t* bar_cb = bars + 5;      // CB done
    uint64_t* bar_y = bars + 6;       // both products of a head done
    uint64_t* bar_rcb = bars + 7;     // C and B tiles split
    uint64_t* bar_rs = bars + 8;      // S tile split (and accumulators free)
    uint64_t* bar_rw = bars + 9;      // W and x tiles ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;
    const int h_first = g * heads_per_group;

    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    PROF_BEGIN()

    if (tid == 0) {
        for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
        for (int i = 7; i < 10; ++i) mbar_init(&bars[i], kThreads / 32);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // CB [128], W*x accumulator [64], W as an A operand: hi [64] and lo [64] columns (row t in lane t, two
    // bf16 contraction elements per column), C*S accumulator [64] (two of them, by head parity, when the x / S
    // tiles are double buffered), C as an A operand for both of its products: hi [N/2] and lo [N/2] columns
    const uint32_t tm_cb = tmem, tm_diag = tmem + 128, tm_whi = tmem + 192, tm_wlo = tmem + 256;
    auto tm_off = [&](int hi) { return tmem + 320u + static_cast<uint32_t>(hi % NB) * 64u; };
    const uint32_t tm_chi = tmem + 320 + NB * 64, tm_clo = tm_chi + N / 2;
    static_assert(320 + NB * 64 + N <= 512, "tensor memory columns");
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;       // hi -> lo distance inside a 128-row block
    constexpr uint32_t kSHalf = 64 * 128;         // the same for a 64-row block

    // ---- warp 16: issues every tensor-core instruction of the CTA
    if (warp >= kThreads / 32) {
        reg_release<kIssuerRegs>();  // this warp group hands most of its registers to the computing groups
        if (warp == kThreads / 32 && lane == 0) {
            const Operand bm{smem_u32(smem + L::kB), smem_u32(smem + L::kB) + kHalf, kTile, false, 2 * kHalf};
            mbar_wait(bar_rcb, 0, status, kStatusMmaTimeout);
            tc_fence_after_sync();
            issue_gemm_split_ta<N / 16>(tm_cb, tm_chi, tm_clo, bm, 0, make_idesc_bf16(128, 128, false, false), false);
            umma_commit(bar_cb);
            uint32_t ps = 0, pw = 0;
            for (int hi = 0; hi < heads_per_group; ++hi) {
                const uint32_t xb = smem_u32(smem + L::kX + (hi % NB) * L::kXTile);
                const uint32_t sb = smem_u32(smem + L::kS + (hi % NB) * L::kSTile);
                const Operand x{xb, xb + kHalf, kTile, true};
                const Operand st{sb, sb + kSHalf, 64, false, 2 * kSHalf};
                mbar_wait(bar_rs, ps, status, kStatusMmaTimeout);
                ps ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<N / 16>(tm_off(hi), tm_chi, tm_clo, st, 0, make_idesc_bf16(128, 64, false, false), false);
                mbar_wait(bar_rw, pw, status, kStatusMmaTimeout);
                pw ^= 1;
                tc_fence_after_sync();
                issue_gemm_split_ta<kTile / 16>(tm_diag, tm_whi, tm_wlo, x, 0, make_idesc_bf16(128, 64, false, true), false);
                umma_commit(bar_y);
            }
        }
        return;
    }
    reg_acquire<kComputeRegs>();

    // ---- loads.  Each lands in its operand tile's own memory.
    auto x_tile = [&](int hi) { return smem + L::kX + (hi % NB) * L::kXTile; };
    auto s_tile = [&](int hi) { return smem + L::kS + (hi % NB) * L::kSTile; };
    auto load_x = [&](int hi) { tma_tile_3d(x_tile(hi), kTile, &map_x, &full_x[hi % NB], 0, h_first + hi, tok0); };
    auto load_s = [&](int hi) {
        const int srow = ((b * s.nheads + h_first + hi) * nchunks + k) * 64;
        mbar_arrive_expect_tx(&full_s[hi % NB], L::kSTile);
        for (int cb = 0; cb < kBlocks; ++cb)
            tma_tile_2d(s_tile(hi) + cb * 2 * kSHalf, 64, &map_s, &full_s[hi % NB], 64 * cb, srow, false);
    };
    if (tid == 0) {
        mbar_arrive_expect_tx(full_c, 2 * L::kCTile);
        for (int cb = 0; cb < kBlocks; ++cb) {
            tma_tile_3d(smem + L::kC + cb * 2 * kHalf, kTile, &map_c, full_c, 64 * cb, g, tok0, false);
            tma_tile_3d(smem + L::kB + cb * 2 * kHalf, kTile, &map_b, full_c, 64 * cb, g, tok0, false);
        }
        for (int hi = 0; hi < NB && hi < heads_per_group; ++hi) {
            load_s(hi);
            load_x(hi);
        }
    }

    // rows (cs, q, decay references) go through registers into three shared-memory sets in rotation
    // (head hi reads set hi % 3): the set of head hi + 2 is written while heads hi and hi + 1 read theirs
    struct RowRegs {
        float cs = 0.f, q = 0.f, ref[4] = {0.f, 0.f, 0.f, 0.f};
    };
    RowRegs r_a, r_b;
    auto fetch_rows = [&](RowRegs& r, int h) {
        if (tid < kTile) {
            const size_t o = (static_cast<size_t>(b) * s.nheads + h) * s.seqlen + k * kTile;
            r.cs = cs[o + tid];
            r.q = q[o + tid];
#pragma unroll
            for (int i = 0; i < 4; ++i) r.ref[i] = cs[o + 32 * i];
        }
    };
    auto row_set = [&](int hi) { return rows + (hi % 3) * L::kRowSet; };
    auto publish_rows = [&](const RowRegs& r, int hi) {
        if (tid < kTile) {
            float* cs_w = row_set(hi);
            cs_w[tid] = r.cs;
            cs_w[kTile + tid] = r.q;
            decay_table_fill(cs_w + 2 * kTile, tid, r.cs, r.ref);
        }
    };
    fetch_rows(r_a, h_first);  // the first two heads' rows are in flight together
    if (heads_per_group > 1) fetch_rows(r_b, h_first + 1);

    ok = mbar_wait(full_c, 0, status, kStatusTmaTimeout) && ok;
    for (int cb = 0; cb < kBlocks; ++cb) split_tile_inplace(smem + L::kB + cb * 2 * kHalf, kTile, nullptr, warp, lane);
    // C goes to tensor memory (row t in lane t): the thread of row t takes 32 of its N entries from the fp32
    // tile as it landed (columns 0-31 of a 64-column block sit in the block's first half, 32-63 in its second)
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
    publish_rows(r_a, 0);
    if (heads_per_group > 1) publish_rows(r_b, 1);
    if (heads_per_group > 2) fetch_rows(r_a, h_first + 2);
    cta_sync();  // rows of the first two heads are visible

    uint32_t px[2] = {0, 0}, ps[2] = {0, 0}, y_parity = 0;
    const int t_row = (warp & 3) * 32 + lane;
    const int cg = warp >> 2;  // 32-column chunk of the W pass, 16-column group of the accumulators
    constexpr int kIoThread = 256;

    // S and x tiles of a head, split in place.  The state product starts as soon as S is split.
    auto prepare_s = [&](int hi) {
        const int bi = hi % NB;
        ok = mbar_wait(&full_s[bi], ps[bi], status, kStatusTmaTimeout) && ok;
        ps[bi] ^= 1;
        for (int cb = 0; cb < kBlocks; ++cb) split_tile_inplace(s_tile(hi) + cb * 2 * kSHalf, 64, nullptr, warp, lane);
        signal_issuer(bar_rs, lane);
    };
    auto prepare_x = [&](int hi) {
        const int bi = hi % NB;
        ok = mbar_wait(&full_x[bi], px[bi], status, kStatusTmaTimeout) && ok;
        px[bi] ^= 1;
        split_tile_inplace(x_tile(hi), kTile, row_set(hi) + kTile, warp, lane);  // scaled by q
    };
    // With two buffers a head's tiles are prepared while the tensor core works on the head before it; with
    // one buffer S is prepared before the W pass and x after it (its load flies during the pass).
    prepare_s(0);
    if (NB == 2) prepare_x(0);
    ok = mbar_wait(bar_cb, 0, status, kStatusMmaTimeout) && ok;  // CB ready
    tc_fence_after_sync();
    PROF_T(0)
    for (int hi = 0; hi < heads_per_group; ++hi) {
        const int h = h_first + hi;
        const float* cs_s = row_set(hi);
        const float* ej_s = cs_s + 2 * kTile;
        if (NB == 1 && hi > 0) prepare_s(hi);

        // ---- W from CB (the previous head's products are complete, so W's columns are free)
        {
            const int qr = warp & 3;
            float v[32];
            if (cg <= qr) {
                tmem_ld32(tmem_addr(tm_cb, warp, 32 * cg), v);
                tmem_ld_wait();
            }
            decay_block_lower(v, t_row, qr, cg, cs_s, ej_s);
            // W never touches shared memory: each thread writes its 32 entries of row t to tensor memory
            uint32_t whi[16], wlo[16];
            split32_packed(v, whi, wlo);
            tmem_st16(tmem_addr(tm_whi, warp, 16 * cg), whi);
            tmem_st16(tmem_addr(tm_wlo, warp, 16 * cg), wlo);
            tmem_st_wait();
        }
        if (NB == 1) prepare_x(hi);
        signal_issuer(bar_rw, lane);  // W and x of this head are ready
        PROF_T(1)

        // ---- while the tensor core works on this head: the next head's tiles (they sit in the other buffers)
        if (NB == 2 && hi + 1 < heads_per_group) {
            prepare_s(hi + 1);
            prepare_x(hi + 1);
        }
        PROF_T(2)

        ok = mbar_wait(bar_y, y_parity, status, kStatusMmaTimeout) && ok;
        y_parity ^= 1;
        tc_fence_after_sync();
        // the S buffer is free again: with two buffers it takes head hi + 2, with one the next head
        if (tid == 0 && hi + NB < heads_per_group) load_s(hi + NB);
        PROF_T(3)

        // ---- epilogue: out[t, p] = diag + exp(cs_t) * off, staged in this head's (dead) x tile
        {
            const float e = expf(cs_s[t_row]);
            float d[16], o[16];
            tmem_ld16(tmem_addr(tm_diag, warp, cg * 16), d);
            tmem_ld16(tmem_addr(tm_off(hi), warp, cg * 16), o);
            tmem_ld_wait();
            uint8_t* slab = x_tile(hi) + (cg >> 1) * kHalf;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(slab + swz(t_row, (cg & 1) * 4 + (i >> 2))) =
                    make_float4(d[i] + e * o[i], d[i + 1] + e * o[i + 1], d[i + 2] + e * o[i + 2], d[i + 3] + e * o[i + 3]);
        }
        if (hi + 2 < heads_per_group) {
            publish_rows(r_a, hi + 2);
            if (hi + 3 < heads_per_group) fetch_rows(r_a, h + 3);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid == kIoThread) {
            if (ok) {
                tma_store_3d(&map_out, x_tile(hi), 0, h, tok0);
                tma_store_3d(&map_out, x_tile(hi) + kHalf, 32, h, tok0);
                tma_store_commit();
            }
            tma_store_wait_read();  // then the buffer can take the next x tile that maps to it
            if (hi + NB < heads_per_group) load_x(hi + NB);
        }
        PROF_T(4)
    }
    PROF_END(scan)
    if (tid == kIoThread) tma_store_wait_all();
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
    if (cudaFuncSetAttribute(chunk_scan_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return SSD_ERR_LAUNCH;
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
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
