// Backward kernel for dB and dC.  One CTA per (batch, group, tile, mode);
// the gradient of the group is accumulated over its heads in TMEM, so each
// output element is written once by one CTA (no atomics, fixed order).
//
// mode 0 (dC), rows i:
//   D0[i,j]  = sum_p dout[i,p] * xdt[j,p]
//   dCB[i,j] = D0[i,j] * exp(cs_i - cs_j)   for j <= i, else 0
//   dC[i,n] += sum_j dCB[i,j] * B[j,n]  +  sum_p (exp(cs_i) dout[i,p]) * S[p,n]
// mode 1 (dB), rows j:
//   D0[j,i]   = sum_p xdt[j,p] * dout[i,p]
//   dCBt[j,i] = D0[j,i] * exp(cs_i - cs_j)  for i >= j, else 0
//   dB[j,n]  += sum_i dCBt[j,i] * C[i,n]  +  sum_p (exp(cs_last - cs_j) xdt[j,p]) * dU[p,n]
//
// with xdt = q .* x, S the state at the start of the tile and dU the gradient
// of the state after the tile.  Computing the transposed product directly in
// mode 1 keeps every tile the kernel writes row-major in its own output row,
// so both modes share one code path.
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

struct BwdDbcSmem {
    static constexpr int N = 64;
    static constexpr uint32_t kPTile = kTile * 128;      // [128 x 64] one of hi/lo
    static constexpr uint32_t kTTile = kTile * 128 * 2;  // [128 x 128] one of hi/lo
    static constexpr uint32_t kSTile = 64 * 128;         // [64 x 64]
    // region 1: dout tile + xdt tile, later the dCB tile (hi, lo)
    static constexpr uint32_t kGHi = 0;
    static constexpr uint32_t kGLo = kGHi + kPTile;
    static constexpr uint32_t kXHi = kGLo + kPTile;
    static constexpr uint32_t kXLo = kXHi + kPTile;
    static constexpr uint32_t kDHi = 0;
    static constexpr uint32_t kDLo = kDHi + kTTile;
    static constexpr uint32_t kRHi = kDLo + kTTile;  // row-scaled dout (mode 0) or xdt (mode 1)
    static constexpr uint32_t kRLo = kRHi + kPTile;
    static constexpr uint32_t kSHi = kRLo + kPTile;  // S (mode 0) or dU (mode 1)
    static constexpr uint32_t kSLo = kSHi + kSTile;
    static constexpr uint32_t kMHi = kSLo + kSTile;  // group tile: B (mode 0) or C (mode 1)
    static constexpr uint32_t kMLo = kMHi + kPTile;
    static constexpr uint32_t kStage = kMLo + kPTile;  // 4 slabs
    static constexpr uint32_t kRows = kStage + 4 * kSlabBytes;
    static constexpr uint32_t kBars = kRows + 4 * kTile * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};

__global__ void __launch_bounds__(kThreads, 1)
bwd_dbc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_dout,
               const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_du,
               const float* __restrict__ q, const float* __restrict__ cs, float* __restrict__ dB,
               float* __restrict__ dC, SsdShape s, int* status) {
    using L = BwdDbcSmem;
    constexpr int N = L::N;
    constexpr int NS = 4;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* cs_s = reinterpret_cast<float*>(smem + L::kRows);  // [128]
    float* q_s = cs_s + kTile;                                // [128] q_t
    float* w_s = cs_s + 2 * kTile;                            // [128] row weight of the scaled tile
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);  // [0..3] ring, [4] mma
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NS + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z >> 1, mode = blockIdx.z & 1;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;

    if (*reinterpret_cast<volatile int*>(status) != 0) return;

    StageRing<NS> ring;
    ring.init(smem + L::kStage, bars, tid);
    if (tid == 0) {
        mbar_init(&bars[NS], 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_d0 = tmem, tm_acc = tmem + 128;
    bool ok = true;
    uint32_t mma_parity = 0;

    // ---- group tile (B for dC, C for dB), MN-major operand of the dCB product
    {
        const CUtensorMap* map_m = mode == 0 ? &map_b : &map_c;
        auto issue = [&](int i, int slot) { ring.issue3d(slot, map_m, 32 * i, g, tok0, kTile); };
        auto conv = [&](int i, const uint8_t* slab) {
            convert_slab(slab, smem + L::kMHi, smem + L::kMLo, kTile, 32 * i, nullptr, tid, kThreads);
        };
        if (tid == 0) {
            issue(0, 0);
            issue(1, 1);
        }
        ok = run_loads<NS>(ring, 2, issue, conv, tid, status) && ok;
        __syncthreads();
    }

    // per-head loads: dout (2 slabs), x (2 slabs), state (2 slabs of 64 rows)
    constexpr int kHeadLoads = 6;
    const CUtensorMap* map_st = mode == 0 ? &map_s : &map_du;
    auto issue_head = [&](int h, int i, int slot) {
        if (i < 2) {
            ring.issue3d(slot, &map_dout, 32 * i, h, tok0, kTile);
        } else if (i < 4) {
            ring.issue3d(slot, &map_x, 32 * (i - 2), h, tok0, kTile);
        } else {
            ring.issue2d(slot, map_st, 32 * (i - 4), ((b * s.nheads + h) * nchunks + k) * 64, 64);
        }
    };
    if (tid == 0) {
        for (int i = 0; i < NS; ++i) issue_head(g * heads_per_group, i, i);
    }

    float r_cs = 0.f, r_q = 0.f, r_last = 0.f;
    auto fetch_rows = [&](int h) {
        const size_t o = (static_cast<size_t>(b) * s.nheads + h) * s.seqlen + k * kTile;
        r_cs = cs[o + tid];
        r_q = q[o + tid];
        r_last = cs[o + kTile - 1];
    };
    if (tid < kTile) fetch_rows(g * heads_per_group);

    for (int hi = 0; hi < heads_per_group; ++hi) {
        const int h = g * heads_per_group + hi;
        if (hi > 0) {
            // the previous head's accumulating products still read the dCB / scaled / state tiles
            ok = mbar_wait(&bars[NS], mma_parity, status, kStatusMmaTimeout) && ok;
            mma_parity ^= 1;
            tc_fence_after_sync();
        }
        if (tid < kTile) {  // rows fetched one head ahead (registers), published here
            cs_s[tid] = r_cs;
            q_s[tid] = r_q;
            w_s[tid] = mode == 0 ? expf(r_cs) : r_q * expf(r_last - r_cs);
            if (hi + 1 < heads_per_group) fetch_rows(h + 1);
        }
        __syncthreads();

        // ---- dout, xdt tiles (+ the row-scaled copy of one of them), state tile
        {
            auto issue = [&](int i, int slot) { issue_head(h, i, slot); };
            auto conv = [&](int i, const uint8_t* slab) {
                if (i < 2) {
                    convert_slab(slab, smem + L::kGHi, smem + L::kGLo, kTile, 32 * i, nullptr, tid, kThreads);
                    if (mode == 0) convert_slab(slab, smem + L::kRHi, smem + L::kRLo, kTile, 32 * i, w_s, tid, kThreads);
                } else if (i < 4) {
                    convert_slab(slab, smem + L::kXHi, smem + L::kXLo, kTile, 32 * (i - 2), q_s, tid, kThreads);
                    if (mode == 1)
                        convert_slab(slab, smem + L::kRHi, smem + L::kRLo, kTile, 32 * (i - 2), w_s, tid, kThreads);
                } else {
                    convert_slab(slab, smem + L::kSHi, smem + L::kSLo, 64, 32 * (i - 4), nullptr, tid, kThreads);
                }
            };
            ok = run_loads<NS>(ring, kHeadLoads, issue, conv, tid, status) && ok;
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            if (hi + 1 < heads_per_group) {
                for (int i = 0; i < NS; ++i) issue_head(h + 1, i, i);
            }
            tc_fence_after_sync();
            const Operand gy{smem_u32(smem + L::kGHi), smem_u32(smem + L::kGLo), kTile, false};
            const Operand xd{smem_u32(smem + L::kXHi), smem_u32(smem + L::kXLo), kTile, false};
            if (mode == 0) {
                issue_gemm_split<64 / 16>(tm_d0, gy, 0, xd, 0, make_idesc_bf16(128, 128, false, false), false);
            } else {
                issue_gemm_split<64 / 16>(tm_d0, xd, 0, gy, 0, make_idesc_bf16(128, 128, false, false), false);
            }
            umma_commit(&bars[NS]);
        }
        ok = mbar_wait(&bars[NS], mma_parity, status, kStatusMmaTimeout) && ok;
        mma_parity ^= 1;
        tc_fence_after_sync();

        // ---- decay-weighted, masked copy of D0 as the K-major dCB tile (overwrites dout / xdt tiles)
        {
            const int r = (warp & 3) * 32 + lane;
            const int row_lo = (warp & 3) * 32, row_hi = row_lo + 31;
            const float csr = cs_s[r];
            {
                const int c0 = (warp >> 2) * 32;  // one 32-column chunk per warp
                const bool live = mode == 0 ? (c0 <= row_hi) : (c0 + 31 >= row_lo);
                float v[32];
                if (live) {
                    tmem_ld32(tmem_addr(tm_d0, warp, c0), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int col = c0 + jj;
                        const bool keep = mode == 0 ? (col <= r) : (col >= r);
                        const float arg = mode == 0 ? csr - cs_s[col] : cs_s[col] - csr;
                        const float e = __expf(keep ? arg : 0.f);
                        v[jj] = keep ? v[jj] * e : 0.f;
                    }
                } else {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) v[jj] = 0.f;
                }
#pragma unroll
                for (int jj = 0; jj < 32; jj += 8)
                    store_split8(smem + L::kDHi, smem + L::kDLo, kTile, r, c0 + jj, v + jj);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
            const Operand dcb{smem_u32(smem + L::kDHi), smem_u32(smem + L::kDLo), kTile, false};
            const Operand mg{smem_u32(smem + L::kMHi), smem_u32(smem + L::kMLo), kTile, true};
            const Operand rs{smem_u32(smem + L::kRHi), smem_u32(smem + L::kRLo), kTile, false};
            const Operand st{smem_u32(smem + L::kSHi), smem_u32(smem + L::kSLo), 64, true};
            const uint32_t idesc = make_idesc_bf16(128, N, false, true);
            issue_gemm_split<kTile / 16>(tm_acc, dcb, 0, mg, 0, idesc, hi > 0);
            issue_gemm_split<64 / 16>(tm_acc, rs, 0, st, 0, idesc, true);
            umma_commit(&bars[NS]);
        }
    }
    ok = mbar_wait(&bars[NS], mma_parity, status, kStatusMmaTimeout) && ok;
    tc_fence_after_sync();

    // ---- epilogue: the group's gradient rows
    {
        const int t = (warp & 3) * 32 + lane;
        const int n0 = (warp >> 2) * 16;
        float v[16];
        tmem_ld16(tmem_addr(tm_acc, warp, n0), v);
        tmem_ld_wait();
        float* dst = (mode == 0 ? dC : dB) + ((static_cast<size_t>(tok0) + t) * s.ngroups + g) * N + n0;
        if (ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_dbc_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                                 const float* dout, const float* states_start, const float* dstates, const float* q,
                                 const float* cs, float* dB, float* dC, int* status, ssd_stream_t stream) {
    using namespace ssd;
    const int rc0 = ssd_check_shape(shape);
    if (rc0 != SSD_OK) return rc0;
    if (!x || !bm || !cm || !dout || !states_start || !dstates || !q || !cs || !dB || !dC || !status)
        return SSD_ERR_NULL;
    const SsdShape& s = *shape;
    if (s.dstate != 64) return SSD_ERR_UNSUPPORTED;
    CUtensorMap map_x, map_b, map_c, map_dout, map_s, map_du;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_b, bm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_c, cm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dout, dout, tokens, s.nheads, s.headdim, kTile);
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_s, states_start, state_rows, s.dstate, 64);
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_du, dstates, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    const size_t smem = BwdDbcSmem::kTotal + 1024;
    cudaFuncSetAttribute(bwd_dbc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch * 2);
    bwd_dbc_kernel<<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        map_x, map_b, map_c, map_dout, map_s, map_du, q, cs, dB, dC, s, status);
    return launch_status();
}
