// Forward output kernel.  One CTA per (batch, group, tile of 128 tokens):
//
//   CB      = C * B^T                                   once per group        [T,T]   (tcgen05)
//   W_h     = tril(CB .* exp(cs_i - cs_j))              per head, TMEM -> registers -> split bf16 tile
//   out_h   = W_h * (q .* x_h)  +  exp(cs_t) .* (C * S_h^T)                   [T,P]   (two tcgen05 products)
//
// S_h is the state at the start of the tile (from the state-passing kernel).
// C, B, x and S arrive as fp32 TMA boxes and are split into bf16 hi/lo
// operand tiles in shared memory; W is built from the CB accumulator in TMEM.
// The B tile is dead once CB exists, so W reuses its shared memory.
#include "ssd_host.h"
#include "ssd_tile.cuh"

PROF_DECL(scan)

namespace ssd {

namespace {

template <int N>
struct ChunkScanSmem {
    static constexpr int kStages = N == 64 ? 4 : 2;
    static constexpr uint32_t kCTile = kTile * 128 * (N / 64);  // one of hi/lo
    static constexpr uint32_t kWTile = kTile * 128 * 2;         // [128 x 128], one of hi/lo
    static constexpr uint32_t kXTile = kTile * 128;             // [128 x 64]
    static constexpr uint32_t kSTile = 64 * 128 * (N / 64);     // [64 x N]
    static constexpr uint32_t kBW = 2 * (kCTile > kWTile ? kCTile : kWTile);
    static constexpr uint32_t kCHi = 0;
    static constexpr uint32_t kCLo = kCHi + kCTile;
    static constexpr uint32_t kBHi = kCLo + kCTile;  // B (hi, lo) first, later W (hi, lo)
    static constexpr uint32_t kBLo = kBHi + kCTile;
    static constexpr uint32_t kWHi = kBHi;
    static constexpr uint32_t kWLo = kWHi + kWTile;
    static constexpr uint32_t kXHi = kBHi + kBW;
    static constexpr uint32_t kXLo = kXHi + kXTile;
    static constexpr uint32_t kSHi = kXLo + kXTile;
    static constexpr uint32_t kSLo = kSHi + kSTile;
    static constexpr uint32_t kStage = kSLo + kSTile;
    static constexpr uint32_t kCs = kStage + kStages * kSlabBytes;  // float[128] cs, float[128] q
    static constexpr uint32_t kBars = kCs + 2 * kTile * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};

template <int N>
__global__ void __launch_bounds__(kThreads, 1)
chunk_scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_s,
                  const __grid_constant__ CUtensorMap map_out, const float* __restrict__ q,
                  const float* __restrict__ cs, SsdShape s, int* status) {
    using L = ChunkScanSmem<N>;
    constexpr int NS = L::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* rowbuf = reinterpret_cast<float*>(smem + L::kCs);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);  // [0..NS) staging, [NS] mma
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NS + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;

    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    PROF_BEGIN()

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
    const uint32_t tm_cb = tmem, tm_diag = tmem + 128, tm_off = tmem + 192;
    bool ok = true;
    uint32_t mma_parity = 0;

    // ---- group tiles C and B, then CB = C * B^T
    {
        constexpr int kSl = N / 32;  // slabs per tile
        auto issue = [&](int i, int slot) {
            ring.issue3d(slot, i < kSl ? &map_c : &map_b, 32 * (i % kSl), g, tok0, kTile);
        };
        auto conv = [&](int i, const uint8_t* slab) {
            convert_slab(slab, smem + (i < kSl ? L::kCHi : L::kBHi), smem + (i < kSl ? L::kCLo : L::kBLo), kTile,
                         32 * (i % kSl), nullptr, tid, kThreads);
        };
        if (tid == 0) {
            for (int i = 0; i < 2 * kSl && i < NS; ++i) issue(i, i);
        }
        ok = run_loads<NS>(ring, 2 * kSl, issue, conv, tid, status) && ok;
        fence_proxy_async_smem();
        cta_sync();
        if (tid == 0) {
            tc_fence_after_sync();
            const Operand c{smem_u32(smem + L::kCHi), smem_u32(smem + L::kCLo), kTile, false};
            const Operand bm{smem_u32(smem + L::kBHi), smem_u32(smem + L::kBLo), kTile, false};
            issue_gemm_split<N / 16>(tm_cb, c, 0, bm, 0, make_idesc_bf16(128, 128, false, false), false);
            umma_commit(&bars[NS]);
        }
    }

    // per-head loads: x (2 slabs of 128 rows) then S (N/32 slabs of 64 rows)
    constexpr int kHeadLoads = 2 + N / 32;
    auto issue_head = [&](int h, int i, int slot) {
        if (i < 2) {
            ring.issue3d(slot, &map_x, 32 * i, h, tok0, kTile);
        } else {
            ring.issue2d(slot, &map_s, 32 * (i - 2), ((b * s.nheads + h) * nchunks + k) * 64, 64);
        }
    };
    if (tid == 0) {
        for (int i = 0; i < kHeadLoads && i < NS; ++i) issue_head(g * heads_per_group, i, i);
    }
    ok = mbar_wait(&bars[NS], mma_parity, status, kStatusMmaTimeout) && ok;  // CB ready, B tile dead
    mma_parity ^= 1;
    tc_fence_after_sync();

    PROF_T(0)
    // (cs, q) rows of the first head; every later head's rows are fetched one head ahead into registers
    if (tid < kTile) {
        const size_t o = (static_cast<size_t>(b) * s.nheads + g * heads_per_group) * s.seqlen + k * kTile + tid;
        rowbuf[tid] = cs[o];
        rowbuf[kTile + tid] = q[o];
    }
    for (int hi = 0; hi < heads_per_group; ++hi) {
        const int h = g * heads_per_group + hi;
        float* cs_s = rowbuf;
        float* q_s = cs_s + kTile;
        float cs_next = 0.f, q_next = 0.f;
        if (tid < kTile && hi + 1 < heads_per_group) {
            const size_t o = (static_cast<size_t>(b) * s.nheads + h + 1) * s.seqlen + k * kTile + tid;
            cs_next = cs[o];
            q_next = q[o];
        }
        if (tid == 0) tma_store_wait_read();  // the previous head's output tile has left the x-tile memory
        cta_sync();
        PROF_T(1)

        // ---- W tile from CB (TMEM): row i per lane, warps w and w+4 split the columns
        {
            const int i = (warp & 3) * 32 + lane;
            const int row_max = (warp & 3) * 32 + 31;
            const float csi = cs_s[i];
            {
                const int j0 = (warp >> 2) * 32;  // one 32-column chunk per warp
                float v[32];
                if (j0 <= row_max) {
                    tmem_ld32(tmem_addr(tm_cb, warp, j0), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int j = j0 + jj;
                        const float e = __expf(j <= i ? csi - cs_s[j] : 0.f);
                        v[jj] = j <= i ? v[jj] * e : 0.f;
                    }
                } else {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) v[jj] = 0.f;
                }
#pragma unroll
                for (int jj = 0; jj < 32; jj += 8)
                    store_split8(smem + L::kWHi, smem + L::kWLo, kTile, i, j0 + jj, v + jj);
            }
        }

        PROF_T(2)
        // ---- x -> q .* x tile, S tile
        {
            auto issue = [&](int i, int slot) { issue_head(h, i, slot); };
            auto conv = [&](int i, const uint8_t* slab) {
                if (i < 2) {
                    convert_slab(slab, smem + L::kXHi, smem + L::kXLo, kTile, 32 * i, q_s, tid, kThreads);
                } else {
                    convert_slab(slab, smem + L::kSHi, smem + L::kSLo, 64, 32 * (i - 2), nullptr, tid, kThreads);
                }
            };
            ok = run_loads<NS>(ring, kHeadLoads, issue, conv, tid, status) && ok;
        }
        PROF_T(3)
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        PROF_T(4)
        if (tid == 0) {
            if (hi + 1 < heads_per_group) {
                for (int i = 0; i < kHeadLoads && i < NS; ++i) issue_head(h + 1, i, i);
            }
            tc_fence_after_sync();
            const Operand w{smem_u32(smem + L::kWHi), smem_u32(smem + L::kWLo), kTile, false};
            const Operand x{smem_u32(smem + L::kXHi), smem_u32(smem + L::kXLo), kTile, true};
            const Operand c{smem_u32(smem + L::kCHi), smem_u32(smem + L::kCLo), kTile, false};
            const Operand st{smem_u32(smem + L::kSHi), smem_u32(smem + L::kSLo), 64, false};
            issue_gemm_split<kTile / 16>(tm_diag, w, 0, x, 0, make_idesc_bf16(128, 64, false, true), false);
            issue_gemm_split<N / 16>(tm_off, c, 0, st, 0, make_idesc_bf16(128, 64, false, false), false);
            umma_commit(&bars[NS]);
        }
        ok = mbar_wait(&bars[NS], mma_parity, status, kStatusMmaTimeout) && ok;
        mma_parity ^= 1;
        tc_fence_after_sync();
        PROF_T(5)

        // ---- epilogue: out[t, p] = diag + exp(cs_t) * off
        {
            const int t = (warp & 3) * 32 + lane;
            const int cg = warp >> 2;  // 16-column group
            const float e = expf(cs_s[t]);
            float d[16], o[16];
            tmem_ld16(tmem_addr(tm_diag, warp, cg * 16), d);
            tmem_ld16(tmem_addr(tm_off, warp, cg * 16), o);
            tmem_ld_wait();
            // the x tile is dead once the MMAs are done: stage the fp32 output there (two swizzled
            // 128 x 32 slabs) and let TMA write it out in full lines
            uint8_t* slab = smem + L::kXHi + (cg >> 1) * kSlabBytes;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(slab + swz(t, (cg & 1) * 4 + (i >> 2))) =
                    make_float4(d[i] + e * o[i], d[i + 1] + e * o[i + 1], d[i + 2] + e * o[i + 2], d[i + 3] + e * o[i + 3]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid < kTile && hi + 1 < heads_per_group) {  // everyone is done with this head's rows
            rowbuf[tid] = cs_next;
            rowbuf[kTile + tid] = q_next;
        }
        if (tid == 0 && ok) {
            tma_store_3d(&map_out, smem + L::kXHi, 0, h, tok0);
            tma_store_3d(&map_out, smem + L::kXHi + kSlabBytes, 32, h, tok0);
            tma_store_commit();
        }
        PROF_T(6)
    }
    PROF_END(scan)
    if (tid == 0) tma_store_wait_all();
    if (warp == 0) tmem_dealloc(tmem, 256);
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
    cudaFuncSetAttribute(chunk_scan_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
    chunk_scan_kernel<N><<<grid, kThreads, smem, stream>>>(map_x, map_b, map_c, map_s, map_out, q, cs, s, status);
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
