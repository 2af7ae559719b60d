// Per-tile state contraction  S[p,n] = sum_t (w_t * X[t,p]) * M[t,n]  for every
// head of one (batch, group, tile), on tcgen05 with split-bf16 operands.
//
//   mode 0 (forward):  X = x,    M = B, w_t = q_t * exp(cs_last - cs_t)  -> chunk state U_k
//   mode 1 (backward): X = dout, M = C, w_t = exp(cs_t)                   -> local dS_k
//
// Two heads of the group are stacked along the MMA's M dimension (2 x P = 128),
// so one instruction group yields both heads' [P,N] blocks; M (B or C) is
// shared by all heads of the group and is converted once per CTA.  Both
// operands are MN-major: the contraction index t runs along the rows of the
// token-major tiles exactly as they arrive from global memory.
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

template <int N>
struct ChunkStateSmem {
    static constexpr uint32_t kXTile = kTile * 128 * 2;       // 128 rows x 2 column blocks (two heads), one of hi/lo
    static constexpr uint32_t kMTile = kTile * 128 * (N / 64);  // 128 rows x N columns, one of hi/lo
    static constexpr uint32_t kXHi = 0;
    static constexpr uint32_t kXLo = kXHi + kXTile;
    static constexpr uint32_t kMHi = kXLo + kXTile;
    static constexpr uint32_t kMLo = kMHi + kMTile;
    static constexpr uint32_t kStage = kMLo + kMTile;         // 4 slabs
    static constexpr uint32_t kScale = kStage + 4 * kSlabBytes;  // float[2][128]
    static constexpr uint32_t kBars = kScale + 2 * kTile * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};

template <int N>
__global__ void __launch_bounds__(kThreads, 1)
chunk_state_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_m,
                   const __grid_constant__ CUtensorMap map_st, const float* __restrict__ q,
                   const float* __restrict__ cs, SsdShape s, int mode, int* status) {
    using L = ChunkStateSmem<N>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* scale = reinterpret_cast<float*>(smem + L::kScale);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);  // [0..3] staging, [4] mma
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;

    if (*reinterpret_cast<volatile int*>(status) != 0) return;  // an earlier CTA gave up: do not pile on

    StageRing<4> ring;
    ring.init(smem + L::kStage, bars, tid);
    if (tid == 0) {
        mbar_init(&bars[4], 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, N);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    // ---- group operand M (B or C): N/32 slabs through the ring
    constexpr int kMSlabs = N / 32;
    if (tid == 0) {
        for (int i = 0; i < kMSlabs && i < 4; ++i) ring.issue3d(i, &map_m, 32 * i, g, tok0, kTile);
    }
    for (int i = 0; i < kMSlabs; ++i) {
        ok = ring.wait(i, status) && ok;
        convert_slab(ring.slab(i), smem + L::kMHi, smem + L::kMLo, kTile, 32 * i, nullptr, tid, kThreads);
    }
    cta_sync();

    const int npairs = (heads_per_group + 1) / 2;
    auto issue_pair = [&](int pair) {
        const int h0 = g * heads_per_group + 2 * pair;
        const int nh = (2 * pair + 1 < heads_per_group) ? 2 : 1;
        for (int i = 0; i < 2 * nh; ++i) ring.issue3d(i, &map_x, 32 * (i & 1), h0 + (i >> 1), tok0, kTile);
    };
    if (tid == 0) issue_pair(0);

    uint32_t mma_parity = 0;
    const uint32_t idesc = make_idesc_bf16(128, N, true, true);
    constexpr int kIoThread = 256;  // issues the state stores
    // per-row weights: raw (q, cs, cs_last) of a pair are fetched one pair ahead into registers
    const int w_hh = tid >> 7, w_t = tid & 127;
    float w_q = 0.f, w_cs = 0.f, w_last = 0.f;
    auto fetch_rows = [&](int pair) {
        const int nh = (2 * pair + 1 < heads_per_group) ? 2 : 1;
        if (w_hh < nh) {
            const size_t row = (static_cast<size_t>(b) * s.nheads + g * heads_per_group + 2 * pair + w_hh) * s.seqlen +
                               k * kTile;
            w_cs = cs[row + w_t];
            w_last = cs[row + kTile - 1];
            w_q = q[row + w_t];
        }
    };
    auto publish_rows = [&]() {
        if (w_hh < 2) scale[w_hh * kTile + w_t] = mode == 0 ? w_q * expf(w_last - w_cs) : expf(w_cs);
    };
    fetch_rows(0);
    publish_rows();
    for (int pair = 0; pair < npairs; ++pair) {
        const int h0 = g * heads_per_group + 2 * pair;
        const int nh = (2 * pair + 1 < heads_per_group) ? 2 : 1;
        if (pair + 1 < npairs) fetch_rows(pair + 1);
        if (tid == kIoThread) tma_store_wait_read();  // the previous pair's states have left the X tile memory
        cta_sync();
        for (int i = 0; i < 2 * nh; ++i) {
            ok = ring.wait(i, status) && ok;
            convert_slab(ring.slab(i), smem + L::kXHi, smem + L::kXLo, kTile, 64 * (i >> 1) + 32 * (i & 1),
                         scale + (i >> 1) * kTile, tid, kThreads);
        }
        fence_proxy_async_smem();
        cta_sync();
        if (tid == 0) {
            if (pair + 1 < npairs) issue_pair(pair + 1);  // staging is free again: prefetch under the MMAs
            tc_fence_after_sync();
            const Operand a{smem_u32(smem + L::kXHi), smem_u32(smem + L::kXLo), kTile, true};
            const Operand m{smem_u32(smem + L::kMHi), smem_u32(smem + L::kMLo), kTile, true};
            issue_gemm_split<kTile / 16>(tmem, a, 0, m, 0, idesc, false);
            umma_commit(&bars[4]);
        }
        ok = mbar_wait(&bars[4], mma_parity, status, kStatusMmaTimeout) && ok;
        mma_parity ^= 1;
        tc_fence_after_sync();

        // epilogue: TMEM row = hh * 64 + p.  The X tile is dead now; the fp32 states are staged there as
        // swizzled [64 rows x 32 floats] slabs (index hh * N/32 + c) and written out by TMA in full lines.
        constexpr uint32_t kOutSlab = 64 * 128;
        {
            const int row = (warp & 3) * 32 + lane;
            const int hh = row >> 6, p = row & 63;
            constexpr int kColsPerWarp = N / 4;
            const int col0 = (warp >> 2) * kColsPerWarp;
            float v[kColsPerWarp];
            if constexpr (kColsPerWarp == 32) {
                tmem_ld32(tmem_addr(tmem, warp, col0), v);
            } else {
                tmem_ld16(tmem_addr(tmem, warp, col0), v);
            }
            tmem_ld_wait();
            uint8_t* slab = smem + L::kXHi + (hh * (N / 32) + col0 / 32) * kOutSlab;
#pragma unroll
            for (int i = 0; i < kColsPerWarp; i += 4)
                *reinterpret_cast<float4*>(slab + swz(p, ((col0 & 31) + i) >> 2)) =
                    make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();  // accumulator may be reused; staged states complete
        if (tid == kIoThread && ok) {
            for (int hh = 0; hh < nh; ++hh) {
                const int row0 = static_cast<int>(((static_cast<size_t>(b) * s.nheads + h0 + hh) * nchunks + k) * 64);
                for (int c = 0; c < N / 32; ++c)
                    tma_store_2d(&map_st, smem + L::kXHi + (hh * (N / 32) + c) * kOutSlab, 32 * c, row0);
            }
            tma_store_commit();
        }
        publish_rows();  // next pair's weights (this pair's conversions are long done)
    }
    if (tid == kIoThread) tma_store_wait_all();
    if (warp == 0) tmem_dealloc(tmem, N);
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
    const size_t smem = ChunkStateSmem<N>::kTotal + 1024;
    cudaFuncSetAttribute(chunk_state_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
    chunk_state_kernel<N><<<grid, kThreads, smem, stream>>>(map_x, map_m, map_st, q, cs, s, mode, status);
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
