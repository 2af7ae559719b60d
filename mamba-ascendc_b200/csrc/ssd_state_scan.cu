// Per-tile state contraction FUSED with the inter-tile recurrence: one CTA owns one (batch, group), walks
// its 128-token tiles in order and keeps the running state of every head of the group on chip (fp32, in
// tensor memory), so the per-tile contributions never travel through global memory and the separate
// state-passing launch disappears.
//
//   mode 0 (forward):  U_k[p,n] = sum_t q_t exp(cs_last - cs_t) x[t,p] B[t,n]      tcgen05, as ssd_chunk_state
//                      tiles ascending:  store S_k ;  S <- exp(cs_last,k) S + U_k  ;  final = S after the last tile
//   mode 1 (backward): dS_k[p,n] = sum_t exp(cs_t) dout[t,p] C[t,n]                tcgen05
//                      tiles descending: store dU_k = g ;  g <- dS_k + exp(cs_last,k) g  ;
//                      d_initial = g after the first tile
//                      (the third output of the reference's reverse scan, d(cs_last) = exp(cs_last,k) sum(dU_k .* S_k),
//                      is formed by the dB/dC kernel, through which both tensors pass anyway)
//
// The reference keeps the running state resident while it projects in the same way
// (mamba_ascendc_ops/mamba2_ssd_chunk_mix/op_kernel/mamba2_ssd_state_epilogue.cpp:208 UpdateState, driven
// from :1179-1186); the reverse recurrence is that of
// mamba_ascendc/csrc/ops/mamba2_ssd_state_passing_bwd/design.md:49-58.
//
// The product of a step is the one of ssd_chunk_state.cu (two heads stacked along M, both operands MN-major,
// tiles loaded by TMA into operand-tile memory and split in place, 8 compute warps + the issuing warp group,
// two CTAs per SM).  The epilogue reads the product and the running state from tensor memory, stages the
// state that leaves (S_k or dU_k) in the dead pair buffer for a TMA store, and writes the updated state
// back to tensor memory with round-to-nearest fp32 arithmetic (the tensor core's own accumulation truncates,
// which would add up over the tiles).  Parallelism is batch x groups CTAs, so the host uses this kernel
// only when that fills the GPU; the tile-parallel pair ssd_chunk_state + ssd_state_passing_* stays for the rest.
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

constexpr int kSsWarps = 8;  // compute warps
constexpr int kSsThreads = kSsWarps * 32;
constexpr int kSsLaunch = kSsThreads + 128;  // plus the issuing warp group
constexpr uint32_t kSsIssuerRegs = 32;       // 80 at launch (2 x 384 threads per SM); the issuing group keeps 32 ...
constexpr uint32_t kSsComputeRegs = 104;     // ... and the two computing groups take 24 more each
constexpr int kSsMaxPairs = 3;               // running states of at most 3 head pairs: 64 + 3 * 64 = 256 columns

__device__ __forceinline__ void ss_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

struct StateScanSmem {
    static constexpr int N = 64;
    static constexpr uint32_t kXTile = kTile * 128 * 2;  // one head: [128 x 64] hi | lo
    static constexpr uint32_t kPair = 2 * kXTile;        // two heads
    static constexpr uint32_t kMTile = kTile * 128 * 2;  // [128 x 64] hi | lo
    static constexpr uint32_t kX = 0;                    // the pair buffer, later the staged states
    static constexpr uint32_t kM = kX + kPair;
    static constexpr uint32_t kScale = kM + kMTile;      // float[2 sets][2 heads][128] row weights
    static constexpr uint32_t kAlpha = kScale + 4 * kTile * 4;  // float[2 sets][2 heads] exp(cs_last)
    static constexpr uint32_t kBars = kAlpha + 16;
    static constexpr uint32_t kTotal = kBars + 64;
};
static_assert(2 * (StateScanSmem::kTotal + 1024) <= 233472, "two state-scan CTAs do not fit one SM");

template <int MODE>
__global__ void __launch_bounds__(kSsLaunch, 2)
chunk_state_scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_m,
                        const __grid_constant__ CUtensorMap map_st, const float* __restrict__ q,
                        const float* __restrict__ cs, const float* __restrict__ start, float* __restrict__ end,
                        SsdShape s, int* status) {
    using L = StateScanSmem;
    constexpr int N = L::N;
    extern __shared__ __align__(1024) uint8_t smem[];
    float* scale = reinterpret_cast<float*>(smem + L::kScale);
    float* alpha_s = reinterpret_cast<float*>(smem + L::kAlpha);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
    uint64_t* full_x = bars;       // pair buffer has landed
    uint64_t* full_m = bars + 1;   // group operand of the tile has landed
    uint64_t* bar_mma = bars + 2;  // product done
    uint64_t* bar_rdy = bars + 3;  // pair split (and accumulator free)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.x, b = blockIdx.y;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int h_first = g * heads_per_group;
    const int npairs = (heads_per_group + 1) / 2;
    const int nsteps = nchunks * npairs;  // step = (tile in walking order) * npairs + pair

    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need the declared alignment
        if (tid == 0) atomicCAS(status, 0, kStatusSmemAlign);
        return;
    }
    // An earlier kernel or CTA gave up on a bounded wait: leave without doing work.  Thread 0 alone reads the
    // status word and the whole CTA branches on its copy after the barrier below.
    if (tid == 0) {
        tmem_slot[1] = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(status));
        for (int i = 0; i < 3; ++i) mbar_init(&bars[i], 1);
        mbar_init(bar_rdy, kSsWarps);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);  // product [128 x 64] + up to three running pair states
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (tmem_slot[1] != 0) {
        if (warp == 0) tmem_dealloc(tmem, 256);
        return;
    }
    bool ok = true;
    constexpr uint32_t kHalf = kTile * 128;

    // ---- warp 8: issues every tensor-core instruction of the CTA
    if (warp >= kSsWarps) {
        reg_release<kSsIssuerRegs>();
        if (warp == kSsWarps && lane == 0) {
            const uint32_t sm = smem_u32(smem + L::kM), sx = smem_u32(smem + L::kX);
            const Operand m{sm, sm + kHalf, kTile, true, 2 * kHalf};
            const Operand a{sx, sx + kHalf, kTile, true, 2 * kHalf};  // column blocks = the two heads
            const uint32_t idesc = make_idesc_bf16(128, N, true, true);
            uint32_t pr = 0;
            for (int step = 0; step < nsteps; ++step) {
                mbar_wait(bar_rdy, pr, status, kStatusMmaTimeout | wait_site(2, 1));
                pr ^= 1;
                tc_fence_after_sync();
                issue_gemm_split<kTile / 16>(tmem, a, 0, m, 0, idesc, false);
                umma_commit(bar_mma);
            }
        }
        return;
    }
    reg_acquire<kSsComputeRegs>();

    uint8_t* buf = smem + L::kX;
    auto tile_of = [&](int step) { return MODE == 0 ? step / npairs : nchunks - 1 - step / npairs; };
    auto heads_in = [&](int pair) { return (2 * pair + 1 < heads_per_group) ? 2 : 1; };
    auto load_pair = [&](int step) {
        const int pair = step % npairs, nh = heads_in(pair);
        const int tok0 = b * s.seqlen + tile_of(step) * kTile;
        mbar_arrive_expect_tx(full_x, nh * L::kXTile);
        for (int hh = 0; hh < nh; ++hh)
            tma_tile_3d(buf + hh * L::kXTile, kTile, &map_x, full_x, 0, h_first + 2 * pair + hh, tok0, false);
    };
    auto load_m = [&](int step) {
        tma_tile_3d(smem + L::kM, kTile, &map_m, full_m, 0, g, b * s.seqlen + tile_of(step) * kTile);
    };
    if (tid == 0) {
        load_m(0);
        load_pair(0);
    }

    // per-row weights: one thread per (head of the pair, row); raw (q, cs, cs_last) are fetched one step
    // ahead into registers and published into the set of that step's parity
    const int w_hh = tid >> 7, w_t = tid & 127;
    float w_q = 0.f, w_cs = 0.f, w_last = 0.f;
    auto fetch_rows = [&](int step) {
        const int pair = step % npairs;
        if (w_hh < heads_in(pair)) {
            const size_t row =
                (static_cast<size_t>(b) * s.nheads + h_first + 2 * pair + w_hh) * s.seqlen + tile_of(step) * kTile;
            w_cs = cs[row + w_t];
            w_last = cs[row + kTile - 1];
            w_q = q[row + w_t];
        }
    };
    auto publish_rows = [&](int step) {
        scale[((step & 1) * 2 + w_hh) * kTile + w_t] = MODE == 0 ? w_q * expf(w_last - w_cs) : expf(w_cs);
        if (w_t == 0) alpha_s[(step & 1) * 2 + w_hh] = expf(w_last);
    };
    fetch_rows(0);
    publish_rows(0);
    if (nsteps > 1) fetch_rows(1);

    // ---- the running states start from `start` (initial state / gradient of the final state) or zero.
    // This thread owns row (hh, p) of a pair's [2 x 64, 64] state and 32 of its columns.
    const int row = (warp & 3) * 32 + lane;
    const int e_hh = row >> 6, e_p = row & 63;
    const int e_col = (warp >> 2) * 32;
    auto tm_state = [&](int pair) { return tmem + 64u + 64u * static_cast<uint32_t>(pair); };
    auto state_elem = [&](int pair) {  // offset of this thread's 32 values inside a [B,H,P,N] tensor
        return ((static_cast<size_t>(b) * s.nheads + h_first + 2 * pair + e_hh) * 64 + e_p) * N + e_col;
    };
    for (int pair = 0; pair < npairs; ++pair) {
        float v[32];
        if (start != nullptr && e_hh < heads_in(pair)) {
            const float4* src = reinterpret_cast<const float4*>(start + state_elem(pair));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 f = src[i];
                v[4 * i] = f.x;
                v[4 * i + 1] = f.y;
                v[4 * i + 2] = f.z;
                v[4 * i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        tmem_st16(tmem_addr(tm_state(pair), warp, e_col), reinterpret_cast<const uint32_t*>(v));
        tmem_st16(tmem_addr(tm_state(pair), warp, e_col + 16), reinterpret_cast<const uint32_t*>(v + 16));
    }
    tmem_st_wait();
    ss_sync();  // weights of the first step are visible

    uint32_t px = 0, pm = 0, pmm = 0;
    constexpr int kIoThread = 128;  // issues the state stores and the next loads
    constexpr uint32_t kOutSlab = 64 * 128;
    for (int step = 0; step < nsteps; ++step) {
        const int pair = step % npairs, k = tile_of(step);
        const int h0 = h_first + 2 * pair;
        const int nh = heads_in(pair);
        if (pair == 0) {  // a new tile: its B (or C) has landed; split it once for all pairs
            ok = mbar_wait(full_m, pm, status, kStatusTmaTimeout | wait_site(2, 2)) && ok;
            pm ^= 1;
            split_tile_inplace(smem + L::kM, kTile, nullptr, warp, lane);
            split_tile_inplace(smem + L::kM, kTile, nullptr, warp + kSsWarps, lane);
        }
        ok = mbar_wait(full_x, px, status, kStatusTmaTimeout | wait_site(2, 3)) && ok;
        px ^= 1;
        {
            const float* sc = scale + (step & 1) * 2 * kTile;
            if (nh == 2) {
                split_two_tiles_inplace(buf, sc, buf + L::kXTile, sc + kTile, kTile, warp, lane);
                split_two_tiles_inplace(buf, sc, buf + L::kXTile, sc + kTile, kTile, warp + kSsWarps, lane);
            } else {
                split_tile_inplace(buf, kTile, sc, warp, lane);
                split_tile_inplace(buf, kTile, sc, warp + kSsWarps, lane);
            }
        }
        signal_issuer(bar_rdy, lane);
        if (step + 1 < nsteps) publish_rows(step + 1);  // other set
        if (step + 2 < nsteps) fetch_rows(step + 2);
        ok = mbar_wait(bar_mma, pmm, status, kStatusMmaTimeout | wait_site(2, 4)) && ok;
        pmm ^= 1;
        tc_fence_after_sync();

        // ---- epilogue: the state that leaves goes to the (dead) pair buffer as swizzled [64 rows x 32 floats]
        // slabs (index hh * 2 + column half), the updated state back to tensor memory
        {
            const float alpha = alpha_s[(step & 1) * 2 + e_hh];
            uint8_t* slab = buf + (e_hh * 2 + (warp >> 2)) * kOutSlab;
#pragma unroll
            for (int c = 0; c < 2; ++c) {  // 16 columns at a time
                float u[16], st[16];
                tmem_ld16(tmem_addr(tmem, warp, e_col + 16 * c), u);
                tmem_ld16(tmem_addr(tm_state(pair), warp, e_col + 16 * c), st);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i += 4)
                    *reinterpret_cast<float4*>(slab + swz(e_p, 4 * c + (i >> 2))) =
                        make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
#pragma unroll
                for (int i = 0; i < 16; ++i) st[i] = fmaf(alpha, st[i], u[i]);
                tmem_st16(tmem_addr(tm_state(pair), warp, e_col + 16 * c), reinterpret_cast<const uint32_t*>(st));
            }
            tmem_st_wait();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        ss_sync();  // staged states complete; next step's weights visible; accumulator free
        if (tid == kIoThread) {
            if (ok) {
                for (int hh = 0; hh < nh; ++hh) {
                    const int row0 = static_cast<int>(((static_cast<size_t>(b) * s.nheads + h0 + hh) * nchunks + k) * 64);
                    for (int c = 0; c < 2; ++c) tma_store_2d(&map_st, buf + (hh * 2 + c) * kOutSlab, 32 * c, row0);
                }
                tma_store_commit();
            }
            tma_store_wait_read();  // then the buffer can take the next pair
            if (step + 1 < nsteps) {
                if ((step + 1) % npairs == 0) load_m(step + 1);  // every product of this tile is done
                load_pair(step + 1);
            }
        }
    }
    // ---- the state after the last tile walked: final state (forward) / gradient of the initial state (backward)
    if (end != nullptr && ok) {
        for (int pair = 0; pair < npairs; ++pair) {
            if (e_hh >= heads_in(pair)) continue;
            float v[32];
            tmem_ld32(tmem_addr(tm_state(pair), warp, e_col), v);
            tmem_ld_wait();
            float4* dst = reinterpret_cast<float4*>(end + state_elem(pair));
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
    }
    if (tid == kIoThread) tma_store_wait_all();
    tc_fence_before_sync();
    ss_sync();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int MODE>
int launch_state_scan(const SsdShape& s, const float* x, const float* m, const float* q, const float* cs,
                      const float* start, float* states, float* end, int* status, cudaStream_t stream) {
    CUtensorMap map_x, map_m, map_st;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc != SSD_OK) return rc;
    rc = make_tmap_f32_tokens(&map_m, m, tokens, s.ngroups, s.dstate, kTile);
    if (rc != SSD_OK) return rc;
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    rc = make_tmap_f32_2d(&map_st, states, state_rows, s.dstate, 64);
    if (rc != SSD_OK) return rc;
    const size_t smem = StateScanSmem::kTotal;
    static std::atomic<uint64_t> smem_set{0};
    rc = set_max_smem_once(reinterpret_cast<const void*>(chunk_state_scan_kernel<MODE>), smem, smem_set);
    if (rc != SSD_OK) return rc;
    const dim3 grid(s.ngroups, s.batch);
    chunk_state_scan_kernel<MODE><<<grid, kSsLaunch, smem, stream>>>(map_x, map_m, map_st, q, cs, start, end, s, status);
    return launch_status();
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_state_scan_supported(const SsdShape* shape) {
    if (ssd_check_shape(shape) != SSD_OK) return 0;
    const int heads_per_group = shape->nheads / shape->ngroups;
    return shape->dstate == 64 && (heads_per_group + 1) / 2 <= ssd::kSsMaxPairs ? 1 : 0;
}

extern "C" int ssd_chunk_state_scan(const SsdShape* shape, const float* x, const float* m, const float* q,
                                    const float* cs, const float* start, float* states, float* end, int mode,
                                    int* status, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!x || !m || !q || !cs || !states || !status) return SSD_ERR_NULL;
    if (mode != 0 && mode != 1) return SSD_ERR_UNSUPPORTED;
    if (!ssd_chunk_state_scan_supported(shape)) return SSD_ERR_UNSUPPORTED;
    for (const float* p : {start, static_cast<const float*>(end)})
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return SSD_ERR_ALIGN;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    return mode == 0 ? launch_state_scan<0>(*shape, x, m, q, cs, start, states, end, status, st)
                     : launch_state_scan<1>(*shape, x, m, q, cs, start, states, end, status, st);
}
