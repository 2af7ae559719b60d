// Backward kernel for dx and the whole dt stage.  One CTA per (batch, group,
// tile of 128 tokens), heads of the group in sequence:
//
//   CB       = C * B^T                                        once per group   (tcgen05)
//   W_h      = tril(CB .* exp(cs_i - cs_j))                    TMEM -> split bf16 tile
//   D1[j,p]  = sum_i W_h[i,j] * dout[i,p]                      (A = W read MN-major)
//   D2[t,p]  = sum_n B[t,n]  * dU_h[p,n]                       dU = d loss / d (state after this tile)
//   dxdt     = D1 + exp(cs_last - cs_t) .* D2 ;  dx = q_t .* dxdt
//
// and, per row t, the gradient with respect to the cumulative decay cs_t:
//
//   g_cs[t] = sum_p dout*out  -  q_t * sum_p x*D1  -  q_t * decay_t * sum_p x*D2
//   g_cs[T-1] += sum_t q_t * decay_t * sum_p x*D2  +  g_last            (g_last from the state scan)
//
// (the first term equals rowsum(dW.*W) plus the state-to-output term because
// out = W*xdt + exp(cs)*C*S; the second is colsum(dW.*W); the third is the
// chunk-state weight).  A reverse in-tile cumulative sum of g_cs gives gw_t,
// then  ddt_t = (sum_p dxdt*x + A_h*gw_t) * softplus'(dt_t)  and the partial
// dA = sum_t gw_t*q_t.  All reductions are fixed-order.
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

// dstate N = 64 only
struct BwdDxSmem {
    static constexpr int N = 64;
    static constexpr uint32_t kCTile = kTile * 128;      // [128 x 64] one of hi/lo
    static constexpr uint32_t kWTile = kTile * 128 * 2;  // [128 x 128]
    static constexpr uint32_t kGTile = kTile * 128;      // dout [128 x 64]
    static constexpr uint32_t kUTile = 64 * 128;         // dU [64 x 64]
    static constexpr uint32_t kCHi = 0;                  // C (hi, lo); afterwards the fp32 x slabs live here
    static constexpr uint32_t kCLo = kCHi + kCTile;
    static constexpr uint32_t kXStage = kCHi;
    static constexpr uint32_t kBHi = kCLo + kCTile;
    static constexpr uint32_t kBLo = kBHi + kCTile;
    static constexpr uint32_t kWHi = kBLo + kCTile;
    static constexpr uint32_t kWLo = kWHi + kWTile;
    static constexpr uint32_t kGHi = kWLo + kWTile;
    static constexpr uint32_t kGLo = kGHi + kGTile;
    static constexpr uint32_t kUHi = kGLo + kGTile;
    static constexpr uint32_t kULo = kUHi + kUTile;
    static constexpr uint32_t kStage = kULo + kUTile;           // 2 slabs
    static constexpr uint32_t kRows = kStage + 2 * kSlabBytes;  // float arrays, see below
    static constexpr uint32_t kRowFloats = 17 * kTile;
    static constexpr uint32_t kBars = kRows + kRowFloats * 4;
    static constexpr uint32_t kTotal = kBars + 64;
};

__global__ void __launch_bounds__(kThreads, 1)
bwd_dx_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
              const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_dout,
              const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_du,
              const __grid_constant__ CUtensorMap map_dx, const float* __restrict__ q, const float* __restrict__ cs, const float* __restrict__ dt,
              const float* __restrict__ A, const float* __restrict__ g_last,
              float* __restrict__ ddt_t, double* __restrict__ dA_part, SsdShape s, int* status) {
    using L = BwdDxSmem;
    constexpr int N = L::N;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    float* rows = reinterpret_cast<float*>(smem + L::kRows);
    float* cs_s = rows;                  // [128]
    float* q_s = rows + kTile;           // [128]
    float* go_p = rows + 2 * kTile;      // [4][128] partial sum_p dout*out
    float* pa_p = rows + 6 * kTile;      // [4][128] partial sum_p x*D1
    float* pb_p = rows + 10 * kTile;     // [4][128] partial sum_p x*D2
    double* red_d = reinterpret_cast<double*>(rows + 14 * kTile);  // [160] scratch of the dt stage
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);  // [0,1] ring, [2] mma, [3] x slabs
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int heads_per_group = s.nheads / s.ngroups;
    const int nchunks = s.seqlen / kTile;
    const int tok0 = b * s.seqlen + k * kTile;
    const bool softplus = (s.flags & SSD_FLAG_DT_SOFTPLUS) != 0;

    if (*reinterpret_cast<volatile int*>(status) != 0) return;

    StageRing<2> ring;
    ring.init(smem + L::kStage, bars, tid);
    if (tid == 0) {
        mbar_init(&bars[2], 1);
        mbar_init(&bars[3], 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tm_cb = tmem, tm_d1 = tmem + 128, tm_d2 = tmem + 192;
    bool ok = true;
    uint32_t mma_parity = 0, x_parity = 0;

    // ---- group tiles C and B, CB = C * B^T
    {
        auto issue = [&](int i, int slot) { ring.issue3d(slot, i < 2 ? &map_c : &map_b, 32 * (i & 1), g, tok0, kTile); };
        auto conv = [&](int i, const uint8_t* slab) {
            convert_slab(slab, smem + (i < 2 ? L::kCHi : L::kBHi), smem + (i < 2 ? L::kCLo : L::kBLo), kTile,
                         32 * (i & 1), nullptr, tid, kThreads);
        };
        if (tid == 0) {
            issue(0, 0);
            issue(1, 1);
        }
        ok = run_loads<2>(ring, 4, issue, conv, tid, status) && ok;
        fence_proxy_async_smem();
        cta_sync();
        if (tid == 0) {
            tc_fence_after_sync();
            const Operand c{smem_u32(smem + L::kCHi), smem_u32(smem + L::kCLo), kTile, false};
            const Operand bm{smem_u32(smem + L::kBHi), smem_u32(smem + L::kBLo), kTile, false};
            issue_gemm_split<N / 16>(tm_cb, c, 0, bm, 0, make_idesc_bf16(128, 128, false, false), false);
            umma_commit(&bars[2]);
        }
        ok = mbar_wait(&bars[2], mma_parity, status, kStatusMmaTimeout) && ok;  // C tile is dead from here on
        mma_parity ^= 1;
        tc_fence_after_sync();
    }

    // Loads of the first head; every later head's loads are issued as soon as their buffers free up.
    constexpr int kIoThread = 256;  // issues the x loads and the dx stores (not one of the dt-stage threads)
    auto issue_x = [&](int h) {
        mbar_arrive_expect_tx(&bars[3], 2 * kSlabBytes);
        tma_load_3d(smem + L::kXStage, &map_x, &bars[3], 0, h, tok0);
        tma_load_3d(smem + L::kXStage + kSlabBytes, &map_x, &bars[3], 32, h, tok0);
    };
    auto issue_first_pair = [&](int h) {
        ring.issue3d(0, &map_dout, 0, h, tok0, kTile);
        ring.issue3d(1, &map_out, 0, h, tok0, kTile);
    };
    if (tid == kIoThread) issue_x(g * heads_per_group);  // fp32 x slabs live in the former C tile
    if (tid == 0) issue_first_pair(g * heads_per_group);
    if (tid < kTile) {
        const size_t o = (static_cast<size_t>(b) * s.nheads + g * heads_per_group) * s.seqlen + k * kTile + tid;
        cs_s[tid] = cs[o];
        q_s[tid] = q[o];
    }
    for (int hi = 0; hi < heads_per_group; ++hi) {
        const int h = g * heads_per_group + hi;
        const size_t bh = static_cast<size_t>(b) * s.nheads + h;
        const int srow = static_cast<int>((bh * nchunks + k) * 64);
        float cs_next = 0.f, q_next = 0.f;  // next head's rows, fetched one head ahead
        if (tid < kTile && hi + 1 < heads_per_group) {
            cs_next = cs[(bh + 1) * s.seqlen + k * kTile + tid];
            q_next = q[(bh + 1) * s.seqlen + k * kTile + tid];
        }
        cta_sync();

        // ---- W tile from CB
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

        // ---- dout tile + row sums of dout*out, two column halves
        float go = 0.f;
        const int r = tid & 127, jh = tid >> 7;  // row and 8-float group (0..3) of each slab
        for (int c = 0; c < 2; ++c) {
            ok = ring.wait(0, status) && ok;
            ok = ring.wait(1, status) && ok;
            const uint8_t* sg = ring.slab(0);
            const uint8_t* so = ring.slab(1);
            {
                const int j = jh;
                const float4 a0 = *reinterpret_cast<const float4*>(sg + swz(r, 2 * j));
                const float4 a1 = *reinterpret_cast<const float4*>(sg + swz(r, 2 * j + 1));
                const float4 o0 = *reinterpret_cast<const float4*>(so + swz(r, 2 * j));
                const float4 o1 = *reinterpret_cast<const float4*>(so + swz(r, 2 * j + 1));
                const float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                go += a0.x * o0.x + a0.y * o0.y + a0.z * o0.z + a0.w * o0.w;
                go += a1.x * o1.x + a1.y * o1.y + a1.z * o1.z + a1.w * o1.w;
                store_split8(smem + L::kGHi, smem + L::kGLo, kTile, r, 32 * c + 8 * j, v);
            }
            cta_sync();
            if (tid == 0) {
                if (c == 0) {
                    ring.issue3d(0, &map_dout, 32, h, tok0, kTile);
                    ring.issue3d(1, &map_out, 32, h, tok0, kTile);
                } else {
                    ring.issue2d(0, &map_du, 0, srow, 64);
                    ring.issue2d(1, &map_du, 32, srow, 64);
                }
            }
        }
        go_p[jh * kTile + r] = go;
        // ---- dU tile
        for (int c = 0; c < 2; ++c) {
            ok = ring.wait(c, status) && ok;
            convert_slab(ring.slab(c), smem + L::kUHi, smem + L::kULo, 64, 32 * c, nullptr, tid, kThreads);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid == 0) {
            if (hi + 1 < heads_per_group) issue_first_pair(h + 1);  // both ring slots are free again
            tc_fence_after_sync();
            const Operand w{smem_u32(smem + L::kWHi), smem_u32(smem + L::kWLo), kTile, true};
            const Operand gy{smem_u32(smem + L::kGHi), smem_u32(smem + L::kGLo), kTile, true};
            const Operand bm{smem_u32(smem + L::kBHi), smem_u32(smem + L::kBLo), kTile, false};
            const Operand du{smem_u32(smem + L::kUHi), smem_u32(smem + L::kULo), 64, false};
            issue_gemm_split<kTile / 16>(tm_d1, w, 0, gy, 0, make_idesc_bf16(128, 64, true, true), false);
            issue_gemm_split<N / 16>(tm_d2, bm, 0, du, 0, make_idesc_bf16(128, 64, false, false), false);
            umma_commit(&bars[2]);
        }
        ok = mbar_wait(&bars[3], x_parity, status, kStatusTmaTimeout) && ok;
        x_parity ^= 1;
        ok = mbar_wait(&bars[2], mma_parity, status, kStatusMmaTimeout) && ok;
        mma_parity ^= 1;
        tc_fence_after_sync();

        // ---- epilogue part 1: dx and the per-row dot products with x
        const float cs_last = cs_s[kTile - 1];
        {
            const int t = (warp & 3) * 32 + lane;
            const int cg = warp >> 2;  // 16-column group of the [T,P] accumulators
            const float decay = expf(cs_last - cs_s[t]);
            const float qt = q_s[t];
            float d1[16], d2[16];
            tmem_ld16(tmem_addr(tm_d1, warp, cg * 16), d1);
            tmem_ld16(tmem_addr(tm_d2, warp, cg * 16), d2);
            tmem_ld_wait();
            // dx overwrites x in place (same thread, same 16 floats); TMA then stores the two slabs
            uint8_t* xs = smem + L::kXStage + (cg >> 1) * kSlabBytes;  // slab of columns 0..31 or 32..63
            float pa = 0.f, pb = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                float4* px = reinterpret_cast<float4*>(xs + swz(t, (cg & 1) * 4 + c4));
                const float4 xv = *px;
                const float* a = d1 + 4 * c4;
                const float* bb = d2 + 4 * c4;
                pa += xv.x * a[0] + xv.y * a[1] + xv.z * a[2] + xv.w * a[3];
                pb += xv.x * bb[0] + xv.y * bb[1] + xv.z * bb[2] + xv.w * bb[3];
                *px = make_float4(qt * (a[0] + decay * bb[0]), qt * (a[1] + decay * bb[1]),
                                  qt * (a[2] + decay * bb[2]), qt * (a[3] + decay * bb[3]));
            }
            pa_p[cg * kTile + t] = pa;
            pb_p[cg * kTile + t] = pb;
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        cta_sync();
        if (tid == kIoThread) {
            if (ok) {
                tma_store_3d(&map_dx, smem + L::kXStage, 0, h, tok0);
                tma_store_3d(&map_dx, smem + L::kXStage + kSlabBytes, 32, h, tok0);
                tma_store_commit();
            }
            tma_store_wait_read();  // the slabs may be overwritten once the store has read them
            if (hi + 1 < heads_per_group) issue_x(h + 1);
        }

        // ---- epilogue part 2 (threads 0..127, one per row): dt stage, accumulated in double so that
        // the long sums feeding dA do not add rounding error of their own
        float a_t = 0.f, b_t = 0.f, qt = 0.f;
        double gcs = 0.0;
        if (tid < kTile) {
            const int t = tid;
            qt = q_s[t];
            a_t = (pa_p[t] + pa_p[kTile + t]) + (pa_p[2 * kTile + t] + pa_p[3 * kTile + t]);
            b_t = expf(cs_last - cs_s[t]) *
                  ((pb_p[t] + pb_p[kTile + t]) + (pb_p[2 * kTile + t] + pb_p[3 * kTile + t]));
            gcs = ((static_cast<double>(go_p[t]) + go_p[kTile + t]) + (static_cast<double>(go_p[2 * kTile + t]) + go_p[3 * kTile + t])) -
                  static_cast<double>(qt) * (static_cast<double>(a_t) + b_t);
            // sum over rows of q_t * b_t (fixed tree), added to the last row together with g_last
            double v = static_cast<double>(qt) * b_t;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0) red_d[warp] = v;
        }
        cta_sync();
        if (tid < kTile) {
            if (tid == kTile - 1) gcs += (red_d[0] + red_d[1]) + (red_d[2] + red_d[3]) + g_last[bh * nchunks + k];
            // reverse inclusive scan inside the warp ...
            double sfx = gcs;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const double dn = __shfl_down_sync(0xffffffffu, sfx, d);
                if (lane + d < 32) sfx += dn;
            }
            if (lane == 0) red_d[8 + warp] = sfx;  // warp total
            red_d[32 + tid] = sfx;
        }
        cta_sync();
        if (tid < kTile) {
            const int t = tid;
            double gw = red_d[32 + t];
            for (int w = warp + 1; w < 4; ++w) gw += red_d[8 + w];  // ... plus the totals of the later warps
            const float dtr = dt[(static_cast<size_t>(tok0) + t) * s.nheads + h];
            const double dq = static_cast<double>(a_t) + b_t + static_cast<double>(A[h]) * gw;
            const float deriv = softplus ? (dtr > 20.f ? 1.f : sigmoid_f(dtr)) : (dtr >= 0.f ? 1.f : 0.f);
            if (ok) ddt_t[bh * s.seqlen + k * kTile + t] = static_cast<float>(dq * deriv);
            double v = gw * qt;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0) red_d[16 + warp] = v;
        }
        cta_sync();
        if (tid == 0 && ok) dA_part[bh * nchunks + k] = (red_d[16] + red_d[17]) + (red_d[18] + red_d[19]);
        if (tid < kTile && hi + 1 < heads_per_group) {  // nobody reads this head's rows any more
            cs_s[tid] = cs_next;
            q_s[tid] = q_next;
        }
    }
    if (tid == kIoThread) tma_store_wait_all();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_chunk_dx_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                                const float* dout, const float* out, const float* dstates, const float* q,
                                const float* cs, const float* dt, const float* A, const float* g_last, float* dx,
                                float* ddt_t, double* dA_partial, int* status, ssd_stream_t stream) {
    using namespace ssd;
    const int rc0 = ssd_check_shape(shape);
    if (rc0 != SSD_OK) return rc0;
    if (!x || !bm || !cm || !dout || !out || !dstates || !q || !cs || !dt || !A || !g_last || !dx || !ddt_t ||
        !dA_partial || !status)
        return SSD_ERR_NULL;
    const SsdShape& s = *shape;
    if (s.dstate != 64) return SSD_ERR_UNSUPPORTED;
    CUtensorMap map_x, map_b, map_c, map_dout, map_out, map_du, map_dx;
    const uint64_t tokens = static_cast<uint64_t>(s.batch) * s.seqlen;
    int rc = make_tmap_f32_tokens(&map_x, x, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_b, bm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_c, cm, tokens, s.ngroups, s.dstate, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dout, dout, tokens, s.nheads, s.headdim, kTile);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_out, out, tokens, s.nheads, s.headdim, kTile);
    const uint64_t state_rows = static_cast<uint64_t>(s.batch) * s.nheads * (s.seqlen / kTile) * s.headdim;
    if (rc == SSD_OK) rc = make_tmap_f32_2d(&map_du, dstates, state_rows, s.dstate, 64);
    if (rc == SSD_OK) rc = make_tmap_f32_tokens(&map_dx, dx, tokens, s.nheads, s.headdim, kTile);
    if (rc != SSD_OK) return rc;
    const size_t smem = BwdDxSmem::kTotal + 1024;
    cudaFuncSetAttribute(bwd_dx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const dim3 grid(s.seqlen / kTile, s.ngroups, s.batch);
    bwd_dx_kernel<<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        map_x, map_b, map_c, map_dout, map_out, map_du, map_dx, q, cs, dt, A, g_last, ddt_t, dA_partial, s, status);
    return launch_status();
}
