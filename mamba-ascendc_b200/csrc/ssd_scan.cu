// Bandwidth-bound scan kernels of the SSD path (no tensor cores):
//   dt_cumsum_kernel        q = softplus(dt), cs = in-tile inclusive cumsum of A*q   (warp scan)
//   state_passing_fwd       S_{k+1} = exp(cs_last,k) * S_k + U_k, in place over the chunk states
//   state_passing_bwd       reverse recurrence, in place over the local dS; also d(cs_last)
//   dt_finalize_bwd         [B,H,L] -> [B,L,H] transpose of ddt and the fixed-order dA reduction
#include "ssd_host.h"
#include "ssd_tile.cuh"

namespace ssd {

namespace {

// ------------------------------------------------------------------ dt softplus + cumsum
// CTA = (tile k, block of 32 heads, batch b).  The [128 tokens x 32 heads]
// patch of dt is read with lanes along heads (contiguous in memory), turned in
// shared memory, and each warp scans four heads with lanes along tokens, four
// tokens per lane plus a shuffle scan of the lane totals.
__global__ void __launch_bounds__(256)
dt_cumsum_kernel(const float* __restrict__ dt, const float* __restrict__ dt_bias, const float* __restrict__ A,
                 float* __restrict__ q, float* __restrict__ cs, SsdShape s) {
    __shared__ float patch[kTile][33];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k = blockIdx.x, h0 = blockIdx.y * 32, b = blockIdx.z;
    const bool softplus = (s.flags & SSD_FLAG_DT_SOFTPLUS) != 0;
    const int h = h0 + lane;
    const float bias = (dt_bias != nullptr && h < s.nheads) ? dt_bias[h] : 0.f;
    for (int t = warp; t < kTile; t += 8) {
        float v = 0.f;
        if (h < s.nheads) {
            v = dt[(static_cast<size_t>(b) * s.seqlen + k * kTile + t) * s.nheads + h] + bias;
            if (softplus) v = softplus_f(v);
            v = fminf(fmaxf(v, s.dt_min), s.dt_max);
            if (s.valid_len > 0 && k * kTile + t >= s.valid_len) v = 0.f;  // padding: no step, no decay
        }
        patch[t][lane] = v;
    }
    __syncthreads();
    for (int hh = warp * 4; hh < warp * 4 + 4; ++hh) {
        const int head = h0 + hh;
        if (head >= s.nheads) break;
        const float a = A[head];
        float qv[4], c[4];
        float run = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qv[i] = patch[lane * 4 + i][hh];
            run += a * qv[i];
            c[i] = run;
        }
        float incl = run;  // inclusive scan of the lane totals
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        const float before = incl - run;
        const size_t o = (static_cast<size_t>(b) * s.nheads + head) * s.seqlen + k * kTile + lane * 4;
        *reinterpret_cast<float4*>(q + o) = make_float4(qv[0], qv[1], qv[2], qv[3]);
        *reinterpret_cast<float4*>(cs + o) = make_float4(before + c[0], before + c[1], before + c[2], before + c[3]);
    }
}

// ------------------------------------------------------------------ forward state passing
// One thread owns four consecutive state elements of one (b,h) and walks the
// chunks; the buffer holds U_k on entry and S_k (state at the START of chunk
// k) on exit.  final receives S_K.
__global__ void __launch_bounds__(256)
state_passing_fwd_kernel(float* __restrict__ states, const float* __restrict__ cs,
                         const float* __restrict__ initial_state, float* __restrict__ final_state, int nchunks,
                         int pn4, int seqlen, size_t total) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t bh = idx / pn4;
    const int e = static_cast<int>(idx % pn4);
    float4* p = reinterpret_cast<float4*>(states) + bh * nchunks * pn4 + e;
    const float* csl = cs + bh * seqlen + (kTile - 1);
    float4 st = initial_state ? reinterpret_cast<const float4*>(initial_state)[bh * pn4 + e]
                              : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 u = p[0];
    for (int k = 0; k < nchunks; ++k) {
        const float4 cur = u;
        if (k + 1 < nchunks) u = p[static_cast<size_t>(k + 1) * pn4];  // next load in flight before the store
        const float alpha = expf(csl[static_cast<size_t>(k) * kTile]);
        p[static_cast<size_t>(k) * pn4] = st;
        st.x = alpha * st.x + cur.x;
        st.y = alpha * st.y + cur.y;
        st.z = alpha * st.z + cur.z;
        st.w = alpha * st.w + cur.w;
    }
    if (final_state != nullptr) reinterpret_cast<float4*>(final_state)[bh * pn4 + e] = st;
}

// ------------------------------------------------------------------ read-only fold of the recurrence
// acc <- exp(cs_last,k) * acc + terms[k], walked over the tiles forward (reverse = 0: the state after the
// last tile from the per-tile contributions U_k) or backward (reverse = 1: the gradient of the state before
// the first tile from the local dS_k).  Nothing is written but the [P,N] result: the sequence-parallel
// mode uses it to learn a rank's outflow before it knows its inflow.
__global__ void __launch_bounds__(256)
state_fold_kernel(const float* __restrict__ terms, const float* __restrict__ cs, const float* __restrict__ start,
                  float* __restrict__ result, int nchunks, int pn4, int seqlen, size_t total, int reverse) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t bh = idx / pn4;
    const int e = static_cast<int>(idx % pn4);
    const float4* p = reinterpret_cast<const float4*>(terms) + bh * nchunks * pn4 + e;
    const float* csl = cs + bh * seqlen + (kTile - 1);
    float4 acc = start ? reinterpret_cast<const float4*>(start)[bh * pn4 + e] : make_float4(0.f, 0.f, 0.f, 0.f);
    auto tile_of = [&](int i) { return reverse ? nchunks - 1 - i : i; };
    float4 u = p[static_cast<size_t>(tile_of(0)) * pn4];
    for (int i = 0; i < nchunks; ++i) {
        const float4 cur = u;
        if (i + 1 < nchunks) u = p[static_cast<size_t>(tile_of(i + 1)) * pn4];
        const float alpha = expf(csl[static_cast<size_t>(tile_of(i)) * kTile]);
        acc.x = alpha * acc.x + cur.x;
        acc.y = alpha * acc.y + cur.y;
        acc.z = alpha * acc.z + cur.z;
        acc.w = alpha * acc.w + cur.w;
    }
    reinterpret_cast<float4*>(result)[bh * pn4 + e] = acc;
}

// ------------------------------------------------------------------ backward state passing
// CTA = one (b,h); thread owns ELEMS float4 of the [P,N] state.  dstates holds
// the local dS_k on entry and dU_k (gradient reaching chunk k's own state
// contribution, i.e. d loss / d S_{k+1}) on exit.  g_last[b,h,k] =
// alpha_k * sum(dU_k * S_k) is the gradient w.r.t. cs_last of chunk k.
// The block reduction is a fixed tree, so results are run-to-run identical.
constexpr int kPartTiles = 384;  // tiles whose per-warp partials share the 48 KB of shared memory
template <int ELEMS, bool LONG>
__global__ void __launch_bounds__(1024)
state_passing_bwd_kernel(float* __restrict__ dstates, const float* __restrict__ states_start,
                         const float* __restrict__ cs, const float* __restrict__ dfinal, float* __restrict__ g_last,
                         float* __restrict__ d_initial, int nchunks, int seqlen) {
    extern __shared__ float part[];  // [min(nchunks, kPartTiles)][32]: per-warp partial dot products
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t bh = blockIdx.x;
    const int pn4 = ELEMS * 1024;
    float4* dp = reinterpret_cast<float4*>(dstates) + bh * nchunks * pn4;
    const float4* sp = reinterpret_cast<const float4*>(states_start) + bh * nchunks * pn4;
    const float* csl = cs + bh * seqlen + (kTile - 1);
    const bool want_g = g_last != nullptr;  // without it the forward's states are not read at all
    float4 g[ELEMS], ds_n[ELEMS], st_n[ELEMS];
#pragma unroll
    for (int i = 0; i < ELEMS; ++i) {
        g[i] = dfinal ? reinterpret_cast<const float4*>(dfinal)[bh * pn4 + i * 1024 + tid] : make_float4(0, 0, 0, 0);
        const size_t o = static_cast<size_t>(nchunks - 1) * pn4 + i * 1024 + tid;
        ds_n[i] = dp[o];
        st_n[i] = want_g ? sp[o] : make_float4(0, 0, 0, 0);
    }
    if constexpr (!LONG) {
        // No block-wide barrier inside the walk over the tiles: each warp reduces its own products and
        // parks the partial; the loads of the next tile are always in flight before this tile's stores.
        for (int k = nchunks - 1; k >= 0; --k) {
            const float alpha = expf(csl[static_cast<size_t>(k) * kTile]);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < ELEMS; ++i) {
                const size_t o = static_cast<size_t>(k) * pn4 + i * 1024 + tid;
                const float4 ds = ds_n[i];
                const float4 st = st_n[i];
                if (k > 0) {
                    ds_n[i] = dp[o - pn4];
                    if (want_g) st_n[i] = sp[o - pn4];
                }
                dp[o] = g[i];
                dot += g[i].x * st.x + g[i].y * st.y + g[i].z * st.z + g[i].w * st.w;
                g[i].x = ds.x + alpha * g[i].x;
                g[i].y = ds.y + alpha * g[i].y;
                g[i].z = ds.z + alpha * g[i].z;
                g[i].w = ds.w + alpha * g[i].w;
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
            if (lane == 0) part[k * 32 + warp] = dot;
        }
        __syncthreads();
        for (int k = warp; k < nchunks; k += 32) {
            float v = part[k * 32 + lane];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0 && want_g) g_last[bh * nchunks + k] = expf(csl[static_cast<size_t>(k) * kTile]) * v;
        }
    } else {
        // More tiles than partials fit the shared memory (sequences beyond 49152 tokens): the same walk in
        // blocks of kPartTiles tiles, with the fixed-order reduction of a block's partials between two blocks.
        for (int k_hi = nchunks; k_hi > 0; k_hi -= kPartTiles) {
            const int k_lo = k_hi > kPartTiles ? k_hi - kPartTiles : 0;
            for (int k = k_hi - 1; k >= k_lo; --k) {
                const float alpha = expf(csl[static_cast<size_t>(k) * kTile]);
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < ELEMS; ++i) {
                    const size_t o = static_cast<size_t>(k) * pn4 + i * 1024 + tid;
                    const float4 ds = ds_n[i];
                    const float4 st = st_n[i];
                    if (k > 0) {
                        ds_n[i] = dp[o - pn4];
                        if (want_g) st_n[i] = sp[o - pn4];
                    }
                    dp[o] = g[i];
                    dot += g[i].x * st.x + g[i].y * st.y + g[i].z * st.z + g[i].w * st.w;
                    g[i].x = ds.x + alpha * g[i].x;
                    g[i].y = ds.y + alpha * g[i].y;
                    g[i].z = ds.z + alpha * g[i].z;
                    g[i].w = ds.w + alpha * g[i].w;
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
                if (lane == 0) part[(k - k_lo) * 32 + warp] = dot;
            }
            __syncthreads();
            for (int k = k_lo + warp; k < k_hi; k += 32) {
                float v = part[(k - k_lo) * 32 + lane];
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
                if (lane == 0 && want_g) g_last[bh * nchunks + k] = expf(csl[static_cast<size_t>(k) * kTile]) * v;
            }
            if (k_lo > 0) __syncthreads();  // the partials are read before the next block overwrites them
        }
    }
    if (d_initial != nullptr) {
#pragma unroll
        for (int i = 0; i < ELEMS; ++i) reinterpret_cast<float4*>(d_initial)[bh * pn4 + i * 1024 + tid] = g[i];
    }
}

// ------------------------------------------------------------------ ddt transpose + dA reduction
// ddt_t [B,H,L] -> ddt [B,L,H] through a 32x32 shared-memory turn.
__global__ void __launch_bounds__(256)
ddt_transpose_kernel(const float* __restrict__ ddt_t, float* __restrict__ ddt, int seqlen, int nheads) {
    __shared__ float tile[32][33];
    const int b = blockIdx.z, t0 = blockIdx.x * 32, h0 = blockIdx.y * 32;
    const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
    for (int i = ly; i < 32; i += 8) {
        const int h = h0 + i;
        tile[i][lx] = h < nheads ? ddt_t[(static_cast<size_t>(b) * nheads + h) * seqlen + t0 + lx] : 0.f;
    }
    __syncthreads();
    for (int i = ly; i < 32; i += 8) {
        const int h = h0 + lx;
        if (h < nheads) ddt[(static_cast<size_t>(b) * seqlen + t0 + i) * nheads + h] = tile[lx][i];
    }
}
// dA[h] = sum over (b, k) of the per-tile partials, one warp per head, fixed order.
__global__ void __launch_bounds__(32)
da_reduce_kernel(const double* __restrict__ part, float* __restrict__ dA, int batch, int nheads, int nchunks) {
    const int h = blockIdx.x, lane = threadIdx.x;
    double acc = 0.0;
    const int n = batch * nchunks;
    for (int i = lane; i < n; i += 32) {
        const int b = i / nchunks, k = i % nchunks;
        acc += part[(static_cast<size_t>(b) * nheads + h) * nchunks + k];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) dA[h] = static_cast<float>(acc);
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_dt_cumsum(const SsdShape* shape, const float* dt, const float* dt_bias, const float* A, float* q,
                             float* cs, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!dt || !A || !q || !cs) return SSD_ERR_NULL;
    const dim3 grid(shape->seqlen / kTile, (shape->nheads + 31) / 32, shape->batch);
    dt_cumsum_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dt, dt_bias, A, q, cs, *shape);
    return launch_status();
}

extern "C" int ssd_state_passing_fwd(const SsdShape* shape, float* states, const float* cs,
                                     const float* initial_state, float* final_state, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!states || !cs) return SSD_ERR_NULL;
    const int pn4 = shape->headdim * shape->dstate / 4;
    const size_t total = static_cast<size_t>(shape->batch) * shape->nheads * pn4;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    state_passing_fwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        states, cs, initial_state, final_state, shape->seqlen / kTile, pn4, shape->seqlen, total);
    return launch_status();
}

extern "C" int ssd_state_fold(const SsdShape* shape, const float* terms, const float* cs, const float* start,
                              float* result, int reverse, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!terms || !cs || !result) return SSD_ERR_NULL;
    const int pn4 = shape->headdim * shape->dstate / 4;
    const size_t total = static_cast<size_t>(shape->batch) * shape->nheads * pn4;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    state_fold_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        terms, cs, start, result, shape->seqlen / kTile, pn4, shape->seqlen, total, reverse != 0);
    return launch_status();
}

extern "C" int ssd_state_passing_bwd(const SsdShape* shape, float* dstates, const float* states_start, const float* cs,
                                     const float* dfinal, float* g_last, float* d_initial, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!dstates || !cs || (g_last && !states_start)) return SSD_ERR_NULL;
    const unsigned blocks = static_cast<unsigned>(shape->batch) * shape->nheads;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int nchunks = shape->seqlen / kTile;
    const size_t part_bytes = static_cast<size_t>(nchunks < kPartTiles ? nchunks : kPartTiles) * 32 * sizeof(float);
    const bool lng = nchunks > kPartTiles;
    auto launch = [&](auto kernel) {
        kernel<<<blocks, 1024, part_bytes, st>>>(dstates, states_start, cs, dfinal, g_last, d_initial, nchunks,
                                                 shape->seqlen);
    };
    if (shape->dstate == 64) {
        lng ? launch(state_passing_bwd_kernel<1, true>) : launch(state_passing_bwd_kernel<1, false>);
    } else {
        lng ? launch(state_passing_bwd_kernel<2, true>) : launch(state_passing_bwd_kernel<2, false>);
    }
    return launch_status();
}

extern "C" int ssd_dt_finalize_bwd(const SsdShape* shape, const float* ddt_t, const double* dA_partial, float* ddt,
                                   float* dA, ssd_stream_t stream) {
    using namespace ssd;
    const int rc = ssd_check_shape(shape);
    if (rc != SSD_OK) return rc;
    if (!ddt_t || !dA_partial || !ddt || !dA) return SSD_ERR_NULL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(shape->seqlen / 32, (shape->nheads + 31) / 32, shape->batch);
    ddt_transpose_kernel<<<grid, 256, 0, st>>>(ddt_t, ddt, shape->seqlen, shape->nheads);
    da_reduce_kernel<<<shape->nheads, 32, 0, st>>>(dA_partial, dA, shape->batch, shape->nheads,
                                                   shape->seqlen / kTile);
    return launch_status();
}
