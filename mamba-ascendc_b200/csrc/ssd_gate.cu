// D skip connection and SiLU(z) gate around the SSD output, as one pass forward and one pass backward:
//
//   out = (y + D .* x) .* silu(z)                 (ssd_reference.py:300-318; either of D, z may be absent)
//
//   dy  = dout .* silu(z) ;  dz = dout .* (y + D .* x) .* silu'(z) ;  dD = sum dy .* x
//   (dx += D .* dy happens in the epilogue of the dx kernel, ssd_bwd_dx.cu)
//
// The reference fuses these into its state-epilogue and gate kernels (mamba2_ssd_state_epilogue.cpp:413-482,
// bwd_gate/design.md:8-13).  Element-wise and bandwidth bound: the tensors are walked as [tokens, H*P] with
// float4 accesses along the row; dD is reduced in two phases in a fixed order (fp64 in the second phase).
#include "ssd_host.h"

namespace ssd {

namespace {

constexpr int kGateThreads = 256;
constexpr int kGateRows = 128;  // tokens per CTA in the backward pass (one dD partial per CTA and column)

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + __expf(-v)); }

// D for the four columns c..c+3 of a row (c % 4 == 0): d_mode 0 none, 1 per head [H], 2 per channel [H,P].
__device__ __forceinline__ float4 load_d(const float* D, int d_mode, int c, int p_dim) {
    if (d_mode == 2) return ld4(D + c);
    if (d_mode == 1) {
        const float d = D[c / p_dim];
        return make_float4(d, d, d, d);
    }
    return make_float4(0.f, 0.f, 0.f, 0.f);
}

__global__ void __launch_bounds__(kGateThreads)
gate_skip_fwd_kernel(const float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ D, int d_mode,
                     const float* __restrict__ z, float* __restrict__ out, long long rows, int cols, int p_dim) {
    const int c = (blockIdx.x * kGateThreads + threadIdx.x) * 4;
    if (c >= cols) return;
    const float4 d = load_d(D, d_mode, c, p_dim);
    for (long long r = blockIdx.y; r < rows; r += gridDim.y) {
        const size_t o = static_cast<size_t>(r) * cols + c;
        float4 v = ld4(y + o);
        if (d_mode) {
            const float4 xv = ld4(x + o);
            v.x += d.x * xv.x;
            v.y += d.y * xv.y;
            v.z += d.z * xv.z;
            v.w += d.w * xv.w;
        }
        if (z) {
            const float4 zv = ld4(z + o);
            v.x *= zv.x * sigmoidf_(zv.x);
            v.y *= zv.y * sigmoidf_(zv.y);
            v.z *= zv.z * sigmoidf_(zv.z);
            v.w *= zv.w * sigmoidf_(zv.w);
        }
        st4(out + o, v);
    }
}

// Backward, one CTA per (1024 columns, kGateRows tokens).  dy and dz may be null (no z: dy equals dout and the
// caller uses dout itself).  part[row_block][cols] receives this CTA's sum over its tokens of dy .* x.
__global__ void __launch_bounds__(kGateThreads)
gate_skip_bwd_kernel(const float* __restrict__ dout, const float* __restrict__ y, const float* __restrict__ x,
                     const float* __restrict__ D, int d_mode, const float* __restrict__ z, float* __restrict__ dy,
                     float* __restrict__ dz, float* __restrict__ part, long long rows, int cols, int p_dim) {
    const int c = (blockIdx.x * kGateThreads + threadIdx.x) * 4;
    if (c >= cols) return;
    const float4 d = load_d(D, d_mode, c, p_dim);
    const long long r0 = static_cast<long long>(blockIdx.y) * kGateRows;
    const long long r1 = r0 + kGateRows < rows ? r0 + kGateRows : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long r = r0; r < r1; ++r) {
        const size_t o = static_cast<size_t>(r) * cols + c;
        const float4 g = ld4(dout + o);
        float4 gy = g;
        float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d_mode) xv = ld4(x + o);
        if (z) {
            const float4 zv = ld4(z + o);
            const float4 yv = ld4(y + o);
            const float zz[4] = {zv.x, zv.y, zv.z, zv.w};
            const float pre[4] = {yv.x + d.x * xv.x, yv.y + d.y * xv.y, yv.z + d.z * xv.z, yv.w + d.w * xv.w};
            const float gg[4] = {g.x, g.y, g.z, g.w};
            float oy[4], oz[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float s = sigmoidf_(zz[i]);
                oy[i] = gg[i] * zz[i] * s;
                oz[i] = gg[i] * pre[i] * s * (1.f + zz[i] * (1.f - s));
            }
            gy = make_float4(oy[0], oy[1], oy[2], oy[3]);
            st4(dy + o, gy);
            st4(dz + o, make_float4(oz[0], oz[1], oz[2], oz[3]));
        }
        acc.x += gy.x * xv.x;
        acc.y += gy.y * xv.y;
        acc.z += gy.z * xv.z;
        acc.w += gy.w * xv.w;
    }
    if (d_mode) st4(part + static_cast<size_t>(blockIdx.y) * cols + c, acc);
}

// Second phase of dD: block per head, thread per channel; row blocks in order, then (per-head D) the channels.
__global__ void gate_dd_reduce_kernel(const float* __restrict__ part, int row_blocks, int cols, int p_dim, int d_mode,
                                      float* __restrict__ dD) {
    extern __shared__ double red[];
    const int h = blockIdx.x, p = threadIdx.x;
    double s = 0.0;
    if (p < p_dim)
        for (int rb = 0; rb < row_blocks; ++rb) s += part[static_cast<size_t>(rb) * cols + h * p_dim + p];
    if (d_mode == 2) {
        if (p < p_dim) dD[h * p_dim + p] = static_cast<float>(s);
        return;
    }
    red[p] = p < p_dim ? s : 0.0;
    __syncthreads();
    if (p == 0) {
        double t = 0.0;
        for (int i = 0; i < p_dim; ++i) t += red[i];
        dD[h] = static_cast<float>(t);
    }
}

int gate_dims(const SsdShape* s, long long* rows, int* cols) {
    if (!s) return SSD_ERR_NULL;
    if (s->batch <= 0 || s->seqlen <= 0 || s->nheads <= 0 || s->headdim <= 0) return SSD_ERR_SHAPE;
    if (s->headdim % 4 != 0 || s->headdim > 1024) return SSD_ERR_UNSUPPORTED;
    *rows = static_cast<long long>(s->batch) * s->seqlen;
    *cols = s->nheads * s->headdim;
    return SSD_OK;
}

}  // namespace

}  // namespace ssd

extern "C" size_t ssd_gate_partial_floats(const SsdShape* shape) {
    long long rows = 0;
    int cols = 0;
    if (ssd::gate_dims(shape, &rows, &cols) != SSD_OK) return 0;
    return static_cast<size_t>((rows + ssd::kGateRows - 1) / ssd::kGateRows) * cols;
}

extern "C" int ssd_gate_skip_fwd(const SsdShape* shape, const float* y, const float* x, const float* D, int d_mode,
                                 const float* z, float* out, ssd_stream_t stream) {
    using namespace ssd;
    long long rows = 0;
    int cols = 0;
    const int rc = gate_dims(shape, &rows, &cols);
    if (rc != SSD_OK) return rc;
    if (!y || !out || (d_mode != 0 && (!D || !x))) return SSD_ERR_NULL;
    if (d_mode < 0 || d_mode > 2) return SSD_ERR_SHAPE;
    const dim3 grid((cols / 4 + kGateThreads - 1) / kGateThreads, static_cast<unsigned>(rows < 1024 ? rows : 1024));
    gate_skip_fwd_kernel<<<grid, kGateThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(y, x, D, d_mode, z, out, rows,
                                                                                            cols, shape->headdim);
    return launch_status();
}

extern "C" int ssd_gate_skip_bwd(const SsdShape* shape, const float* dout, const float* y, const float* x, const float* D,
                                 int d_mode, const float* z, float* dy, float* dz, float* dD_partial, float* dD,
                                 ssd_stream_t stream) {
    using namespace ssd;
    long long rows = 0;
    int cols = 0;
    const int rc = gate_dims(shape, &rows, &cols);
    if (rc != SSD_OK) return rc;
    if (d_mode < 0 || d_mode > 2) return SSD_ERR_SHAPE;
    if (!dout || (z && (!y || !dy || !dz)) || (d_mode != 0 && (!D || !x || !dD_partial || !dD))) return SSD_ERR_NULL;
    if (!z && d_mode == 0) return SSD_OK;  // nothing to do
    const long long row_blocks = (rows + kGateRows - 1) / kGateRows;
    if (row_blocks > 65535) return SSD_ERR_UNSUPPORTED;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid((cols / 4 + kGateThreads - 1) / kGateThreads, static_cast<unsigned>(row_blocks));
    gate_skip_bwd_kernel<<<grid, kGateThreads, 0, st>>>(dout, y, x, D, d_mode, z, dy, dz, dD_partial, rows, cols,
                                                        shape->headdim);
    if (d_mode != 0) {
        const int threads = (shape->headdim + 31) / 32 * 32;
        gate_dd_reduce_kernel<<<shape->nheads, threads, threads * sizeof(double), st>>>(
            dD_partial, static_cast<int>(row_blocks), cols, shape->headdim, d_mode, dD);
    }
    return launch_status();
}
