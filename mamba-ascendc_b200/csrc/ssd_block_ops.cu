// Element-wise companions of the SSD inside a Mamba-2 block, forward only, for the Vision-Mamba2 network of
// benchmark configuration 4 (RMSNorm -> in_proj -> depthwise causal conv1d + SiLU -> SSD -> gated RMSNorm ->
// out_proj).  Bandwidth-bound kernels that each read their input once and write their output once, in place of
// the ten-odd framework launches per step they replace:
//
//   block_rmsnorm_kernel     out = x * rsqrt(mean(x^2) + eps) * w,  optionally x <- x * silu(z) first (the gated norm)
//   block_conv_silu_kernel   depthwise causal convolution of width 4 along the sequence, bias, SiLU, and the split of
//                            the result into contiguous x [B,L,d_in], B [B,L,GN] and C [B,L,GN] tensors
//
// Inputs may be column slices of a wider row-major matrix (the in_proj output holds z | xBC | dt side by side),
// hence the explicit row strides; rows need not be 16-byte aligned, so loads are scalar with lanes along the
// channels (coalesced).  The reference's demo network applies the same operations with framework calls
// (mamba_torch/vmamba2_network.py:197-302).
#include "ssd_host.h"

namespace ssd {

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

// One warp per row; d <= 32 * kMaxPerLane.
constexpr int kMaxPerLane = 16;

__global__ void __launch_bounds__(256)
block_rmsnorm_kernel(const float* __restrict__ x, long long x_stride, const float* __restrict__ z, long long z_stride,
                     const float* __restrict__ w, float* __restrict__ out, long long rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* xr = x + row * x_stride;
    const float* zr = z ? z + row * z_stride : nullptr;
    float v[kMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        float t = 0.f;
        if (c < d) {
            t = xr[c];
            if (zr) t *= silu_f(zr[c]);
        }
        v[i] = t;
        ss = fmaf(t, t, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = rsqrtf(ss / static_cast<float>(d) + eps);
    float* orow = out + row * d;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < d) orow[c] = v[i] * r * w[c];
    }
}

// CTA = 128 channels x kConvTokens tokens of one batch row; a thread walks its channel along the tokens with the
// last three inputs in registers.  weight [C,4] (tap k multiplies the input 3-k tokens back), bias [C].
constexpr int kConvTokens = 64;

__global__ void __launch_bounds__(128)
block_conv_silu_kernel(const float* __restrict__ xbc, long long row_stride, const float* __restrict__ weight,
                       const float* __restrict__ bias, float* __restrict__ x_out, float* __restrict__ b_out,
                       float* __restrict__ c_out, int seqlen, int d_in, int gn) {
    const int channels = d_in + 2 * gn;
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= channels) return;
    const int t0 = blockIdx.y * kConvTokens;
    const long long b = blockIdx.z;
    const float* src = xbc + (b * seqlen) * row_stride + c;
    const float w0 = weight[c * 4], w1 = weight[c * 4 + 1], w2 = weight[c * 4 + 2], w3 = weight[c * 4 + 3];
    const float bs = bias ? bias[c] : 0.f;
    float* dst;
    int width, col;
    if (c < d_in) {
        dst = x_out, width = d_in, col = c;
    } else if (c < d_in + gn) {
        dst = b_out, width = gn, col = c - d_in;
    } else {
        dst = c_out, width = gn, col = c - d_in - gn;
    }
    dst += (b * seqlen) * width + col;
    float a = t0 >= 3 ? src[(t0 - 3) * row_stride] : 0.f;  // inputs 3, 2 and 1 tokens back
    float bb = t0 >= 2 ? src[(t0 - 2) * row_stride] : 0.f;
    float cc = t0 >= 1 ? src[(t0 - 1) * row_stride] : 0.f;
    const int t1 = t0 + kConvTokens < seqlen ? t0 + kConvTokens : seqlen;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        const float cur = src[static_cast<long long>(t) * row_stride];
        const float v = fmaf(w0, a, fmaf(w1, bb, fmaf(w2, cc, fmaf(w3, cur, bs))));
        dst[static_cast<long long>(t) * width] = silu_f(v);
        a = bb, bb = cc, cc = cur;
    }
}

}  // namespace

}  // namespace ssd

extern "C" int ssd_block_rmsnorm_fwd(const float* x, long long x_stride, const float* z, long long z_stride,
                                     const float* w, float* out, long long rows, int d, float eps,
                                     ssd_stream_t stream) {
    using namespace ssd;
    if (!x || !w || !out) return SSD_ERR_NULL;
    if (rows <= 0 || d <= 0 || x_stride < d || (z && z_stride < d)) return SSD_ERR_SHAPE;
    if (d > 32 * kMaxPerLane) return SSD_ERR_UNSUPPORTED;
    const long long blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffffLL) return SSD_ERR_RANGE;
    block_rmsnorm_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_stride, z, z_stride, w, out, rows, d, eps);
    return launch_status();
}

extern "C" int ssd_block_conv_silu_fwd(const float* xbc, long long row_stride, const float* weight, const float* bias,
                                       float* x_out, float* b_out, float* c_out, int batch, int seqlen, int d_in, int gn,
                                       ssd_stream_t stream) {
    using namespace ssd;
    if (!xbc || !weight || !x_out || !b_out || !c_out) return SSD_ERR_NULL;
    if (batch <= 0 || seqlen <= 0 || d_in <= 0 || gn <= 0 || row_stride < d_in + 2 * gn) return SSD_ERR_SHAPE;
    if (batch > 65535 || (seqlen + kConvTokens - 1) / kConvTokens > 65535) return SSD_ERR_RANGE;
    const int channels = d_in + 2 * gn;
    const dim3 grid((channels + 127) / 128, (seqlen + kConvTokens - 1) / kConvTokens, batch);
    block_conv_silu_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(xbc, row_stride, weight, bias, x_out,
                                                                                    b_out, c_out, seqlen, d_in, gn);
    return launch_status();
}
