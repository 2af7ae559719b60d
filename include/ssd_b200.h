/* C ABI of the B200 (sm_100a) Mamba-2 SSD library, libssd_b200.so.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; the
 * caller owns all memory (outputs and workspace included), the library never
 * allocates or frees.  Work is enqueued on `stream` and the call returns
 * without synchronising.  Return value: SSD_OK (0) or a negative SSD_ERR_*
 * code, in which case nothing was launched.  All tensors are contiguous fp32.
 *
 * Citations name the file of the So-cean/mamba-ascendc tree whose interface
 * the entry point stands in for.
 *
 * Shape order everywhere: x[B,L,H,P], dt[B,L,H], A[H], B/C[B,L,G,N],
 * out[B,L,H,P], final_state[B,H,P,N].  Head h reads group h / (H/G).
 */
#ifndef SSD_B200_H_
#define SSD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ssd_stream_t; /* same type as cudaStream_t */

enum {
    SSD_OK = 0,
    SSD_ERR_NULL = -1,        /* a required pointer is null                                  */
    SSD_ERR_SHAPE = -2,       /* a dimension is non-positive or H % G != 0                   */
    SSD_ERR_UNSUPPORTED = -3, /* valid SSD problem, but outside what the kernels cover       */
    SSD_ERR_WORKSPACE = -4,   /* workspace smaller than ssd_workspace_bytes()                */
    SSD_ERR_ALIGN = -5,       /* a tensor base address is not 16-byte aligned                */
    SSD_ERR_TENSORMAP = -6,   /* the driver rejected a TMA tensor map                        */
    SSD_ERR_LAUNCH = -7       /* kernel launch failed (cudaGetLastError)                     */
};

enum { SSD_FLAG_DT_SOFTPLUS = 1u };

/* Problem shape.  `tile` is the number of tokens one CTA treats as a chunk
 * (the results do not depend on it mathematically); the kernels need
 * tile == 128 and seqlen % tile == 0.  Supported: headdim == 64,
 * dstate in {64, 128}. */
typedef struct SsdShape {
    int32_t batch;   /* B */
    int32_t seqlen;  /* L */
    int32_t nheads;  /* H */
    int32_t headdim; /* P */
    int32_t dstate;  /* N */
    int32_t tile;    /* T */
    int32_t ngroups; /* G */
    uint32_t flags;  /* SSD_FLAG_* */
} SsdShape;

/* Human-readable text for a return code ("ssd: ..." style, used by the Python
 * layer for its RuntimeError messages). */
const char* ssd_error_string(int code);

/* Shape validation shared by every entry point.  Mirrors the host checks of
 * mamba_ascendc/csrc/ops/mamba2_ssd_fwd/op_host/mamba2_ssd_fwd.cpp:59-112
 * (ranks, positivity, H % G == 0, chunk > 0) and adds this library's own
 * limits (SSD_ERR_UNSUPPORTED). */
int ssd_check_shape(const SsdShape* shape);

/* Tile-level check of the tensor-core path: D[128,n] = A * B^T with K = 128,
 * fp32 in, split-bf16 tcgen05 MMAs, fp32 out.  a_mn / b_mn select whether the
 * operand is given as [rows = non-contracted index, cols = k] (0) or as
 * [rows = k, cols = non-contracted index] (1).  `status` is a device int the
 * kernel sets non-zero if a bounded wait gave up.  Test-only; no counterpart
 * in the reference (its analogue is the Cube matmul unit,
 * mamba_ascendc_ops/mamba2_ssd_chunk_mix/op_kernel/mamba2_dynamic_matmul.h:195-233). */
int ssd_selftest_umma(const float* a, const float* b, float* d, int n, int a_mn, int b_mn, int* status,
                      ssd_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* SSD_B200_H_ */
