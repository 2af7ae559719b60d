/* C ABI of the B200 (sm_100a) Mamba-2 SSD library, libssd_b200.so.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; the
 * caller owns all memory (outputs and workspace included), the library never
 * allocates or frees.  Work is enqueued on `stream` and the call returns
 * without synchronising.  Return value: SSD_OK (0) or a negative SSD_ERR_*
 * code, in which case nothing was launched (ssd_forward_static, which runs
 * four stages, says below what holds for it).  All tensors are contiguous fp32.
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
    SSD_ERR_RANGE = -4,       /* a size is beyond what one launch can index, see ssd_check_shape */
    SSD_ERR_ALIGN = -5,       /* a tensor base address is not 16-byte aligned                */
    SSD_ERR_TENSORMAP = -6,   /* the driver rejected a TMA tensor map                        */
    SSD_ERR_LAUNCH = -7,      /* kernel launch failed (cudaGetLastError)                     */
    SSD_ERR_STATIC_SCRATCH = -8 /* problem too large for ssd_forward_static's built-in scratch */
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
    float dt_min;    /* q = clamp(softplus(dt + dt_bias), dt_min, dt_max); the reference's dt_limit, */
    float dt_max;    /* default (0, +inf)                                                          */
    int32_t valid_len; /* tokens >= valid_len of every sequence are padding (q = 0); 0 = no padding  */
} SsdShape;

/* Human-readable text for a return code ("ssd: ..." style, used by the Python
 * layer for its RuntimeError messages). */
const char* ssd_error_string(int code);

/* Shape validation shared by every entry point.  Mirrors the host checks of
 * mamba_ascendc/csrc/ops/mamba2_ssd_fwd/op_host/mamba2_ssd_fwd.cpp:59-112
 * (ranks, positivity, H % G == 0, chunk > 0) and adds this library's own
 * limits: SSD_ERR_UNSUPPORTED for headdim != 64, dstate not in {64, 128}, tile != 128 or a ragged
 * seqlen; SSD_ERR_RANGE for batch or ngroups above 65535 (grid dimensions) or for
 * batch * seqlen or batch * nheads * (seqlen / tile) * headdim at or above 2^31 (TMA coordinates). */
int ssd_check_shape(const SsdShape* shape);

/* Size in bytes of one caller-allocated internal buffer for `shape`, so that a binder need not transcribe
 * the layouts below; 0 for an invalid shape or an unknown `which`.  Query-then-allocate, the role of the
 * workspace-size call of the reference's launch helper
 * (mamba_ascendc/csrc/utils/torch_aclnn_helper.h:526-546). */
enum {
    SSD_BUF_Q = 0,          /* float [B,H,L]                                   */
    SSD_BUF_CS = 1,         /* float [B,H,L]                                   */
    SSD_BUF_STATES = 2,     /* float [B,H,K,P,N]   (also the size of dstates)  */
    SSD_BUF_FINAL_STATE = 3,/* float [B,H,P,N]     (initial_state, dfinal, d_initial alike) */
    SSD_BUF_G_LAST = 4,     /* float [B,H,K]                                   */
    SSD_BUF_DDT_T = 5,      /* float [B,H,L]                                   */
    SSD_BUF_DA_PARTIAL = 6, /* double [B,H,K]                                  */
    SSD_BUF_GATE_PARTIAL = 7,/* float [ssd_gate_partial_floats()]              */
    SSD_BUF_STATUS = 8      /* one int32                                       */
};
size_t ssd_buffer_bytes(const SsdShape* shape, int which);

/* ---------------------------------------------------------------- forward stages
 *
 * Internal buffers (caller-allocated fp32, K = L / tile):
 *   q, cs        [B,H,L]      q = dt after softplus/clamp; cs = inclusive in-tile cumulative sum of A*q
 *   states       [B,H,K,P,N]  chunk states U_k, turned in place into the state at the START of tile k
 *   status       one int32, zeroed by the caller once; a kernel whose bounded wait gives up stores a
 *                non-zero code there and writes no results; its low four bits say why: 1 = a TMA load did
 *                not arrive, 2 = a tensor-core product (or the hand-off to the issuing warp) did not
 *                complete, 3 = the dynamic shared memory did not start on the 1024-byte boundary it was
 *                declared with.  The bits above locate the wait for diagnosis (source file in bits 12 and up,
 *                number of the wait within the file in bits 4-11).
 *                Kernels launched while the word is non-zero return at once WITHOUT writing their outputs:
 *                the caller must read the word (after synchronising) before it trusts any result, and
 *                zero it before the next use.
 */

/* q and cs from dt, the optional per-head dt_bias[H] (null = none) and A.  Warp-scan kernel.  Stands in for the dt / dA part of
 * mamba2_ssd_preprocess (mamba_ascendc/csrc/ops/mamba2_ssd_preprocess/op_host/
 * mamba2_ssd_preprocess.cpp:26-109; softplus op_kernel :300-320, scan :328-349). */
int ssd_dt_cumsum(const SsdShape* shape, const float* dt, const float* dt_bias, const float* A, float* q, float* cs,
                  ssd_stream_t stream);

/* states[b,h,k,p,n] = sum_t w_t X[t,p] M[t,n] on tcgen05.
 * mode 0: X = x, M = B, w_t = q_t exp(cs_last - cs_t): the chunk-state product of
 *         mamba2_ssd_chunk_mix (mamba_ascendc/csrc/aclnn/mamba2_ssd_chunk_mix.cpp:7-69).
 * mode 1: X = dout, M = C, w_t = exp(cs_t): the local state gradient dS_k of
 *         mamba2_ssd_bwd_off_prepare + matmul(Q^T, C) (ascend_kernel/mamba2.py:1009-1023). */
int ssd_chunk_state(const SsdShape* shape, const float* x, const float* m, const float* q, const float* cs,
                    float* states, int mode, int* status, ssd_stream_t stream);

/* In-place inter-tile recurrence S_0 = initial_state (zeros if null), S_{k+1} = exp(cs_last,k) S_k + U_k;
 * initial_state and final_state are [B,H,P,N], either may be null.  Stands in for
 * mamba2_ssd_state_passing (mamba_ascendc/csrc/ops/mamba2_ssd_state_passing/op_host/
 * mamba2_ssd_state_passing.cpp:12-78, which takes the same optional initial state). */
int ssd_state_passing_fwd(const SsdShape* shape, float* states, const float* cs, const float* initial_state,
                          float* final_state, ssd_stream_t stream);

/* out = tril(C B^T .* decay) (q x) + exp(cs) C S^T on tcgen05.  Stands in for the CB / W / y_diag
 * part of mamba2_ssd_chunk_mix plus the torch glue that adds the state term
 * (ascend_kernel/mamba2.py:388-402). */
int ssd_chunk_scan_fwd(const SsdShape* shape, const float* x, const float* bm, const float* cm,
                       const float* states_start, const float* q, const float* cs, float* out, int* status,
                       ssd_stream_t stream);

/* ---------------------------------------------------------------- backward stages (dstate == 64)
 *
 *   dstates      [B,H,K,P,N]  ssd_chunk_state(mode 1) output; ssd_state_passing_bwd turns it in place
 *                             into dU_k = d loss / d (state after tile k)
 *   g_last       [B,H,K]      d loss / d cs_last of tile k through the state recurrence
 *   ddt_t        [B,H,L]      ddt in head-major layout; dA_partial [B,H,K] (fp64)
 */

/* Reverse inter-tile recurrence; dfinal[B,H,P,N] may be null (treated as zeros, as
 * ascend_kernel/mamba2.py:1801-1802 does for a missing gradient).  Stands in for
 * mamba2_ssd_state_passing_bwd (mamba_ascendc/csrc/ops/mamba2_ssd_state_passing_bwd/design.md:49-58).
 * d_initial[B,H,P,N] (may be null) receives the gradient of the initial state.  Any seqlen the forward
 * takes (long sequences are walked in blocks of 384 tiles).  g_last may be null: then states_start is not
 * read (ssd_chunk_dbc_bwd, which streams both state tensors anyway, can produce g_last instead). */
int ssd_state_passing_bwd(const SsdShape* shape, float* dstates, const float* states_start, const float* cs,
                          const float* dfinal, float* g_last, float* d_initial, ssd_stream_t stream);

/* Read-only fold of the inter-tile recurrence: result[B,H,P,N] = acc after acc <- exp(cs_last,k) * acc + terms[k]
 * over the tiles k = 0..K-1 (reverse = 0) or K-1..0 (reverse = 1), starting from `start` (zeros if null).
 * With terms = the chunk states U_k it gives the state a block of tokens hands on; with terms = the local
 * dS_k, start = dfinal and reverse = 1 it gives the gradient the block hands back.  `terms` is not modified.
 * Same recurrences as mamba2_ssd_state_passing / mamba2_ssd_state_passing_bwd (cited above) without their
 * per-tile outputs; used by the sequence-parallel mode, which the single-device reference does not have. */
int ssd_state_fold(const SsdShape* shape, const float* terms, const float* cs, const float* start, float* result,
                   int reverse, ssd_stream_t stream);

/* ssd_chunk_state fused with the inter-tile recurrence: one CTA per (batch, group) walks the tiles in
 * order with the running state of every head of the group in tensor memory, so no per-tile contribution
 * travels through global memory and no separate state-passing launch is needed.
 *   mode 0: x, m = B, start = initial_state (null = zeros); states[k] <- state at the START of tile k
 *           (what ssd_chunk_state + ssd_state_passing_fwd leave there); end = final_state (may be null).
 *   mode 1: x = dout, m = C, start = dfinal (null = zeros); states[k] <- dU_k (what ssd_chunk_state mode 1 +
 *           ssd_state_passing_bwd leave in dstates); end = d_initial (may be null).  g_last, the third output
 *           of the reverse scan, comes from ssd_chunk_dbc_bwd.
 * Takes dstate == 64 and at most 6 heads per group (ssd_chunk_state_scan_supported() == 1); parallelism
 * is batch * ngroups CTAs, so callers use it when that is at least a few times the SM count and the two
 * tile-parallel entry points otherwise.  The resident-state design follows the reference's fused state
 * epilogue (mamba_ascendc_ops/mamba2_ssd_chunk_mix/op_kernel/mamba2_ssd_state_epilogue.cpp:208,
 * :1179-1186); the reverse recurrence is mamba_ascendc/csrc/ops/mamba2_ssd_state_passing_bwd/design.md:49-58. */
int ssd_chunk_state_scan_supported(const SsdShape* shape);
int ssd_chunk_state_scan(const SsdShape* shape, const float* x, const float* m, const float* q, const float* cs,
                         const float* start, float* states, float* end, int mode, int* status, ssd_stream_t stream);

/* dx plus the dt stage (ddt_t, dA_partial).  Stands in for the dx / dR products of
 * mamba2_ssd_chunk_scan_bwd_diag_state, mamba2_ssd_bwd_diag_finalize and mamba2_ssd_dt_bwd
 * (ascend_kernel/mamba2.py:839-962, 1607-1617; mamba2_ssd_dt_bwd/design.md:63-77).
 * `out` is the forward output; dt_bias[H] may be null.  d(dt_bias) is the sum of ddt over batch and sequence.
 * With a D skip connection (d_mode 1: D[H], 2: D[H,P]; 0: none, D ignored) its share of dx, D .* dout, is
 * added in the epilogue; `dout` and `out` are then the gradient and the value of the SSD output BEFORE the
 * skip connection and the gate (the dy of ssd_gate_skip_bwd and the y of ssd_gate_skip_fwd). */
int ssd_chunk_dx_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm, const float* dout,
                     const float* out, const float* dstates, const float* q, const float* cs, const float* dt,
                     const float* dt_bias, const float* A, const float* g_last, float* dx, float* ddt_t,
                     double* dA_partial, const float* D, int d_mode, int* status, ssd_stream_t stream);

/* dB and dC [B,L,G,N], summed over the heads of each group inside the kernel.  Stands in for
 * prepare_dcb, the dC/dB products and group sums of mamba2_ssd_chunk_scan_bwd_diag_state,
 * mamba2_ssd_chunk_scan_bwd_off and mamba2_ssd_bwd_off_finalize (ascend_kernel/mamba2.py:844-859,
 * 946-949, 1023-1045).  If g_last[B,H,K] is not null the kernel also writes it
 * (exp(cs_last,k) * sum(dstates[k] .* states_start[k]), the g_cs_chunk_last output of
 * mamba2_ssd_state_passing_bwd, design.md:49-58): both tensors pass through this kernel tile by tile, so the
 * reverse state scan need not read states_start for it.  ssd_chunk_dx_bwd consumes g_last. */
int ssd_chunk_dbc_bwd(const SsdShape* shape, const float* x, const float* bm, const float* cm, const float* dout,
                      const float* states_start, const float* dstates, const float* q, const float* cs, float* dB,
                      float* dC, float* g_last, int* status, ssd_stream_t stream);

/* ddt[B,L,H] from ddt_t and dA[H] from dA_partial (fixed-order sums).  Stands in for the reduce
 * phase of mamba2_ssd_dt_bwd (op_kernel :1013-1068). */
int ssd_dt_finalize_bwd(const SsdShape* shape, const float* ddt_t, const double* dA_partial, float* ddt, float* dA,
                        ssd_stream_t stream);

/* ---------------------------------------------------------------- D skip connection and SiLU(z) gate
 *
 * out = (y + D .* x) .* silu(z) around the SSD output y, one pass forward and one pass backward.  Stands in
 * for the D / z part of the reference's fused epilogue and gate kernels (mamba_ascendc_ops/.../
 * mamba2_ssd_state_epilogue.cpp:413-482; mamba_ascendc/csrc/ops/mamba2_ssd_bwd_gate/design.md:8-13; the
 * semantics are those of mamba_torch/ssd_reference.py:300-318).  Tensors y, x, z, out [B,L,H,P] fp32, any L,
 * P % 4 == 0; only batch, seqlen, nheads and headdim of the shape are read.
 *   d_mode   0: no D;  1: D[H];  2: D[H,P].        z may be null (no gate).
 * Backward: dy = dout .* silu(z), dz = dout .* (y + D .* x) .* silu'(z) (both only written when z is given;
 * without z the caller uses dout as dy), dD = sum over batch, tokens (and channels for d_mode 1) of dy .* x,
 * reduced in a fixed order through dD_partial (ssd_gate_partial_floats() floats).  The skip connection's
 * share of dx is added by ssd_chunk_dx_bwd (its D / d_mode arguments). */
size_t ssd_gate_partial_floats(const SsdShape* shape);
int ssd_gate_skip_fwd(const SsdShape* shape, const float* y, const float* x, const float* D, int d_mode, const float* z,
                      float* out, ssd_stream_t stream);
int ssd_gate_skip_bwd(const SsdShape* shape, const float* dout, const float* y, const float* x, const float* D,
                      int d_mode, const float* z, float* dy, float* dz, float* dD_partial, float* dD,
                      ssd_stream_t stream);

/* ---------------------------------------------------------------- the SSD's neighbours inside a Mamba-2 block
 *
 * Forward-only element-wise kernels for the Vision-Mamba2 network of the benchmark definition (RMSNorm,
 * depthwise causal conv1d of width 4 + SiLU, gated RMSNorm); the reference's demo network does the same steps
 * with framework calls (mamba_torch/vmamba2_network.py:197-302).  Inputs may be column slices of a wider
 * row-major matrix: `*_stride` is the distance between rows in floats.
 *
 * ssd_block_rmsnorm_fwd: out[rows,d] = t * rsqrt(mean(t^2) + eps) * w with t = x, or x .* silu(z) when z is
 *   not null (the gated norm in front of out_proj).  d <= 512.
 * ssd_block_conv_silu_fwd: xbc[batch*seqlen rows, d_in + 2*gn channels] -> silu(conv(xbc) + bias), written as the
 *   three contiguous tensors the SSD takes: x_out [B,L,d_in], b_out [B,L,gn], c_out [B,L,gn].  weight [C,4]: tap k
 *   multiplies the input 3-k tokens back (torch.nn.Conv1d(groups=C, padding=3) cut to the first L outputs);
 *   bias [C] may be null. */
int ssd_block_rmsnorm_fwd(const float* x, long long x_stride, const float* z, long long z_stride, const float* w,
                          float* out, long long rows, int d, float eps, ssd_stream_t stream);
int ssd_block_conv_silu_fwd(const float* xbc, long long row_stride, const float* weight, const float* bias,
                            float* x_out, float* b_out, float* c_out, int batch, int seqlen, int d_in, int gn,
                            ssd_stream_t stream);

/* ---------------------------------------------------------------- forward without any allocation
 *
 * No counterpart in the reference (its host functions allocate outputs and workspace through the
 * framework allocator, mamba_ascendc/csrc/utils/torch_aclnn_helper.h:526-546).
 *
 * For callers that may not allocate device memory at call time (memory plan fixed at start-up, no
 * caching allocator, a host runtime that owns all allocations): the whole forward pass
 * (ssd_dt_cumsum, ssd_chunk_state mode 0, ssd_state_passing_fwd, ssd_chunk_scan_fwd) with its three
 * temporaries (q, cs, per-tile states) in a fixed 64 MiB array inside the library's device image.
 * The caller passes only inputs, outputs (final_state may be null) and the status word.
 *
 *  - Limit: 2 * align256(4*B*H*L) + 4*B*H*(L/128)*P*N <= ssd_static_scratch_bytes(); larger problems
 *    return SSD_ERR_STATIC_SCRATCH and launch nothing.
 *  - Every GPU that loads the library holds the array until the process exits.
 *  - The first call on each device looks the array's address up (cudaGetSymbolAddress); make that
 *    first call outside any stream capture.
 *  - All calls share the array: calls that overlap on one GPU race.  It needs no clearing between calls.
 *  - Calls no cudaMalloc, cudaFree or allocating library routine.
 *  - Basic path only: no dt_bias and no initial state (use the staged entry points for those); dt_min,
 *    dt_max and valid_len of the shape are honoured.
 *  - The device that owns `out` must be the current device (checked: SSD_ERR_UNSUPPORTED otherwise), since
 *    the scratch address is the current device's.
 *  - Pointer alignment (16 bytes for x, bm, cm, out) is checked before the first stage; an error code from
 *    these checks means nothing was launched.  A launch failure reported by a later stage (SSD_ERR_LAUNCH)
 *    can leave earlier stages enqueued; they only write the scratch array and the outputs. */
size_t ssd_static_scratch_bytes(void);
int ssd_forward_static(const SsdShape* shape, const float* x, const float* dt, const float* A, const float* bm,
                       const float* cm, float* out, float* final_state, int* status, ssd_stream_t stream);

/* ---------------------------------------------------------------- test hooks
 *
 * The two entry points below exist for the test suite only (source: csrc/ssd_selftest.cu); a library built with
 * `build.py --product-only` does not export them. */

/* Tile-level check of the tensor-core path: D[128,n] = A * B^T with K = 128,
 * fp32 in, split-bf16 tcgen05 MMAs, fp32 out.  a_mn / b_mn select whether the
 * operand is given as [rows = non-contracted index, cols = k] (0) or as
 * [rows = k, cols = non-contracted index] (1); inplace = 1 loads the tiles straight
 * into operand-tile memory and splits them in place instead of going through a staging slab.  `status` is a device int the
 * kernel sets non-zero if a bounded wait gave up.  Test-only; no counterpart
 * in the reference (its analogue is the Cube matmul unit,
 * mamba_ascendc_ops/mamba2_ssd_chunk_mix/op_kernel/mamba2_dynamic_matmul.h:195-233). */
int ssd_selftest_umma(const float* a, const float* b, float* d, int n, int a_mn, int b_mn, int inplace, int* status,
                      ssd_stream_t stream);

/* Test-only: one warp waits on a barrier that nothing ever completes, with no copy and no tensor-core
 * instruction in flight; after `polls` polls (1..65536, about a microsecond each) the wait gives up, stores
 * code 1 in *status and the kernel ends normally.  Exercises the give-up path of every bounded wait in the
 * library without disturbing the GPU.  No counterpart in the reference. */
int ssd_selftest_wait_expiry(int* status, int polls, ssd_stream_t stream);

/* Test hook, host only: the first `count` (head, tile) positions that CTA `cta` of a persistent kernel launched
 * with `grid` CTAs visits, as 4 ints each (group, head, first token of the tile, (batch, head, tile) index), computed
 * with the same incremental, division-free arithmetic the kernels use.  tests/ compare it with the closed form.
 * No counterpart in the reference. */
int ssd_selftest_tile_walk(const SsdShape* shape, int grid, int cta, int count, int* out);

#ifdef __cplusplus
}
#endif

#endif /* SSD_B200_H_ */
