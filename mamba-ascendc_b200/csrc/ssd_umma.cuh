// Blackwell (sm_100a) building blocks shared by the SSD tile kernels:
// mbarrier waits with an iteration limit, TMA tile loads, tcgen05 MMA issue,
// TMEM allocation / loads, and the fp32 -> (bf16 hi, bf16 lo) operand split.
//
// Operand tiles in shared memory use ONE physical layout for everything:
// "rows x 64-element column blocks", 128 bytes per row, 128-byte swizzle
// (16-byte chunk index XOR (row & 7)), 8-row groups 1024 bytes apart, column
// blocks `rows * 128` bytes apart.  The same bytes are a K-major operand when
// the contraction runs along the columns and an MN-major operand when it runs
// along the rows; only the matrix descriptor differs.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ssd {

// A wait gives up after this many polls, records a code in the status word and
// lets the kernel run to its end (TMEM is still released).
constexpr uint32_t kSpinLimit = 1u << 21;
#ifndef SSD_WAIT_HINT_NS
#define SSD_WAIT_HINT_NS 1000
#endif
constexpr uint32_t kWaitHintNs = SSD_WAIT_HINT_NS;  // suspend-time hint of one poll

enum StatusCode : int {
    kStatusOk = 0,
    kStatusTmaTimeout = 1,
    kStatusMmaTimeout = 2,
    kStatusSmemAlign = 3,  // the dynamic shared memory did not start on a 1024-byte boundary
};
// The low four bits of a status word say what kind of wait gave up; the bits above locate it, for
// diagnosis: source file (1 ssd_chunk_state, 2 ssd_state_scan, 3 ssd_chunk_scan, 4 ssd_bwd_dx, 5 ssd_bwd_dbc,
// 6 ssd_selftest) in bits 12 and up, the number of the wait inside that file, in source order, in bits 4-11.
__host__ __device__ constexpr int wait_site(int file, int n) { return (file << 12) | (n << 4); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread (up to about a microsecond, woken
// as soon as the phase completes) instead of returning at once: waiting warps then leave the issue
// slots of their scheduler to the warps that still have work.
// Plain arrival (release at CTA scope: the arriving thread's earlier shared-memory writes are visible to
// a thread that has waited on the phase).
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait.  `status` is a device-global int; once any CTA has set it the
// remaining waits everywhere stop polling early.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          uint32_t limit = kSpinLimit) {
#pragma unroll 1
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *reinterpret_cast<volatile int*>(status) != 0) break;
    }
    atomicCAS(status, 0, code);
    return false;
}

// ---------------------------------------------------------------- register budget
// Warp groups (4 consecutive warps) of one CTA trade registers: the group that only issues
// instructions gives most of its share back, the computing groups take it.  Every warp of the group
// executes the instruction; N is a multiple of 8.
template <uint32_t N>
__device__ __forceinline__ void reg_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <uint32_t N>
__device__ __forceinline__ void reg_acquire() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------- fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    // generic-proxy writes to shared memory become visible to the async proxy
    // (tcgen05.mma operand reads, TMA stores)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
            "r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Tile stores shared -> global.  The writer threads fence (fence_proxy_async_smem) and synchronise
// first; one thread issues the store, commits the group and, before the shared memory is reused,
// waits until the engine has finished READING it.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------- TMEM
// One full warp allocates `cols` (power of two, >= 32) columns; the base
// address lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane
// (lane-quarter base + i); `taddr` carries that lane base in bits [31:16].
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// Same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Same for 8 consecutive columns.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Registers -> TMEM: thread i of the warp writes 16 consecutive 32-bit columns of lane (base + i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// The same for 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- MMA
// 64-bit shared-memory matrix descriptor, 128-byte swizzle, sm_100 version.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand read from tensor memory: row m of A in lane m, two bf16 contraction
// elements per 32-bit column (element 2c in the low half of column c), 8 columns per instruction.
__device__ __forceinline__ void umma_bf16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// One operand of a split-precision GEMM: two tiles (hi, lo) in the layout
// described at the top of this file.
struct Operand {
    uint32_t hi;          // shared-memory address of the hi tile (1024-byte aligned)
    uint32_t lo;          // shared-memory address of the lo tile
    uint32_t rows;        // rows of the tile (row pitch is always 128 bytes)
    bool mn_major;        // contraction runs along the rows
    uint32_t blk = 0;     // distance between 64-element column blocks in bytes; 0 = rows * 128
    __device__ __forceinline__ uint32_t block_stride() const { return blk ? blk : rows * 128u; }
};

// Byte offset of the 16-element contraction step `s` inside an operand tile.
__device__ __forceinline__ constexpr uint32_t kstep_offset(uint32_t blk, bool mn_major, int s) {
    // MN-major: 16 rows per step.  K-major: four 32-byte steps per 64-element column block.
    return mn_major ? static_cast<uint32_t>(s) * 2048u
                    : static_cast<uint32_t>(s >> 2) * blk + static_cast<uint32_t>(s & 3) * 32u;
}
// Descriptor of step 0; later steps only add (offset >> 4) to the low word.
__device__ __forceinline__ uint64_t operand_desc0(uint32_t base, uint32_t blk, bool mn_major) {
    // MN-major: 8-row groups 1024 B apart (SBO), 64-wide column blocks `blk` bytes apart (LBO).
    // K-major: 8-row groups 1024 B apart (SBO); LBO is not used with swizzling.
    return mn_major ? make_smem_desc(base, blk, 1024u) : make_smem_desc(base, 16u, 1024u);
}

// D[128 x N] (+)= A * B^T over KSTEPS 16-element steps, three MMAs per step:
// hi*hi + lo*hi + hi*lo.  `a_off`/`b_off` are byte offsets added to both tile
// bases (to select a row range of a K-major tile or a column block of an
// MN-major tile).  Issued by ONE thread; the loops are unrolled so that each
// MMA costs that thread one add per descriptor.
//
// Order matters for accuracy: the tensor core truncates when it adds a product
// block to the fp32 accumulator (measured: about -3e-7 relative per 24 MMAs on
// same-sign data).  The two correction products are 2^-8 of the result, so all
// of them go first, while the accumulator is still small and their truncation
// is negligible; only the KSTEPS hi*hi MMAs then add at full magnitude.
template <int KSTEPS>
__device__ __forceinline__ void issue_gemm_split(uint32_t d_tmem, const Operand& a, uint32_t a_off, const Operand& b,
                                                 uint32_t b_off, uint32_t idesc, bool accumulate) {
    const uint32_t ablk = a.block_stride(), bblk = b.block_stride();
    const uint64_t ah0 = operand_desc0(a.hi + a_off, ablk, a.mn_major);
    const uint64_t al0 = operand_desc0(a.lo + a_off, ablk, a.mn_major);
    const uint64_t bh0 = operand_desc0(b.hi + b_off, bblk, b.mn_major);
    const uint64_t bl0 = operand_desc0(b.lo + b_off, bblk, b.mn_major);
    uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t ao = kstep_offset(ablk, a.mn_major, s) >> 4;
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16(d_tmem, al0 + ao, bh0 + bo, idesc, acc);
        umma_bf16(d_tmem, ah0 + ao, bl0 + bo, idesc, 1u);
        acc = 1u;
    }
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t ao = kstep_offset(ablk, a.mn_major, s) >> 4;
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16(d_tmem, ah0 + ao, bh0 + bo, idesc, 1u);
    }
}

// The same three-product scheme with A (hi and lo, K-major) resident in tensor memory.
template <int KSTEPS>
__device__ __forceinline__ void issue_gemm_split_ta(uint32_t d_tmem, uint32_t a_hi_tmem, uint32_t a_lo_tmem,
                                                    const Operand& b, uint32_t b_off, uint32_t idesc, bool accumulate) {
    const uint32_t bblk = b.block_stride();
    const uint64_t bh0 = operand_desc0(b.hi + b_off, bblk, b.mn_major);
    const uint64_t bl0 = operand_desc0(b.lo + b_off, bblk, b.mn_major);
    uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16_ta(d_tmem, a_lo_tmem + 8u * s, bh0 + bo, idesc, acc);
        umma_bf16_ta(d_tmem, a_hi_tmem + 8u * s, bl0 + bo, idesc, 1u);
        acc = 1u;
    }
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16_ta(d_tmem, a_hi_tmem + 8u * s, bh0 + bo, idesc, 1u);
    }
}

// Variant for an N <= 128 product whose B operand has its lo tile right behind its hi tile as the next
// block along N (K-major: the following rows; MN-major: the following column block, i.e. lo - hi ==
// block stride).  One MMA of width 2N then yields [A_hi*B_hi^T | A_hi*B_lo^T] at once; the accumulator
// takes 2N columns (main | correction) that the epilogue adds.  Two MMAs per step instead of three, and
// wide ones run at twice the efficiency of N = 64.  The hi*hi terms enter first here, so use it where
// 1e-7 relative truncation effects do not matter.
template <int KSTEPS>
__device__ __forceinline__ void issue_gemm_split_wide(uint32_t d_tmem, const Operand& a, const Operand& b,
                                                      uint32_t idesc_2n, uint32_t idesc_n, bool accumulate) {
    const uint32_t ablk = a.block_stride(), bblk = b.block_stride();
    const uint64_t ah0 = operand_desc0(a.hi, ablk, a.mn_major);
    const uint64_t al0 = operand_desc0(a.lo, ablk, a.mn_major);
    const uint64_t bh0 = operand_desc0(b.hi, bblk, b.mn_major);
    uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t ao = kstep_offset(ablk, a.mn_major, s) >> 4;
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16(d_tmem, ah0 + ao, bh0 + bo, idesc_2n, acc);
        acc = 1u;
    }
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
        const uint64_t ao = kstep_offset(ablk, a.mn_major, s) >> 4;
        const uint64_t bo = kstep_offset(bblk, b.mn_major, s) >> 4;
        umma_bf16(d_tmem, al0 + ao, bh0 + bo, idesc_n, 1u);
    }
}

// ---------------------------------------------------------------- operand split
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);  // a -> low half, b -> high half
    return *reinterpret_cast<uint32_t*>(&v);
}
// v = hi + lo with hi, lo in bf16 (16 mantissa bits kept in total).
__device__ __forceinline__ void split8(const float* v, uint4& hi, uint4& lo) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        h[i] = pack_bf16x2(a, b);
        const float ah = __uint_as_float(h[i] << 16);
        const float bh = __uint_as_float(h[i] & 0xFFFF0000u);
        l[i] = pack_bf16x2(a - ah, b - bh);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}
// 32 consecutive values of one row -> 16 packed bf16 pairs of hi parts and 16 of lo parts, the form in
// which a row of an A operand is written to tensor memory (tmem_st16).
__device__ __forceinline__ void split32_packed(const float* v, uint32_t* hi, uint32_t* lo) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        hi[i] = pack_bf16x2(a, b);
        lo[i] = pack_bf16x2(a - __uint_as_float(hi[i] << 16), b - __uint_as_float(hi[i] & 0xFFFF0000u));
    }
}
// The same for 16 consecutive values (8 packed pairs each, tmem_st8).
__device__ __forceinline__ void split16_packed(const float* v, uint32_t* hi, uint32_t* lo) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        hi[i] = pack_bf16x2(a, b);
        lo[i] = pack_bf16x2(a - __uint_as_float(hi[i] << 16), b - __uint_as_float(hi[i] & 0xFFFF0000u));
    }
}
// Byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside one column block.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t chunk) { return r * 128u + ((chunk ^ (r & 7u)) << 4); }

// Store 8 consecutive values of row r starting at tile column `col` (multiple of 8).
__device__ __forceinline__ void store_split8(uint8_t* hi_tile, uint8_t* lo_tile, uint32_t rows, uint32_t r,
                                             uint32_t col, const float* v) {
    uint4 h, l;
    split8(v, h, l);
    const uint32_t off = (col >> 6) * rows * 128u + swz(r, (col & 63u) >> 3);
    *reinterpret_cast<uint4*>(hi_tile + off) = h;
    *reinterpret_cast<uint4*>(lo_tile + off) = l;
}

// A staged fp32 slab is what one TMA box of 32 floats x `rows` rows leaves in
// shared memory with 128-byte swizzle.  Convert it into columns
// [col0, col0 + 32) of an operand tile, multiplying row r by scale[r] when
// `scale` is not null.  Lanes run along rows, so loads and stores are free of
// bank conflicts.
__device__ __forceinline__ void convert_slab(const uint8_t* stage, uint8_t* hi_tile, uint8_t* lo_tile, uint32_t rows,
                                             uint32_t col0, const float* scale, int tid, int nthreads) {
    for (uint32_t item = tid; item < rows * 4u; item += nthreads) {
        const uint32_t r = item % rows, j = item / rows;
        const float4 a = *reinterpret_cast<const float4*>(stage + swz(r, 2 * j));
        const float4 b = *reinterpret_cast<const float4*>(stage + swz(r, 2 * j + 1));
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (scale != nullptr) {
            const float s = scale[r];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= s;
        }
        store_split8(hi_tile, lo_tile, rows, r, col0 + 8 * j, v);
    }
}

}  // namespace ssd
