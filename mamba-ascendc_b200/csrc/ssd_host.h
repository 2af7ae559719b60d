// Host-side helpers shared by the launchers: error codes, the shape record,
// tensor-map construction for fp32 tiles and launch-error translation.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/ssd_b200.h"

namespace ssd {

// Tensor map over fp32 data for TMA tile loads with 128-byte swizzle.
// dims/box are innermost first; strides_bytes has rank-1 entries (stride of
// dims[1], dims[2], ...).  The innermost box extent must be 32 floats.
// A map depends only on the base address and the geometry, so encoded maps are kept in a small
// process-wide table and reused by later calls on the same buffers (a training loop whose allocator hands
// out the same blocks every step never encodes again).
int make_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box);

// 2-D row-major fp32 matrix [rows x cols], box = [box_rows x 32].
inline int make_tmap_f32_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    const uint64_t dims[2] = {cols, rows};
    const uint64_t strides[1] = {cols * sizeof(float)};
    const uint32_t box[2] = {32u, box_rows};
    return make_tmap_f32(map, base, 2, dims, strides, box);
}

// Token-major activation [tokens, heads, width] (x, dout, out: width = P; B, C:
// heads = G, width = N); box = 32 floats of one head for `box_rows` tokens.
inline int make_tmap_f32_tokens(CUtensorMap* map, const void* base, uint64_t tokens, uint64_t heads, uint64_t width,
                                uint32_t box_rows) {
    const uint64_t dims[3] = {width, heads, tokens};
    const uint64_t strides[2] = {width * sizeof(float), heads * width * sizeof(float)};
    const uint32_t box[3] = {32u, 1u, box_rows};
    return make_tmap_f32(map, base, 3, dims, strides, box);
}

// Index of the current device, or -1.
int current_device();

// SMs of the current device (the grid size of the persistent kernels); 0 on error.  Looked up once per device.
int sm_count();

// Raise a kernel's dynamic shared-memory limit once per device (the attribute belongs to the function in
// each device's context); `done` is the launcher's own bit set, one bit per device.
int set_max_smem_once(const void* func, size_t bytes, std::atomic<uint64_t>& done);

inline int launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SSD_OK : SSD_ERR_LAUNCH;
}

}  // namespace ssd
