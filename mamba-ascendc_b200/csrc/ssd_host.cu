// Host-side utilities of libssd_b200: tensor-map construction, error strings
// and the shape validation every entry point runs before launching.
#include "ssd_host.h"

#include <mutex>

namespace ssd {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up once; this is the only process-wide
// state the library keeps.
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

}  // namespace

int make_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return SSD_ERR_TENSORMAP;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return SSD_ERR_ALIGN;
    cuuint64_t gdim[5];
    cuuint64_t gstride[4];
    cuuint32_t gbox[5];
    cuuint32_t estride[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        gbox[i] = box[i];
        estride[i] = 1;
        if (i > 0) gstride[i - 1] = strides_bytes[i - 1];
    }
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, static_cast<cuuint32_t>(rank),
                          const_cast<void*>(base), gdim, gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? SSD_OK : SSD_ERR_TENSORMAP;
}

}  // namespace ssd

extern "C" const char* ssd_error_string(int code) {
    switch (code) {
        case SSD_OK: return "ssd: ok";
        case SSD_ERR_NULL: return "ssd: a required tensor pointer is null";
        case SSD_ERR_SHAPE:
            return "ssd: all dimensions must be positive, nheads must be divisible by ngroups and tile must be positive";
        case SSD_ERR_UNSUPPORTED:
            return "ssd: unsupported shape (need headdim == 64, dstate in {64, 128}, tile == 128, seqlen % 128 == 0)";
        case SSD_ERR_WORKSPACE: return "ssd: workspace too small";
        case SSD_ERR_ALIGN: return "ssd: tensor base addresses must be 16-byte aligned";
        case SSD_ERR_TENSORMAP: return "ssd: the CUDA driver rejected a TMA tensor map";
        case SSD_ERR_LAUNCH: return "ssd: kernel launch failed";
        case SSD_ERR_STATIC_SCRATCH:
            return "ssd: problem needs more scratch than the 64 MiB built into ssd_forward_static; use the staged entry "
                   "points with caller-allocated buffers";
        default: return "ssd: unknown error code";
    }
}

extern "C" int ssd_check_shape(const SsdShape* s) {
    if (s == nullptr) return SSD_ERR_NULL;
    if (s->batch <= 0 || s->seqlen <= 0 || s->nheads <= 0 || s->headdim <= 0) return SSD_ERR_SHAPE;
    if (s->dstate <= 0 || s->ngroups <= 0 || s->tile <= 0) return SSD_ERR_SHAPE;
    if (s->nheads % s->ngroups != 0) return SSD_ERR_SHAPE;
    if (!(s->dt_min <= s->dt_max)) return SSD_ERR_SHAPE;
    if (s->valid_len < 0 || s->valid_len > s->seqlen) return SSD_ERR_SHAPE;
    if (s->headdim != 64) return SSD_ERR_UNSUPPORTED;
    if (s->dstate != 64 && s->dstate != 128) return SSD_ERR_UNSUPPORTED;
    if (s->tile != 128 || s->seqlen % s->tile != 0) return SSD_ERR_UNSUPPORTED;
    return SSD_OK;
}
