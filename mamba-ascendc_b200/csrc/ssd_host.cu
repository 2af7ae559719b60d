// Host-side utilities of libssd_b200: tensor-map construction, error strings
// and the shape validation every entry point runs before launching.
#include "ssd_host.h"

#include <cstdio>
#include <cstdlib>

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

namespace {

// Direct-mapped table of encoded maps.  Key = everything cuTensorMapEncodeTiled reads.
struct TmapKey {
    const void* base;
    uint32_t rank;
    uint64_t dims[3];
    uint64_t strides[2];
    uint32_t box[3];
    bool operator==(const TmapKey& o) const {
        if (base != o.base || rank != o.rank) return false;
        for (int i = 0; i < 3; ++i)
            if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        return strides[0] == o.strides[0] && strides[1] == o.strides[1];
    }
};
struct TmapSlot {
    bool used = false;
    TmapKey key;
    CUtensorMap map;
};
constexpr size_t kTmapSlots = 1024;
TmapSlot g_tmap_table[kTmapSlots];
std::mutex g_tmap_mutex;

size_t tmap_hash(const TmapKey& k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
    h = h * 0x9E3779B97F4A7C15ull + k.dims[0];
    h = h * 0x9E3779B97F4A7C15ull + k.dims[1] + (k.dims[2] << 20);
    h = h * 0x9E3779B97F4A7C15ull + k.box[1] + (static_cast<uint64_t>(k.box[2]) << 12) + k.rank;
    return static_cast<size_t>((h >> 17) % kTmapSlots);
}

}  // namespace

int make_tmap_f32(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return SSD_ERR_TENSORMAP;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return SSD_ERR_ALIGN;
    if (rank < 2 || rank > 3) return SSD_ERR_TENSORMAP;
    TmapKey key{};
    key.base = base;
    key.rank = static_cast<uint32_t>(rank);
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
    }
    TmapSlot& slot = g_tmap_table[tmap_hash(key)];
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    if (slot.used && slot.key == key) {
        *map = slot.map;
        return SSD_OK;
    }
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
    // The encoder is a DRIVER entry point and wants a context current on the calling thread.  A thread that has
    // made no runtime call yet has none -- e.g. the framework's backward thread on device 0, when its allocations
    // all came out of a cache -- and the driver then answers CUDA_ERROR_INVALID_CONTEXT.  Any runtime call binds
    // the primary context; this path (a map that is not in the table yet) is rare, so it is made every time.
    (void)cudaFree(nullptr);
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, static_cast<cuuint32_t>(rank),
                          const_cast<void*>(base), gdim, gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        // SSD_B200_DEBUG=1: say what the driver answered (an error left behind by an earlier asynchronous fault
        // comes back from this call as well, with a code of its own)
        if (const char* dbg = std::getenv("SSD_B200_DEBUG"); dbg != nullptr && dbg[0] == '1')
            std::fprintf(stderr, "ssd_b200: cuTensorMapEncodeTiled -> %d (base %p, rank %d, dims %llu %llu %llu, box %u %u %u)\n",
                         static_cast<int>(r), base, rank, static_cast<unsigned long long>(key.dims[0]),
                         static_cast<unsigned long long>(key.dims[1]), static_cast<unsigned long long>(key.dims[2]),
                         key.box[0], key.box[1], key.box[2]);
        return SSD_ERR_TENSORMAP;
    }
    slot.used = true;
    slot.key = key;
    slot.map = *map;
    return SSD_OK;
}

int current_device() {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int sm_count() {
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cached[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return 0;
    if (dev < kMaxDevices) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev < kMaxDevices) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

int set_max_smem_once(const void* func, size_t bytes, std::atomic<uint64_t>& done) {
    const int dev = current_device();
    if (dev < 0) return SSD_ERR_LAUNCH;
    const uint64_t bit = dev < 64 ? (uint64_t(1) << dev) : 0;
    if (bit != 0 && (done.load(std::memory_order_acquire) & bit) != 0) return SSD_OK;
    if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) !=
        cudaSuccess) {
        (void)cudaGetLastError();
        return SSD_ERR_LAUNCH;
    }
    if (bit != 0) done.fetch_or(bit, std::memory_order_release);
    return SSD_OK;
}

}  // namespace ssd

extern "C" const char* ssd_error_string(int code) {
    switch (code) {
        case SSD_OK: return "ssd: ok";
        case SSD_ERR_NULL: return "ssd: a required tensor pointer is null";
        case SSD_ERR_SHAPE:
            return "ssd: all dimensions must be positive, nheads must be divisible by ngroups and tile must be positive";
        case SSD_ERR_UNSUPPORTED:
            return "ssd: unsupported problem (need headdim == 64, dstate in {64, 128}, tile == 128, seqlen % 128 == 0; "
                   "ssd_forward_static also needs its outputs on the current device)";
        case SSD_ERR_RANGE:
            return "ssd: size out of range (batch and ngroups at most 65535; batch * seqlen and the number of state rows "
                   "below 2^31)";
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
    // grid.y / grid.z of the tile kernels, and the int32 coordinates of the TMA tile loads
    if (s->batch > 65535 || s->ngroups > 65535) return SSD_ERR_RANGE;
    const int64_t tokens = static_cast<int64_t>(s->batch) * s->seqlen;
    const int64_t state_rows = static_cast<int64_t>(s->batch) * s->nheads * (s->seqlen / s->tile) * s->headdim;
    if (tokens >= (int64_t(1) << 31) || state_rows >= (int64_t(1) << 31)) return SSD_ERR_RANGE;
    return SSD_OK;
}

extern "C" size_t ssd_buffer_bytes(const SsdShape* s, int which) {
    if (ssd_check_shape(s) != SSD_OK) return 0;
    const size_t bh = static_cast<size_t>(s->batch) * s->nheads;
    const size_t k = static_cast<size_t>(s->seqlen / s->tile);
    const size_t pn = static_cast<size_t>(s->headdim) * s->dstate;
    switch (which) {
        case SSD_BUF_Q:
        case SSD_BUF_CS:
        case SSD_BUF_DDT_T: return sizeof(float) * bh * s->seqlen;
        case SSD_BUF_STATES: return sizeof(float) * bh * k * pn;
        case SSD_BUF_FINAL_STATE: return sizeof(float) * bh * pn;
        case SSD_BUF_G_LAST: return sizeof(float) * bh * k;
        case SSD_BUF_DA_PARTIAL: return sizeof(double) * bh * k;
        case SSD_BUF_GATE_PARTIAL: return sizeof(float) * ssd_gate_partial_floats(s);
        case SSD_BUF_STATUS: return sizeof(int32_t);
        default: return 0;
    }
}
