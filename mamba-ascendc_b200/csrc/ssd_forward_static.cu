// Forward pass for callers that must not allocate device memory.
//
// Some hosts of this library hand an operator nothing but raw device pointers
// for its inputs and outputs and forbid allocator calls on the hot path: a
// serving process whose device memory was carved up once at start-up, a
// plug-in that runs without torch's caching allocator (where a cudaMalloc
// would stall the whole device), an embedding in another runtime that owns
// the memory plan.  The staged forward needs three temporaries (q, cs and the
// per-tile states).  Here they live in a fixed array inside the library's
// device image, so this entry point calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
// The price: the array has a fixed size (kStaticScratchBytes, 64 MiB), every
// GPU that loads the library keeps that much memory until the process exits,
// larger problems are rejected, and all calls share the one array: two calls
// that overlap on the same GPU (different streams or threads) race on it.
// Nothing in it has to start at zero -- every element is written by an
// earlier stage of the same call before a later stage reads it -- so stale
// contents of the previous call are harmless.
#include <initializer_list>
#include <mutex>

#include "ssd_host.h"

namespace {

constexpr size_t kStaticScratchBytes = size_t(64) << 20;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime, not a device
// address; the address for the current device comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_ssd_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// First call on a device: look the array's address up once, with that device current.
int scratch_for_current_device(unsigned char** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SSD_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_ssd_static_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return SSD_ERR_LAUNCH;
        }
        g_scratch_addr[dev] = p;
    }
    *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
    return SSD_OK;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

extern "C" size_t ssd_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int ssd_forward_static(const SsdShape* shape, const float* x, const float* dt, const float* A,
                                  const float* bm, const float* cm, float* out, float* final_state, int* status,
                                  ssd_stream_t stream) {
    const int rc0 = ssd_check_shape(shape);
    if (rc0 != SSD_OK) return rc0;
    if (!x || !dt || !A || !bm || !cm || !out || !status) return SSD_ERR_NULL;
    const SsdShape& s = *shape;
    const size_t row_bytes = align256(sizeof(float) * s.batch * s.nheads * static_cast<size_t>(s.seqlen));
    const size_t state_bytes =
        sizeof(float) * s.batch * s.nheads * static_cast<size_t>(s.seqlen / s.tile) * s.headdim * s.dstate;
    if (2 * row_bytes + state_bytes > kStaticScratchBytes) return SSD_ERR_STATIC_SCRATCH;
    // everything a later stage would reject is checked here, before the first launch
    for (const void* p : {static_cast<const void*>(x), static_cast<const void*>(bm), static_cast<const void*>(cm),
                          static_cast<const void*>(out)})
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return SSD_ERR_ALIGN;
    {   // the scratch address below is the current device's: `out` must live there too
        int dev = -1;
        cudaPointerAttributes attr;
        if (cudaGetDevice(&dev) != cudaSuccess) return SSD_ERR_LAUNCH;
        if (cudaPointerGetAttributes(&attr, out) != cudaSuccess) {
            (void)cudaGetLastError();
            return SSD_ERR_UNSUPPORTED;
        }
        if (attr.type != cudaMemoryTypeDevice || attr.device != dev) return SSD_ERR_UNSUPPORTED;
    }
    unsigned char* base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc != SSD_OK) return rc;
    float* q = reinterpret_cast<float*>(base);
    float* cs = reinterpret_cast<float*>(base + row_bytes);
    float* states = reinterpret_cast<float*>(base + 2 * row_bytes);
    rc = ssd_dt_cumsum(shape, dt, nullptr, A, q, cs, stream);
    if (rc == SSD_OK) rc = ssd_chunk_state(shape, x, bm, q, cs, states, 0, status, stream);
    if (rc == SSD_OK) rc = ssd_state_passing_fwd(shape, states, cs, nullptr, final_state, stream);
    if (rc == SSD_OK) rc = ssd_chunk_scan_fwd(shape, x, bm, cm, states, q, cs, out, status, stream);
    return rc;
}
