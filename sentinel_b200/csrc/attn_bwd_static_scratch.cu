// Backward entry point for callers that are not able to allocate device memory.
//
// Who this is for: code that runs where a device allocation is impossible or forbidden -- a plugin called from
// inside somebody else's CUDA-graph capture or from a latency-critical loop whose owner bans cudaMalloc (it
// serialises the device and may fail late), a host process that has handed all of its memory to a pool it does not
// control, or a binding that simply has no allocator to lend.  The normal entry point, sntl_attn_bwd, needs the
// caller to bring a scratch buffer; this one brings its own.
//
// How: the scratch (delta, LSE*log2e and the fp32 dQ accumulator, or just delta on the exact-fp32 route) lives in
// a fixed array in device global memory that is part of the library image.  Its size, kStaticScratchBytes, is the
// limit: a problem whose sntl_attn_bwd_workspace_bytes() is larger is refused with SNTL_ERR_SCRATCH_LIMIT and
// nothing is launched.  Every GPU on which this library is loaded carries the array until the process exits.
//
// Rules of use
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress, once per
//     device, with that device current).  Make that first call eagerly, before any stream capture begins.
//   * All calls on one device share the one array, and it still holds whatever the previous call left there.  The
//     backward itself rewrites every word it later reads (its first pass stores delta and LSE*log2e and clears the
//     dQ accumulator), so nothing has to be cleared by the caller.
//   * For the same reason two calls whose kernels can be in flight together on one GPU (different streams, or two
//     host threads) race on the array and corrupt each other's gradients.  Keep such calls on one stream, or order
//     them with events.
//   * Nothing here calls cudaMalloc, cudaFree or any routine that allocates.
#include <mutex>

#include <cuda_runtime.h>

#include "sntl_attn.h"

namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;   // 32 MiB per device

// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the array on the current device; resolved once per device.
int static_scratch_pointer(void** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return SNTL_ERR_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return SNTL_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return SNTL_ERR_CUDA;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return SNTL_OK;
}

}  // namespace

extern "C" {

size_t sntl_attn_static_scratch_capacity(void) { return kStaticScratchBytes; }

int sntl_attn_bwd_static_scratch(const sntl_attn_desc* desc, const void* q, const void* k, const void* v, const void* o,
                                 const float* lse, const void* dout, void* dq, void* dk, void* dv, void* stream)
{
    if (!desc) return SNTL_ERR_BAD_ARGUMENT;
    const size_t need = sntl_attn_bwd_workspace_bytes(desc);
    if (need == 0)  // the descriptor does not validate: let the normal entry point name the reason (it launches nothing)
        return sntl_attn_bwd(desc, q, k, v, o, lse, dout, dq, dk, dv, nullptr, 0, stream);
    if (need > kStaticScratchBytes) return SNTL_ERR_SCRATCH_LIMIT;
    void* scratch = nullptr;
    const int rc = static_scratch_pointer(&scratch);
    if (rc != SNTL_OK) return rc;
    return sntl_attn_bwd(desc, q, k, v, o, lse, dout, dq, dk, dv, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
