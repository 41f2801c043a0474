// sihc_read_bwd_static: the read's backward pass for callers that cannot allocate device memory.
//
// Who needs this: a host that gave every byte of the GPU to its own memory plan at
// start-up (an inference server with a fixed arena, an embedded or safety-certified
// runtime whose memory map is frozen after initialisation), or a caller on a
// latency-critical thread that must not hit the device-wide synchronisation a
// cudaMalloc / cudaFree can imply.  Such a caller has nowhere to get the scratch
// buffer that sihc_read_bwd asks for, and no allocator to ask.
//
// What it does instead: the per-block partial sums of the weight gradient go into
// one fixed array that lives inside this library's device image.  The array is
// part of the module, so every GPU that loads the library carries its
// SIHC_STATIC_SCRATCH_BYTES (16 MiB) from load until the process exits, whether or
// not this entry point is ever called.
//
// The array's name below is only a handle in host code, not a device address; the
// address used by the kernels comes from cudaGetSymbolAddress, asked once per device
// (with that device current) on the first call made on that device.  That first call
// may also trigger the lazy loading of the module, so it should be made before any
// stream capture is started on that device.  No call here reaches cudaMalloc, cudaFree
// or an allocating library routine.
//
// Sharing: there is exactly one array per device.  Calls that may overlap on the
// GPU (different streams, different host threads) race on it and must be serialised
// by the caller.  Nothing in the array has to start at zero - every block overwrites
// all of its rows before the finishing pass reads them - and what the last call left
// behind is never read, so no clearing is done or needed.
#include "sihc_b200.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[SIHC_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices];   // device address of g_static_scratch, per device; null = not looked up yet

// Resolve the device address of the scratch array for the current device (once per device).
int static_scratch(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return SIHC_ERR_CAPACITY;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);   // device `dev` is current here
        if (e != cudaSuccess) return static_cast<int>(e);
        if (ptr == nullptr) return SIHC_ERR_WORKSPACE;
        g_scratch_address[dev] = ptr;
    }
    *out = g_scratch_address[dev];
    return SIHC_OK;
}

}  // namespace

extern "C" int sihc_read_bwd_static(const void* x, const void* const* g, const void* alpha, void* dx, float* dalpha,
                                    int events, int64_t batch, int grid, int kh, int kw, int channels, int dtype,
                                    int wdtype, void* stream) {
    // Size check first: nothing is launched and no pointer is touched when the case does not fit.
    if (dalpha != nullptr) {
        const size_t need = sihc_wgrad_workspace_bytes(events, batch, grid, kh, kw, channels, dtype);
        if (need > static_cast<size_t>(SIHC_STATIC_SCRATCH_BYTES)) return SIHC_ERR_CAPACITY;
    }
    void* scratch = nullptr;
    if (int st = static_scratch(&scratch)) return st;
    return sihc_read_bwd(x, g, alpha, dx, dalpha, scratch, static_cast<size_t>(SIHC_STATIC_SCRATCH_BYTES), events, batch,
                         grid, kh, kw, channels, dtype, wdtype, stream);
}
