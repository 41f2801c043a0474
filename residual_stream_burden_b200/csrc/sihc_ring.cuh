// `cp.async` wrappers and the per-thread ring addressing shared by the kernels that stage loads in shared memory.
#pragma once

#include "sihc_common.cuh"

namespace sihc {

template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem, const void* gmem, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int src_bytes = valid ? BYTES : 0;       // 0 source bytes = fill the slot with zeros, no global read
    if constexpr (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(src_bytes) : "memory");
    else if constexpr (BYTES == 8)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(gmem), "r"(src_bytes) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Ring addressing: [stage][vector index][thread], one Raw per entry (conflict-free for a warp).
template <typename Raw>
struct Ring {
    Raw* base;
    uint32_t nthreads, tid;
    int nvec;
    __device__ __forceinline__ Raw* slot(int stage, int j) const {
        return base + (static_cast<size_t>(stage) * nvec + j) * nthreads + tid;
    }
};

}  // namespace sihc
