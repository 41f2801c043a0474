// Compile-time dispatch helpers: runtime (dtype, wdtype, S, V, TT) -> template instantiation.
#pragma once

#include <type_traits>

#include "sihc_launch.h"

namespace sihc {

// Channels per thread on the vector path.  16-byte accesses wherever the
// S*V per-thread coefficient/accumulator footprint stays within 32 registers.
template <typename T, int S> struct VecWidth {
    static constexpr int kFull = 16 / int(sizeof(T));
    static constexpr int kCap = 32 / S;
    static constexpr int value = kFull < kCap ? kFull : kCap;
};
inline int vec_width(DType dtype, int S) {
    const int full = dtype == kBF16 ? 8 : 4;
    const int cap = S > 0 ? 32 / S : full;
    return full < cap ? full : cap;
}

// Single-event forward kernels hold one coefficient set and no accumulators: they can afford twice the
// per-thread footprint (S*V <= 64), i.e. full 16-byte vectors up to n = 8 and 8-byte vectors at n = 16.
template <typename T, int S> struct VecWidthFwd {
    static constexpr int kFull = 16 / int(sizeof(T));
    static constexpr int kCap = 64 / S;
    static constexpr int value = kFull < kCap ? kFull : kCap;
};
inline int vec_width_fwd(DType dtype, int S) {
    const int full = dtype == kBF16 ? 8 : 4;
    const int cap = S > 0 ? 64 / S : full;
    return full < cap ? full : cap;
}

template <int N> using Int = std::integral_constant<int, N>;

// f(T tag, W tag): (fp32,fp32), (bf16,bf16), (bf16,fp32)
template <typename F>
inline cudaError_t dispatch_types(DType dtype, DType wdtype, F&& f) {
    if (dtype == kF32) return f(float{}, float{});
    if (wdtype == kBF16) return f(bf16_t{}, bf16_t{});
    return f(bf16_t{}, float{});
}

template <typename F>
inline cudaError_t dispatch_slots(int S, F&& f) {
    switch (S) {
        case 2: return f(Int<2>{});
        case 4: return f(Int<4>{});
        case 8: return f(Int<8>{});
        case 16: return f(Int<16>{});
        default: return cudaErrorInvalidValue;
    }
}

// f(V tag, TT tag): vector path with TT in {1,2,4}, scalar path with TT = 1.
template <int VMAX, typename F>
inline cudaError_t dispatch_vec_tt(int V, int tt, F&& f) {
    if (V == 1 || VMAX == 1) return f(Int<1>{}, Int<1>{});
    if (tt >= 4) return f(Int<VMAX>{}, Int<4>{});
    if (tt >= 2) return f(Int<VMAX>{}, Int<2>{});
    return f(Int<VMAX>{}, Int<1>{});
}

// Fill the tiling and launch a persistent kernel; returns the x-grid used.
template <typename K, typename P>
inline cudaError_t launch_persistent(K kernel, P& params, const Problem& pb, int V, int TT, int default_threads,
                                     uint32_t gz, bool emits_partials, uint32_t* gx_out, int max_threads = kMaxThreads) {
    const Tuning& tn = tuning();
    const uint32_t ncv = pb.C / static_cast<uint32_t>(V);
    const BlockShape bs = block_shape(ncv, tn.threads > 0 ? tn.threads : default_threads, max_threads);
    Tiling& t = params.t;
    t.M = pb.M; t.g = pb.g; t.C = pb.C; t.ncv = ncv; t.cl = bs.cl; t.tl = bs.tl;
    const uint32_t per_tile = bs.tl * static_cast<uint32_t>(TT);
    t.ntiles = (pb.M + per_tile - 1) / per_tile;
    int nb = occupancy_blocks(kernel, static_cast<int>(bs.threads));
    uint32_t gx;
    if (emits_partials) {
        const int cap = tn.rbps > 0 ? tn.rbps : 2;
        if (nb > cap) nb = cap;
        gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / (bs.gy * gz);
        const uint32_t bound = partial_blocks_bound(pb.M);
        if (gx > bound) gx = bound;
    } else {
        if (tn.bps > 0 && nb > tn.bps) nb = tn.bps;
        gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / (bs.gy * gz);
    }
    if (gx < 1) gx = 1;
    if (gx > t.ntiles) gx = t.ntiles;
    if (gx_out) *gx_out = gx;
    kernel<<<dim3(gx, bs.gy, gz), bs.threads, 0, pb.stream>>>(params);
    count_launch();
    return cudaGetLastError();
}

// Variant for kernels that stage their loads in dynamic shared memory, `smem_per_thread` bytes per thread.
// The block is shrunk (fewer token lanes) until its ring fits the 227 KB a block may use.
template <typename K, typename P>
inline cudaError_t launch_persistent_smem(K kernel, P& params, const Problem& pb, int V, int default_threads,
                                          size_t smem_per_thread, bool emits_partials, uint32_t* gx_out,
                                          int max_threads = kMaxThreads, uint32_t min_token_lanes = 1) {
    constexpr size_t kMaxDynamic = 200 * 1024;     // leaves room for the static reduction buffer
    const Tuning& tn = tuning();
    const uint32_t ncv = pb.C / static_cast<uint32_t>(V);
    BlockShape bs = block_shape(ncv, tn.threads > 0 ? tn.threads : default_threads, max_threads);
    // A kernel whose speed comes from token-level parallelism (many warps each walking its own tokens) can ask for a
    // minimum number of token lanes: the channel vectors are then split evenly over blockIdx.y until they fit.
    for (uint32_t parts = 2; bs.tl < min_token_lanes && parts <= 8 && ncv / parts >= 16; ++parts) {
        if (ncv % parts != 0) continue;
        BlockShape alt = block_shape(ncv / parts, tn.threads > 0 ? tn.threads : default_threads, max_threads);
        alt.gy = parts;
        if (alt.tl > bs.tl) bs = alt;
    }
    while (bs.tl > 1 && static_cast<size_t>(bs.threads) * smem_per_thread > kMaxDynamic) { --bs.tl; bs.threads = bs.cl * bs.tl; }
    const size_t smem = static_cast<size_t>(bs.threads) * smem_per_thread;
    if (smem > kMaxDynamic) return cudaErrorInvalidConfiguration;
    if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxDynamic)) return e;
    Tiling& t = params.t;
    t.M = pb.M; t.g = pb.g; t.C = pb.C; t.ncv = ncv; t.cl = bs.cl; t.tl = bs.tl;
    t.ntiles = (pb.M + bs.tl - 1) / bs.tl;          // one token per thread per ring stage
    int nb = cached_occupancy(reinterpret_cast<const void*>(kernel), static_cast<int>(bs.threads), smem);
    uint32_t gx;
    if (emits_partials) {
        const int cap = tn.rbps > 0 ? tn.rbps : 2;
        if (nb > cap) nb = cap;
        gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / bs.gy;
        const uint32_t bound = partial_blocks_bound(pb.M);
        if (gx > bound) gx = bound;
    } else {
        if (tn.bps > 0 && nb > tn.bps) nb = tn.bps;
        gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / bs.gy;
    }
    if (gx < 1) gx = 1;
    if (gx > t.ntiles) gx = t.ntiles;
    if (gx_out) *gx_out = gx;
    kernel<<<dim3(gx, bs.gy, 1), bs.threads, smem, pb.stream>>>(params);
    count_launch();
    return cudaGetLastError();
}

}  // namespace sihc
