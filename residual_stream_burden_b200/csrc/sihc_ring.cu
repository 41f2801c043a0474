// Fused single-event adjoints with their loads staged through an asynchronous-copy ring.
//
// The register-staged kernels in sihc_rw.cu issue a tile's loads, wait, compute, store, and only
// then issue the next tile's loads, so a warp's bytes in flight fall to zero once per tile and the
// accumulators (32) + coefficients (32) leave no registers to prefetch a second tile.  Here every
// thread owns NST private 16-byte slots per input vector in shared memory and keeps NST-1 tokens'
// worth of `cp.async` copies in flight at all times; the data never occupies registers while it
// travels.  Slots are private to the issuing thread (it alone reads what it copied), so the ring
// needs no block barrier: `cp.async.wait_group` orders a thread's own copies.
//
// Same results as the register-staged kernels: same per-thread token order, same accumulation order.
#include "sihc_dispatch.cuh"
#include "sihc_ring.cuh"

namespace sihc {

// dx[m,s,c] = alpha[c,s] * g[m,c];  partial[block][s][c] = sum_m X[m,s,c] * g[m,c]
template <typename T, typename W, int S, int V, int NST>
__global__ void __launch_bounds__(kMaxThreads) read_bwd1_ring_kernel(const __grid_constant__ ReadBwd1Params p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    constexpr int VB = int(sizeof(Raw));
    static_assert(VB == 16 || VB == 8 || VB == 4, "ring slots are 4, 8 or 16 bytes");
    extern __shared__ __align__(16) unsigned char ring_bytes[];
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const Ring<Raw> ring{reinterpret_cast<Raw*>(ring_bytes), blockDim.x, threadIdx.x, S + 1};
    const T* __restrict__ x = static_cast<const T*>(p.x) + ln.c0;
    const T* __restrict__ g = static_cast<const T*>(p.g) + ln.c0;
    T* __restrict__ dx = p.dx ? static_cast<T*>(p.dx) + ln.c0 : nullptr;
    const bool want_w = p.partial != nullptr;
    float w1[S][V];
    float acc[S][V];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int v = 0; v < V; ++v) { acc[s][v] = 0.f; w1[s][v] = 0.f; }
    if (ln.active) {
        load_coeffs<W, S, V>(static_cast<const W*>(p.w) + static_cast<size_t>(ln.c0) * S, w1);
        auto issue = [&](uint32_t tile, int stage) {
            const uint32_t m = tile * t.tl + ln.tl;
            const bool ok = tile < t.ntiles && m < t.M;
            const uint32_t mm = ok ? m : 0u;
            const T* cell = x + cell_origin<S>(mm, t.g, t.C);
#pragma unroll
            for (int s = 0; s < S; ++s) cp_async<VB>(ring.slot(stage, s), cell + slot_offset<S>(s, t.g, t.C), ok && want_w);
            cp_async<VB>(ring.slot(stage, S), g + static_cast<size_t>(mm) * t.C, ok);
            cp_async_commit();
        };
        uint32_t tile = blockIdx.x;
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) issue(tile + st * gridDim.x, st);
        int stage = 0;
        for (; tile < t.ntiles; tile += gridDim.x) {
            cp_async_wait<NST - 2>();                       // this tile's copies have landed
            Raw xr[S];
#pragma unroll
            for (int s = 0; s < S; ++s) xr[s] = *ring.slot(stage, s);
            const Raw gr = *ring.slot(stage, S);
            // refill the stage consumed one iteration ago with the tile NST-1 ahead
            issue(tile + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
            const uint32_t m = tile * t.tl + ln.tl;
            const bool ok = m < t.M;
            const size_t origin = cell_origin<S>(ok ? m : 0u, t.g, t.C);
            float gv[V];
            IO::unpack(gr, gv);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                float xv[V];
                float d[V];
                IO::unpack(xr[s], xv);
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    d[v] = w1[s][v] * gv[v];
                    acc[s][v] = fmaf(xv[v], gv[v], acc[s][v]);
                }
                if (dx != nullptr && ok) IO::store(dx + origin + slot_offset<S>(s, t.g, t.C), d);
            }
            stage = stage + 1 == NST ? 0 : stage + 1;
        }
        cp_async_wait<0>();
    }
    if (want_w)
        block_reduce_rows<S, V>(acc, p.partial + static_cast<size_t>(blockIdx.x) * S * t.C, t.C, ln.c0, ln.cl, ln.tl,
                                t.cl, t.tl, ln.active, red);
}

// ddz[m,c] = sum_s beta[c,s] * h[m,s,c];  partial[block][s][c] = sum_m dz[m,c] * h[m,s,c]
template <typename T, typename W, int S, int V, int NST>
__global__ void __launch_bounds__(kMaxThreads) write_bwd1_ring_kernel(const __grid_constant__ WriteBwd1Params p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    constexpr int VB = int(sizeof(Raw));
    extern __shared__ __align__(16) unsigned char ring_bytes[];
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const Ring<Raw> ring{reinterpret_cast<Raw*>(ring_bytes), blockDim.x, threadIdx.x, S + 1};
    const T* __restrict__ h = static_cast<const T*>(p.h) + ln.c0;
    const T* __restrict__ dz = p.dz ? static_cast<const T*>(p.dz) + ln.c0 : nullptr;
    T* __restrict__ ddz = p.ddz ? static_cast<T*>(p.ddz) + ln.c0 : nullptr;
    const bool want_w = p.partial != nullptr && dz != nullptr;
    float w1[S][V];
    float acc[S][V];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int v = 0; v < V; ++v) { acc[s][v] = 0.f; w1[s][v] = 0.f; }
    if (ln.active) {
        load_coeffs<W, S, V>(static_cast<const W*>(p.w) + static_cast<size_t>(ln.c0) * S, w1);
        auto issue = [&](uint32_t tile, int stage) {
            const uint32_t m = tile * t.tl + ln.tl;
            const bool ok = tile < t.ntiles && m < t.M;
            const uint32_t mm = ok ? m : 0u;
            const T* cell = h + cell_origin<S>(mm, t.g, t.C);
#pragma unroll
            for (int s = 0; s < S; ++s) cp_async<VB>(ring.slot(stage, s), cell + slot_offset<S>(s, t.g, t.C), ok);
            cp_async<VB>(ring.slot(stage, S), want_w ? dz + static_cast<size_t>(mm) * t.C : h, ok && want_w);
            cp_async_commit();
        };
        uint32_t tile = blockIdx.x;
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) issue(tile + st * gridDim.x, st);
        int stage = 0;
        for (; tile < t.ntiles; tile += gridDim.x) {
            cp_async_wait<NST - 2>();
            Raw hr[S];
#pragma unroll
            for (int s = 0; s < S; ++s) hr[s] = *ring.slot(stage, s);
            const Raw dr = *ring.slot(stage, S);
            issue(tile + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
            const uint32_t m = tile * t.tl + ln.tl;
            float dv[V];
            float z[V];
            IO::unpack(dr, dv);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                float hv[V];
                IO::unpack(hr[s], hv);
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    z[v] = s == 0 ? hv[v] * w1[0][v] : fmaf(hv[v], w1[s][v], z[v]);
                    acc[s][v] = fmaf(hv[v], dv[v], acc[s][v]);
                }
            }
            if (ddz != nullptr && m < t.M) IO::store(ddz + static_cast<size_t>(m) * t.C, z);
            stage = stage + 1 == NST ? 0 : stage + 1;
        }
        cp_async_wait<0>();
    }
    if (p.partial != nullptr)
        block_reduce_rows<S, V>(acc, p.partial + static_cast<size_t>(blockIdx.x) * S * t.C, t.C, ln.c0, ln.cl, ln.tl,
                                t.cl, t.tl, ln.active, red);
}

namespace {
template <typename F>
inline cudaError_t dispatch_stages(int stages, F&& f) {
    if (stages >= 8) return f(Int<8>{});
    if (stages >= 6) return f(Int<6>{});
    if (stages >= 4) return f(Int<4>{});
    return f(Int<3>{});
}
}  // namespace

cudaError_t launch_read_bwd1_ring(const Problem& pb, const void* x, const void* g, const void* alpha, void* dx,
                                  float* partial, uint32_t* blocks, int stages, int threads) {
    ReadBwd1Params p{};
    p.x = x; p.g = g; p.w = alpha; p.dx = dx; p.partial = partial;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int V = VecWidth<T, S>::value;
            return dispatch_stages(stages, [&](auto n_) {
                constexpr int NST = decltype(n_)::value;
                if constexpr (V * int(sizeof(T)) < 4) return cudaErrorInvalidValue;
                else return launch_persistent_smem(read_bwd1_ring_kernel<T, W, S, V, NST>, p, pb, V, threads,
                                                   static_cast<size_t>(NST) * (S + 1) * V * sizeof(T), partial != nullptr, blocks);
            });
        });
    });
}

cudaError_t launch_write_bwd1_ring(const Problem& pb, const void* h, const void* dz, const void* beta, void* ddz,
                                   float* partial, uint32_t* blocks, int stages, int threads) {
    WriteBwd1Params p{};
    p.h = h; p.dz = dz; p.w = beta; p.ddz = ddz; p.partial = partial;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int V = VecWidth<T, S>::value;
            return dispatch_stages(stages, [&](auto n_) {
                constexpr int NST = decltype(n_)::value;
                if constexpr (V * int(sizeof(T)) < 4) return cudaErrorInvalidValue;
                else return launch_persistent_smem(write_bwd1_ring_kernel<T, W, S, V, NST>, p, pb, V, threads,
                                                   static_cast<size_t>(NST) * (S + 1) * V * sizeof(T), partial != nullptr, blocks);
            });
        });
    });
}

}  // namespace sihc
