// Backward of the literal step  y = x + beta * dz,  z_next = sum_s alpha_next * y  (sihc_write_read_fwd), fused.
//
// With h = dL/dy arriving from the later events and gz = dL/dz_next from the next sublayer, one pass produces
//     hh[m,s,c]      = h[m,s,c] + alpha_next[c,s] * gz[m,c]          total gradient at y (= gradient w.r.t. x)
//     ddz[m,c]       = sum_s beta[c,s] * hh[m,s,c]
//     dalpha_next    = sum_m y[m,s,c] * gz[m,c]
//     dbeta          = sum_m dz[m,c] * hh[m,s,c]
// reading h, y, gz, dz once and writing hh, ddz: 3S+3 elements per (token, channel).  The unfused reference path
// differentiates `write_torch` and `read_torch` separately (sihc/bench/fusion_controls.py:14-31): the read's two
// adjoints (2S+1 and S+1 elements in the reference's two-pass form, sihc/models/sihc/sublayer_kernels.py:280-284),
// the addition of the two carrier gradients by autograd (3S) and the write's adjoints (:300-303).
//
// Same block shape and reduction as the single-event adjoints in sihc_rw.cu: a thread owns V channels, walks tokens
// over a persistent grid, keeps 2*S*V fp32 accumulators, and the block leaves one fp32 row set
// [dalpha rows 0..S-1, dbeta rows S..2S-1] in scratch; a fixed-order finishing pass sums the blocks.
#include "sihc_dispatch.cuh"
#include "sihc_ring.cuh"

namespace sihc {

struct WriteReadBwdParams {
    const void* h;        // dL/dy, may be null (no later consumer of the carrier): treated as zero
    const void* gz;       // dL/dz_next, may be null (the next read was not used): hh = h, dalpha_next = 0
    const void* y;        // the carrier after the write (forward output), read only when gz is given
    const void* dz;       // the written update, read only when dbeta is wanted
    const void* beta;
    const void* alpha;    // alpha_next
    void* hh;             // out: gradient w.r.t. x; may be null; may be the same buffer as h
    void* ddz;            // out, may be null
    float* partial;       // [blocks][2S][C] or null
    Tiling t;
};

constexpr int kLiteralBwdThreads = 384;     // 2*S*V accumulators + 2*S*V coefficients want the 168-register budget

template <typename T, typename W, int S, int V>
__global__ void __launch_bounds__(kLiteralBwdThreads) write_read_bwd_kernel(const __grid_constant__ WriteReadBwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    __shared__ float red[kLiteralBwdThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const T* h = p.h ? static_cast<const T*>(p.h) + ln.c0 : nullptr;          // may alias hh: coherent loads
    const T* __restrict__ gz = p.gz ? static_cast<const T*>(p.gz) + ln.c0 : nullptr;
    const T* __restrict__ y = p.y ? static_cast<const T*>(p.y) + ln.c0 : nullptr;
    const T* __restrict__ dz = p.dz ? static_cast<const T*>(p.dz) + ln.c0 : nullptr;
    T* hh = p.hh ? static_cast<T*>(p.hh) + ln.c0 : nullptr;
    T* __restrict__ ddz = p.ddz ? static_cast<T*>(p.ddz) + ln.c0 : nullptr;
    const bool want_w = p.partial != nullptr;
    const bool in_place = p.h == p.hh;
    // bf16 coefficients over bf16 tensors stay packed (half the registers) and feed the mixed-precision FMA;
    // ddz is then formed as  sum_s beta*h + (sum_s alpha*beta) * gz,  the same sum with packed operands only.
    constexpr bool kPacked = std::is_same<T, W>::value && sizeof(T) == 2;
    float wa[kPacked ? 1 : S][V], wb[kPacked ? 1 : S][V], da[S][V], db[S][V], kappa[V];
    Raw war[kPacked ? S : 1], wbr[kPacked ? S : 1];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int v = 0; v < V; ++v) { da[s][v] = 0.f; db[s][v] = 0.f; }
#pragma unroll
    for (int v = 0; v < V; ++v) kappa[v] = 0.f;
    if (ln.active) {
        {
            float fa[S][V], fb[S][V];
            load_coeffs<W, S, V>(static_cast<const W*>(p.alpha) + static_cast<size_t>(ln.c0) * S, fa);
            load_coeffs<W, S, V>(static_cast<const W*>(p.beta) + static_cast<size_t>(ln.c0) * S, fb);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if constexpr (kPacked) {
                    war[s] = IO::pack(fa[s]); wbr[s] = IO::pack(fb[s]);          // exact: the values are storage values
#pragma unroll
                    for (int v = 0; v < V; ++v) kappa[v] = fmaf(fa[s][v], fb[s][v], kappa[v]);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) { wa[s][v] = fa[s][v]; wb[s][v] = fb[s][v]; }
                }
            }
        }
        for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
            const uint32_t m = tile * t.tl + ln.tl;
            if (m >= t.M) continue;
            const size_t origin = cell_origin<S>(m, t.g, t.C);
            const size_t row = static_cast<size_t>(m) * t.C;
            Raw hr[S], yr[S];
            const Raw gr = gz != nullptr ? IO::load_raw(gz + row) : IO::zero_raw();
            const Raw dr = (dz != nullptr && want_w) ? IO::load_raw(dz + row) : IO::zero_raw();
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const size_t off = origin + slot_offset<S>(s, t.g, t.C);
                hr[s] = h == nullptr ? IO::zero_raw() : (in_place ? IO::load_raw_coherent(h + off) : IO::load_raw(h + off));
                yr[s] = (gz != nullptr && want_w && y != nullptr) ? IO::load_raw(y + off) : IO::zero_raw();
            }
            float gv[V], dv[V], zacc[V];
            IO::unpack(gr, gv);
            IO::unpack(dr, dv);
            if constexpr (kPacked) {
#pragma unroll
                for (int v = 0; v < V; ++v) zacc[v] = kappa[v] * gv[v];
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float hv[V];
                    IO::unpack(hr[s], hv);
                    IO::fma_raw(wbr[s], hr[s], zacc);                      // beta * h
                    IO::fma_raw(war[s], gr, hv);                           // h + alpha_next * gz
                    IO::fma_raw(yr[s], gr, da[s]);
#pragma unroll
                    for (int v = 0; v < V; ++v) db[s][v] = fmaf(dv[v], hv[v], db[s][v]);
                    if (hh != nullptr) IO::store(hh + origin + slot_offset<S>(s, t.g, t.C), hv);
                }
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) zacc[v] = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float hv[V], yv[V];
                    IO::unpack(hr[s], hv);
                    IO::unpack(yr[s], yv);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        hv[v] = fmaf(wa[s][v], gv[v], hv[v]);                 // total gradient at y
                        da[s][v] = fmaf(yv[v], gv[v], da[s][v]);
                        db[s][v] = fmaf(dv[v], hv[v], db[s][v]);
                        zacc[v] = fmaf(wb[s][v], hv[v], zacc[v]);
                    }
                    if (hh != nullptr) IO::store(hh + origin + slot_offset<S>(s, t.g, t.C), hv);
                }
            }
            if (ddz != nullptr) IO::store(ddz + row, zacc);
        }
    }
    if (want_w) {
        float* dst = p.partial + static_cast<size_t>(blockIdx.x) * 2 * S * t.C;
        block_reduce_rows<S, V>(da, dst, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl, ln.active, red);
        block_reduce_rows<S, V>(db, dst + static_cast<size_t>(S) * t.C, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl, ln.active, red);
    }
}


// The same pass with its 2S+2 input vectors per token staged through a per-thread `cp.async` ring in shared memory
// (NST stages, private slots, no block barrier - the scheme of the single-event adjoints in sihc_ring.cu).  The
// register-staged kernel above holds 2*S*V accumulators and 2*S*V coefficients and has no registers left to keep a
// second token's loads in flight; here the loads never occupy registers while they travel.  Vector path only.
// Block shape of the ring form.  Its speed comes from token-level parallelism - many warps, each walking its own tokens
// through ~500 dependent instructions per token - so the channel vectors are split over blockIdx.y until a block of
// about 256 threads has at least 4 (width <= 768) or 6 token lanes.  Measured on B200, bf16, GB/s of the 3S+3 elements:
// 65 536 tokens x 768: 3 lanes x 96 channel lanes 4475, 4 x 96 (384 threads) 4750, 5 x 48 5185; 8192 x 768: 3934;
// 8192 x 1152: 2 x 144 3485, 7 x 36 4045; 65 536 x 1152: 4600-4750.  Half-width vectors (twice the channel lanes, same
// token lanes) gain 3 % over 3 x 96 and lose against more token lanes.
constexpr int kLiteralRingThreads = 256;       // target; whole channel slices round it to at most kLiteralRingMaxThreads
constexpr int kLiteralRingMaxThreads = 384;
constexpr int kLiteralRingStages = 3;
// Half-width form: V/2 channels per thread, twice the threads (and warps) for the same bytes in flight.
constexpr int kLiteralHalfThreads = 512;
constexpr int kLiteralHalfMaxThreads = 576;

template <typename T, typename W, int S, int V, int NST, int MAXT>
__global__ void __launch_bounds__(MAXT) write_read_bwd_ring_kernel(const __grid_constant__ WriteReadBwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    constexpr int VB = int(sizeof(Raw));
    constexpr int NV = 2 * S + 2;                 // h slots, y slots, gz, dz
    extern __shared__ __align__(16) unsigned char ring_bytes[];
    __shared__ float red[MAXT * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const Ring<Raw> ring{reinterpret_cast<Raw*>(ring_bytes), blockDim.x, threadIdx.x, NV};
    const T* h = p.h ? static_cast<const T*>(p.h) + ln.c0 : nullptr;
    const T* __restrict__ gz = p.gz ? static_cast<const T*>(p.gz) + ln.c0 : nullptr;
    const T* __restrict__ y = p.y ? static_cast<const T*>(p.y) + ln.c0 : nullptr;
    const T* __restrict__ dz = p.dz ? static_cast<const T*>(p.dz) + ln.c0 : nullptr;
    T* hh = p.hh ? static_cast<T*>(p.hh) + ln.c0 : nullptr;
    T* __restrict__ ddz = p.ddz ? static_cast<T*>(p.ddz) + ln.c0 : nullptr;
    const bool want_w = p.partial != nullptr;
    const bool want_y = gz != nullptr && want_w && y != nullptr;
    const bool want_dz = dz != nullptr && want_w;
    constexpr bool kPacked = std::is_same<T, W>::value && sizeof(T) == 2;
    float wa[kPacked ? 1 : S][V], wb[kPacked ? 1 : S][V], da[S][V], db[S][V], kappa[V];
    Raw war[kPacked ? S : 1], wbr[kPacked ? S : 1];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int v = 0; v < V; ++v) { da[s][v] = 0.f; db[s][v] = 0.f; }
#pragma unroll
    for (int v = 0; v < V; ++v) kappa[v] = 0.f;
    if (ln.active) {
        {
            float fa[S][V], fb[S][V];
            load_coeffs<W, S, V>(static_cast<const W*>(p.alpha) + static_cast<size_t>(ln.c0) * S, fa);
            load_coeffs<W, S, V>(static_cast<const W*>(p.beta) + static_cast<size_t>(ln.c0) * S, fb);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if constexpr (kPacked) {
                    war[s] = IO::pack(fa[s]); wbr[s] = IO::pack(fb[s]);
#pragma unroll
                    for (int v = 0; v < V; ++v) kappa[v] = fmaf(fa[s][v], fb[s][v], kappa[v]);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) { wa[s][v] = fa[s][v]; wb[s][v] = fb[s][v]; }
                }
            }
        }
        // `src_or` keeps the address valid when a copy is switched off (zero source bytes = zero fill)
        const T* const src_or = static_cast<const T*>(p.beta ? p.beta : p.alpha);
        auto issue = [&](uint32_t tile, int stage) {
            const uint32_t m = tile * t.tl + ln.tl;
            const bool ok = tile < t.ntiles && m < t.M;
            const uint32_t mm = ok ? m : 0u;
            const size_t origin = cell_origin<S>(mm, t.g, t.C);
            const size_t row = static_cast<size_t>(mm) * t.C;
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const size_t off = origin + slot_offset<S>(s, t.g, t.C);
                cp_async<VB>(ring.slot(stage, s), h != nullptr ? h + off : src_or, ok && h != nullptr);
                cp_async<VB>(ring.slot(stage, S + s), want_y ? y + off : src_or, ok && want_y);
            }
            cp_async<VB>(ring.slot(stage, 2 * S), gz != nullptr ? gz + row : src_or, ok && gz != nullptr);
            cp_async<VB>(ring.slot(stage, 2 * S + 1), want_dz ? dz + row : src_or, ok && want_dz);
            cp_async_commit();
        };
        uint32_t tile = blockIdx.x;
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) issue(tile + st * gridDim.x, st);
        int stage = 0;
        for (; tile < t.ntiles; tile += gridDim.x) {
            cp_async_wait<NST - 2>();
            Raw hr[S], yr[S];
#pragma unroll
            for (int s = 0; s < S; ++s) { hr[s] = *ring.slot(stage, s); yr[s] = *ring.slot(stage, S + s); }
            const Raw gr = *ring.slot(stage, 2 * S);
            const Raw dr = *ring.slot(stage, 2 * S + 1);
            issue(tile + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
            const uint32_t m = tile * t.tl + ln.tl;
            const bool ok = m < t.M;
            const size_t origin = cell_origin<S>(ok ? m : 0u, t.g, t.C);
            float gv[V], dv[V], zacc[V];
            IO::unpack(gr, gv);
            IO::unpack(dr, dv);
            if constexpr (kPacked) {
#pragma unroll
                for (int v = 0; v < V; ++v) zacc[v] = kappa[v] * gv[v];
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float hv[V];
                    IO::unpack(hr[s], hv);
                    IO::fma_raw(wbr[s], hr[s], zacc);
                    IO::fma_raw(war[s], gr, hv);
                    IO::fma_raw(yr[s], gr, da[s]);
#pragma unroll
                    for (int v = 0; v < V; ++v) db[s][v] = fmaf(dv[v], hv[v], db[s][v]);
                    if (hh != nullptr && ok) IO::store(hh + origin + slot_offset<S>(s, t.g, t.C), hv);
                }
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) zacc[v] = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float hv[V], yv[V];
                    IO::unpack(hr[s], hv);
                    IO::unpack(yr[s], yv);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        hv[v] = fmaf(wa[s][v], gv[v], hv[v]);
                        da[s][v] = fmaf(yv[v], gv[v], da[s][v]);
                        db[s][v] = fmaf(dv[v], hv[v], db[s][v]);
                        zacc[v] = fmaf(wb[s][v], hv[v], zacc[v]);
                    }
                    if (hh != nullptr && ok) IO::store(hh + origin + slot_offset<S>(s, t.g, t.C), hv);
                }
            }
            if (ddz != nullptr && ok) IO::store(ddz + static_cast<size_t>(m) * t.C, zacc);
            stage = stage + 1 == NST ? 0 : stage + 1;
        }
        cp_async_wait<0>();
    }
    if (want_w) {
        float* dst = p.partial + static_cast<size_t>(blockIdx.x) * 2 * S * t.C;
        block_reduce_rows<S, V>(da, dst, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl, ln.active, red);
        block_reduce_rows<S, V>(db, dst + static_cast<size_t>(S) * t.C, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl, ln.active, red);
    }
}

cudaError_t launch_write_read_bwd(const Problem& pb, const void* h, const void* gz, const void* y, const void* dz,
                                  const void* beta, const void* alpha_next, void* hh, void* ddz, float* partial,
                                  uint32_t* blocks) {
    WriteReadBwdParams p{};
    p.h = h; p.gz = gz; p.y = y; p.dz = dz; p.beta = beta; p.alpha = alpha_next; p.hh = hh; p.ddz = ddz; p.partial = partial;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int VM = VecWidth<T, S>::value;
            if (pb.V == 1)
                return launch_persistent(write_read_bwd_kernel<T, W, S, 1>, p, pb, 1, 1, kLiteralBwdThreads, 1,
                                         partial != nullptr, blocks, kLiteralBwdThreads);
            // In place (hh == h) the carrier gradient must be read with coherent loads: the ring's asynchronous copies
            // go through L2 and a thread only rewrites what it has already consumed, so the ring form covers it too.
            const int ring = tuning().ring;       // 0 = register-staged form, otherwise the ring (default)
            if constexpr (VM * int(sizeof(T)) >= 4) {
                constexpr int VH = (S * VM >= 32 && VM * int(sizeof(T)) >= 8) ? VM / 2 : VM;
                if (ring != 0 && tuning().half_vectors > 0 && VH != VM) {
                    return launch_persistent_smem(write_read_bwd_ring_kernel<T, W, S, VH, kLiteralRingStages, kLiteralHalfMaxThreads>,
                                                  p, pb, VH, kLiteralHalfThreads,
                                                  static_cast<size_t>(kLiteralRingStages) * (2 * S + 2) * VH * sizeof(T),
                                                  partial != nullptr, blocks, kLiteralHalfMaxThreads);
                }
                if (ring >= 4) {
                    return launch_persistent_smem(write_read_bwd_ring_kernel<T, W, S, VM, 4, kLiteralRingMaxThreads>, p, pb, VM,
                                                  kLiteralRingThreads, static_cast<size_t>(4) * (2 * S + 2) * VM * sizeof(T),
                                                  partial != nullptr, blocks, kLiteralRingMaxThreads);
                }
                if (ring != 0) {
                    return launch_persistent_smem(write_read_bwd_ring_kernel<T, W, S, VM, kLiteralRingStages, kLiteralRingMaxThreads>,
                                                  p, pb, VM, kLiteralRingThreads,
                                                  static_cast<size_t>(kLiteralRingStages) * (2 * S + 2) * VM * sizeof(T),
                                                  partial != nullptr, blocks, kLiteralRingMaxThreads,
                                                  static_cast<uint32_t>(tuning().token_lanes > 0 ? tuning().token_lanes : (pb.C / VM <= 96 ? 4 : 6)));
                }
            }
            return launch_persistent(write_read_bwd_kernel<T, W, S, VM>, p, pb, VM, 1, kLiteralBwdThreads, 1,
                                     partial != nullptr, blocks, kLiteralBwdThreads);
        });
    });
}

}  // namespace sihc
