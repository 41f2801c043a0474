// Stage (multi-event) read and write with the coefficients staged in shared memory.
//
// In the [E, C, S] parameter layout the S*V coefficients of one event for a thread's V channels are one
// contiguous run, but neighbouring threads' runs are S*V elements apart: a warp-wide 16-byte load touches 16
// different 128-byte lines.  Here the block copies its channel slice of ALL events once (coalesced) into
// shared memory, transposed to [event][slot][channel], so that an event's coefficients are S conflict-free
// vector reads per thread.  The reference reaches the same layout with a transposed copy of the weights in
// global memory (`alpha.transpose(1, 2).contiguous()`, sihc/models/sihc/sublayer_kernels.py:224); this
// library allocates nothing, so the transpose lives in shared memory.
//
// The slice is kept small (at most 35 KB and 32 channel lanes per block, more blocks per SM): residency matters more
// than a wide tile.  Measured on B200 (bf16, width 768, against re-reading the coefficients from L1): 4 slots E=24
// read 4599 -> 5074 GB/s, write 3945 -> 4517; 16 slots E=12 read 2347 -> 2938, write 2134 -> 2649.  With a 160 KB slice
// (one block per SM) the 4-slot case was slower than the L1 form (4118 / 3761).
#include "sihc_dispatch.cuh"

namespace sihc {

// Copy alpha[l][cbase + c][s] (l < E, c < CS, s < S) into wsm[(l*S + s)*CS + c].  All threads of the block.
template <typename W, int S>
__device__ __forceinline__ void stage_coefficients(const W* __restrict__ w, W* wsm, int E, uint32_t C, uint32_t cbase,
                                                   uint32_t CS, uint32_t c_valid) {
    const uint32_t per_event = CS * S;
    for (uint32_t idx = threadIdx.x; idx < static_cast<uint32_t>(E) * per_event; idx += blockDim.x) {
        const uint32_t l = idx / per_event, r = idx - l * per_event;
        const uint32_t c = r / S, s = r - c * S;                       // global order: channel-major, slot fastest
        W v = W();
        if (c < c_valid) v = __ldg(w + (static_cast<size_t>(l) * C + cbase + c) * S + s);
        wsm[(l * S + s) * CS + c] = v;
    }
}

template <typename W, int V>
__device__ __forceinline__ void smem_coeffs(const W* p, float (&w)[V]) {     // V contiguous channels of one (event, slot)
    constexpr int BYTES = int(sizeof(W)) * V;
    if constexpr (BYTES <= 16) {
        typedef typename RawBits<BYTES>::type Raw;
        const Raw r = *reinterpret_cast<const Raw*>(p);
        if constexpr (sizeof(W) == 2) VecIO<bf16_t, V>::unpack(r, w);
        else VecIO<float, V>::unpack(r, w);
    } else {                                       // fp32 coefficients for 8 channels: two 16-byte reads
        static_assert(sizeof(W) == 4 && V == 8, "wide coefficient read");
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
}

// out[l][m,c] = sum_s alpha[l,c,s] * X[m,s,c]
template <typename T, typename W, int S, int V, int TT>
__global__ void __launch_bounds__(384) read_fwd_stage_kernel(const __grid_constant__ ReadFwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    W* wsm = reinterpret_cast<W*>(smem_bytes);
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const uint32_t CS = t.cl * V, cbase = blockIdx.y * CS;
    stage_coefficients<W, S>(static_cast<const W*>(p.w), wsm, p.E, t.C, cbase, CS, t.C > cbase ? min(CS, t.C - cbase) : 0u);
    __syncthreads();
    if (!ln.active) return;
    const T* __restrict__ x = static_cast<const T*>(p.x) + ln.c0;
    const W* wme = wsm + ln.cl * V;
    const uint32_t per_tile = t.tl * TT;
    for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
        Raw xr[TT][S];
        uint32_t m[TT];
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            m[i] = tile * per_tile + i * t.tl + ln.tl;
            const bool ok = m[i] < t.M;
            const T* cell = x + cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
#pragma unroll
            for (int s = 0; s < S; ++s) xr[i][s] = ok ? IO::load_raw(cell + slot_offset<S>(s, t.g, t.C)) : IO::zero_raw();
        }
#pragma unroll 1
        for (int l = 0; l < p.E; ++l) {
            if (p.out.p[l] == nullptr) continue;      // output not wanted
            T* __restrict__ out = static_cast<T*>(p.out.p[l]) + ln.c0;
            float acc[TT][V];
            if constexpr (std::is_same<T, W>::value) {      // packed operands straight into the accumulating FMA
#pragma unroll
                for (int i = 0; i < TT; ++i)
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[i][v] = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    const Raw wr = *reinterpret_cast<const Raw*>(wme + (static_cast<uint32_t>(l) * S + s) * CS);
#pragma unroll
                    for (int i = 0; i < TT; ++i) IO::fma_raw(xr[i][s], wr, acc[i]);
                }
            } else {
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float w[V];
                    smem_coeffs<W, V>(wme + (static_cast<uint32_t>(l) * S + s) * CS, w);
#pragma unroll
                    for (int i = 0; i < TT; ++i) {
                        float xv[V];
                        IO::unpack(xr[i][s], xv);
#pragma unroll
                        for (int v = 0; v < V; ++v) acc[i][v] = s == 0 ? xv[v] * w[v] : fmaf(xv[v], w[v], acc[i][v]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < TT; ++i)
                if (m[i] < t.M) IO::store(out + static_cast<size_t>(m[i]) * t.C, acc[i]);
        }
    }
}

// y[m,s,c] = (x ? x[m,s,c] : 0) + sum_l beta[l,c,s] * dz[l][m,c]     (null dz[l] skipped)
template <typename T, typename W, int S, int V, int TT>
__global__ void __launch_bounds__(384) write_fwd_stage_kernel(const __grid_constant__ WriteFwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    W* wsm = reinterpret_cast<W*>(smem_bytes);
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const uint32_t CS = t.cl * V, cbase = blockIdx.y * CS;
    stage_coefficients<W, S>(static_cast<const W*>(p.w), wsm, p.E, t.C, cbase, CS, t.C > cbase ? min(CS, t.C - cbase) : 0u);
    __syncthreads();
    if (!ln.active) return;
    const T* __restrict__ x = p.x ? static_cast<const T*>(p.x) + ln.c0 : nullptr;
    T* __restrict__ y = static_cast<T*>(p.y) + ln.c0;
    const W* wme = wsm + ln.cl * V;
    const uint32_t per_tile = t.tl * TT;
    for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
        float acc[TT][S][V];
        uint32_t m[TT];
        size_t origin[TT];
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            m[i] = tile * per_tile + i * t.tl + ln.tl;
            const bool ok = m[i] < t.M;
            origin[i] = cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (ok && x != nullptr) IO::load(x + origin[i] + slot_offset<S>(s, t.g, t.C), acc[i][s]);
                else {
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[i][s][v] = 0.f;
                }
            }
        }
#pragma unroll 1
        for (int l0 = 0; l0 < p.E; l0 += 4) {           // four update streams in flight per trip
            Raw dr[4][TT];
            bool have[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int l = l0 + k;
                have[k] = l < p.E && p.dz.p[l] != nullptr;
                const T* __restrict__ dz = have[k] ? static_cast<const T*>(p.dz.p[l]) + ln.c0 : nullptr;
#pragma unroll
                for (int i = 0; i < TT; ++i)
                    dr[k][i] = (have[k] && m[i] < t.M) ? IO::load_raw(dz + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (!have[k]) continue;
                if constexpr (std::is_same<T, W>::value) {
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        const Raw wr = *reinterpret_cast<const Raw*>(wme + (static_cast<uint32_t>(l0 + k) * S + s) * CS);
#pragma unroll
                        for (int i = 0; i < TT; ++i) IO::fma_raw(wr, dr[k][i], acc[i][s]);
                    }
                } else {
                    float d[TT][V];
#pragma unroll
                    for (int i = 0; i < TT; ++i) IO::unpack(dr[k][i], d[i]);
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        float w[V];
                        smem_coeffs<W, V>(wme + (static_cast<uint32_t>(l0 + k) * S + s) * CS, w);
#pragma unroll
                        for (int i = 0; i < TT; ++i)
#pragma unroll
                            for (int v = 0; v < V; ++v) acc[i][s][v] = fmaf(w[v], d[i][v], acc[i][s][v]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            if (m[i] < t.M) {
#pragma unroll
                for (int s = 0; s < S; ++s) IO::store(y + origin[i] + slot_offset<S>(s, t.g, t.C), acc[i][s]);
            }
        }
    }
}

namespace {

// Block shape: 32, 16 or 8 channel lanes (a warp then covers whole token rows), the most whose coefficient slice
// (E*S*V elements of W per lane) fits the shared-memory budget, preferring a count that divides the channel vectors
// evenly over blockIdx.y.  Measured on B200 (bf16, read / write GB/s): width 1152, E=24, 8192 tokens: 29 lanes
// 3081 / 4050, 16 lanes 4409 / 4535; width 768, E=8, 65 536 tokens: 96 lanes 4960 / 5599, 32 lanes 5326 / 5943.
struct StageShape { uint32_t cl, tl, gy, threads; size_t smem; };
inline StageShape stage_shape(uint32_t ncv, int E, int S, int V, size_t wbytes, int target_threads) {
    const size_t kBudget = static_cast<size_t>(tuning().stage_budget_kb > 0 ? tuning().stage_budget_kb : 35) * 1024;
    const size_t per_lane = static_cast<size_t>(E) * S * V * wbytes;
    uint32_t cl = 32;
    while (cl > 8 && per_lane * cl > kBudget) cl >>= 1;
    for (uint32_t c = cl; c >= 8; c >>= 1)
        if (ncv % c == 0) { cl = c; break; }
    if (cl > ncv) cl = ncv;
    StageShape sh;
    sh.cl = cl;
    sh.gy = (ncv + cl - 1) / cl;
    uint32_t tl = (static_cast<uint32_t>(target_threads) + sh.cl / 2) / sh.cl;
    if (tl < 1) tl = 1;
    while (tl > 1 && tl * sh.cl > 384u) --tl;
    sh.tl = tl;
    sh.threads = sh.cl * tl;
    sh.smem = per_lane * sh.cl;
    return sh;
}

template <typename K, typename P>
inline cudaError_t launch_stage(K kernel, P& p, const Problem& pb, int V, int TT, const StageShape& sh) {
    if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024)) return e;
    Tiling& t = p.t;
    t.M = pb.M; t.g = pb.g; t.C = pb.C; t.ncv = pb.C / static_cast<uint32_t>(V); t.cl = sh.cl; t.tl = sh.tl;
    const uint32_t per_tile = sh.tl * static_cast<uint32_t>(TT);
    t.ntiles = (pb.M + per_tile - 1) / per_tile;
    int nb = cached_occupancy(reinterpret_cast<const void*>(kernel), static_cast<int>(sh.threads), sh.smem);
    if (tuning().bps > 0 && nb > tuning().bps) nb = tuning().bps;
    uint32_t gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / sh.gy;
    if (gx < 1) gx = 1;
    if (gx > t.ntiles) gx = t.ntiles;
    kernel<<<dim3(gx, sh.gy, 1), sh.threads, sh.smem, pb.stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_read_fwd_stage(const Problem& pb, ReadFwdParams& p) {
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int V = VecWidth<T, S>::value;
            const int threads = tuning().threads > 0 ? tuning().threads : 384;
            const StageShape sh = stage_shape(pb.C / V, pb.E, S, V, sizeof(W), threads);
            if (tuning().tt > 0 && tuning().tt < 4)
                return launch_stage(read_fwd_stage_kernel<T, W, S, V, 2>, p, pb, V, 2, sh);
            return launch_stage(read_fwd_stage_kernel<T, W, S, V, 4>, p, pb, V, 4, sh);
        });
    });
}

cudaError_t launch_write_fwd_stage(const Problem& pb, WriteFwdParams& p) {
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int V = VecWidth<T, S>::value;
            const int threads = tuning().threads > 0 ? tuning().threads : 384;
            const StageShape sh = stage_shape(pb.C / V, pb.E, S, V, sizeof(W), threads);
            if (tuning().tt >= 2)
                return launch_stage(write_fwd_stage_kernel<T, W, S, V, 2>, p, pb, V, 2, sh);
            return launch_stage(write_fwd_stage_kernel<T, W, S, V, 1>, p, pb, V, 1, sh);
        });
    });
}

}  // namespace sihc
