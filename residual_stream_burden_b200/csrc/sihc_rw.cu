// SiHC read / write streaming kernels (forward, and the fused single-event adjoints).
//
// The single-event kernels are HBM-bound diagonal maps: per workspace token and
// channel they touch S carrier elements and a handful of workspace elements, with
// at most 2*S FMAs.  The design goal is therefore bytes in flight, not math: every
// thread issues TT*(S+1) independent 16-byte loads (read-only path) before its
// first use, keeps its coefficient vectors in registers, and stores 16-byte
// streaming vectors.  The multi-event forms in this file fetch each event's
// coefficients from L1 in the native [E,C,S] layout; they serve the scalar path -
// on the vector path the stage read and write run the staged-coefficient kernels
// of sihc_stage.cu, and the fused adjoints the ring kernels of sihc_ring.cu.
//
// Algorithmic traffic per (token, channel) element, in elements:
//   read  fwd : S + E          write fwd : 2S + E (S + E without the carry)
//   read  bwd (E = 1, fused dX + dalpha) : 2S + 1
//   write bwd (E = 1, fused ddz + dbeta) : S + 2
#include "sihc_dispatch.cuh"

namespace sihc {

// ---- stage read, forward ---------------------------------------------------------------------
// out[l][m,c] = sum_s alpha[l,c,s] * X[m,s,c]
// (reference: `_read`, sihc/models/sihc/sublayer_kernels.py:28-49; E = 1: `read_torch`,
//  sihc/bench/fusion_controls.py:14-20)
template <typename T, typename W, int S, int V, int TT, bool SINGLE>
__global__ void __launch_bounds__(SINGLE || TT < 4 ? kMaxThreads : 384) read_fwd_kernel(const __grid_constant__ ReadFwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    if (!ln.active) return;
    const T* __restrict__ x = static_cast<const T*>(p.x) + ln.c0;
    const W* __restrict__ wt = static_cast<const W*>(p.w) + static_cast<size_t>(ln.c0) * S;
    float w1[S][V];
    if constexpr (SINGLE) load_coeffs<W, S, V>(wt, w1);
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
        if constexpr (SINGLE) {
            T* __restrict__ out = static_cast<T*>(p.out.p[0]) + ln.c0;
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                float acc[V];
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float xv[V];
                    IO::unpack(xr[i][s], xv);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = s == 0 ? xv[v] * w1[0][v] : fmaf(xv[v], w1[s][v], acc[v]);
                }
                if (m[i] < t.M) IO::store(out + static_cast<size_t>(m[i]) * t.C, acc);
            }
        } else {
#pragma unroll 1
            for (int l = 0; l < p.E; ++l) {
                if (p.out.p[l] == nullptr) continue;      // output not wanted
                float w[S][V];
                load_coeffs<W, S, V>(wt + static_cast<size_t>(l) * t.C * S, w);
                T* __restrict__ out = static_cast<T*>(p.out.p[l]) + ln.c0;
#pragma unroll
                for (int i = 0; i < TT; ++i) {
                    float acc[V];
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        float xv[V];
                        IO::unpack(xr[i][s], xv);
#pragma unroll
                        for (int v = 0; v < V; ++v) acc[v] = s == 0 ? xv[v] * w[0][v] : fmaf(xv[v], w[s][v], acc[v]);
                    }
                    if (m[i] < t.M) IO::store(out + static_cast<size_t>(m[i]) * t.C, acc);
                }
            }
        }
    }
}

// ---- stage write, forward ----------------------------------------------------------------------
// y[m,s,c] = (x ? x[m,s,c] : 0) + sum_l beta[l,c,s] * dz[l][m,c]
// (reference: `_write`, sihc/models/sihc/sublayer_kernels.py:82-97; a null dz[l] is skipped,
//  which is how the read's carrier gradient treats unused read outputs)
template <typename T, typename W, int S, int V, int TT, bool SINGLE>
__global__ void __launch_bounds__(kMaxThreads) write_fwd_kernel(const __grid_constant__ WriteFwdParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    if (!ln.active) return;
    const T* __restrict__ x = p.x ? static_cast<const T*>(p.x) + ln.c0 : nullptr;
    T* __restrict__ y = static_cast<T*>(p.y) + ln.c0;
    const W* __restrict__ wt = static_cast<const W*>(p.w) + static_cast<size_t>(ln.c0) * S;
    float w1[S][V];
    if constexpr (SINGLE) load_coeffs<W, S, V>(wt, w1);
    const uint32_t per_tile = t.tl * TT;

    for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
        uint32_t m[TT];
        size_t origin[TT];
        if constexpr (SINGLE) {
            Raw xr[TT][S];
            Raw dr[TT];
            const T* __restrict__ dz = static_cast<const T*>(p.dz.p[0]) + ln.c0;
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                m[i] = tile * per_tile + i * t.tl + ln.tl;
                const bool ok = m[i] < t.M;
                origin[i] = cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
                dr[i] = ok ? IO::load_raw(dz + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
#pragma unroll
                for (int s = 0; s < S; ++s)
                    xr[i][s] = (ok && x != nullptr) ? IO::load_raw(x + origin[i] + slot_offset<S>(s, t.g, t.C)) : IO::zero_raw();
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                float d[V];
                IO::unpack(dr[i], d);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float r[V];
                    IO::unpack(xr[i][s], r);
#pragma unroll
                    for (int v = 0; v < V; ++v) r[v] = fmaf(w1[s][v], d[v], r[v]);
                    if (m[i] < t.M) IO::store(y + origin[i] + slot_offset<S>(s, t.g, t.C), r);
                }
            }
        } else {
            float acc[TT][S][V];
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
                    have[k] = l < p.E && p.dz.p[l] != nullptr;      // a null update is skipped
                    const T* __restrict__ dz = have[k] ? static_cast<const T*>(p.dz.p[l]) + ln.c0 : nullptr;
#pragma unroll
                    for (int i = 0; i < TT; ++i)
                        dr[k][i] = (have[k] && m[i] < t.M) ? IO::load_raw(dz + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (!have[k]) continue;
                    float w[S][V];
                    load_coeffs<W, S, V>(wt + static_cast<size_t>(l0 + k) * t.C * S, w);
#pragma unroll
                    for (int i = 0; i < TT; ++i) {
                        float d[V];
                        IO::unpack(dr[k][i], d);
#pragma unroll
                        for (int s = 0; s < S; ++s)
#pragma unroll
                            for (int v = 0; v < V; ++v) acc[i][s][v] = fmaf(w[s][v], d[v], acc[i][s][v]);
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
}

// ---- literal step: write event i, read event i+1, one pass (inference) ------------------------------
// y[m,s,c] = x[m,s,c] + beta[c,s] * dz[m,c]   (rounded to the storage type, as the unfused path stores it)
// z[m,c]   = sum_s alpha_next[c,s] * y[m,s,c] (read from the ROUNDED carrier, as the unfused path reads it)
// Moves 2S+2 elements per (token, channel); the unfused pair moves 3S+2.  `y` may be `x` (in place): every
// element is read and written by the same thread, and in that case the carrier is read with ordinary coherent
// loads (the read-only path is reserved for memory that no thread writes during the kernel).
template <typename T, typename W, int S, int V, int TT>
__global__ void __launch_bounds__(kMaxThreads) write_read_kernel(const __grid_constant__ WriteReadParams p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    if (!ln.active) return;
    const T* x = static_cast<const T*>(p.x) + ln.c0;
    T* y = static_cast<T*>(p.y) + ln.c0;
    const bool in_place = p.x == p.y;            // uniform over the grid
    const T* __restrict__ dz = static_cast<const T*>(p.dz) + ln.c0;
    T* __restrict__ z = static_cast<T*>(p.z) + ln.c0;
    float wb[S][V], wa[S][V];
    load_coeffs<W, S, V>(static_cast<const W*>(p.beta) + static_cast<size_t>(ln.c0) * S, wb);
    load_coeffs<W, S, V>(static_cast<const W*>(p.alpha) + static_cast<size_t>(ln.c0) * S, wa);
    // Same-type coefficients are kept packed per slot (half the registers) and fed to the mixed-precision FMA.
    constexpr bool kPacked = std::is_same<T, W>::value;
    Raw wbr[kPacked ? S : 1], war[kPacked ? S : 1];
    if constexpr (kPacked) {
#pragma unroll
        for (int s = 0; s < S; ++s) { wbr[s] = IO::pack(wb[s]); war[s] = IO::pack(wa[s]); }    // exact: the values are storage values
    }
    const uint32_t per_tile = t.tl * TT;
    for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
        Raw xr[TT][S];
        Raw dr[TT];
        uint32_t m[TT];
        size_t origin[TT];
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            m[i] = tile * per_tile + i * t.tl + ln.tl;
            const bool ok = m[i] < t.M;
            origin[i] = cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
            dr[i] = ok ? IO::load_raw(dz + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const T* src = x + origin[i] + slot_offset<S>(s, t.g, t.C);
                xr[i][s] = !ok ? IO::zero_raw() : (in_place ? IO::load_raw_coherent(src) : IO::load_raw(src));
            }
        }
        if constexpr (kPacked) {
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                float acc[V];
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float r[V];
                    IO::unpack(xr[i][s], r);
                    IO::fma_raw(wbr[s], dr[i], r);              // x + beta * dz
                    const Raw yr = IO::pack(r);                 // rounded to storage: what the read sees
                    if (m[i] < t.M) IO::store_raw(y + origin[i] + slot_offset<S>(s, t.g, t.C), yr);
                    IO::fma_raw(yr, war[s], acc);
                }
                if (m[i] < t.M) IO::store(z + static_cast<size_t>(m[i]) * t.C, acc);
            }
            continue;
        }
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            float d[V], acc[V];
            IO::unpack(dr[i], d);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                float r[V];
                IO::unpack(xr[i][s], r);
#pragma unroll
                for (int v = 0; v < V; ++v) r[v] = fmaf(wb[s][v], d[v], r[v]);
                if constexpr (sizeof(T) == 2) {             // round to storage before the read uses it
#pragma unroll
                    for (int v = 0; v < V; ++v) r[v] = __uint_as_float(static_cast<uint32_t>(pack_bf16(r[v])) << 16);
                }
                if (m[i] < t.M) IO::store(y + origin[i] + slot_offset<S>(s, t.g, t.C), r);
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = s == 0 ? r[v] * wa[0][v] : fmaf(r[v], wa[s][v], acc[v]);
            }
            if (m[i] < t.M) IO::store(z + static_cast<size_t>(m[i]) * t.C, acc);
        }
    }
}

// ---- single-event read, backward (fused) ---------------------------------------------------
// dx[m,s,c] = alpha[c,s] * g[m,c];  partial[block][s][c] = sum_{m in block} X[m,s,c] * g[m,c]
// One pass over X and g produces both adjoints (the reference makes two passes:
// `_write_impl(add_x=False)` and `_weights_backward`, sihc/models/sihc/sublayer_kernels.py:284).
template <typename T, typename W, int S, int V, int TT>
__global__ void __launch_bounds__(kMaxThreads) read_bwd1_kernel(const __grid_constant__ ReadBwd1Params p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
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
        const uint32_t per_tile = t.tl * TT;
        for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
            Raw xr[TT][S];
            Raw gr[TT];
            uint32_t m[TT];
            size_t origin[TT];
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                m[i] = tile * per_tile + i * t.tl + ln.tl;
                const bool ok = m[i] < t.M;
                origin[i] = cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
                gr[i] = ok ? IO::load_raw(g + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
#pragma unroll
                for (int s = 0; s < S; ++s)
                    xr[i][s] = (ok && want_w) ? IO::load_raw(x + origin[i] + slot_offset<S>(s, t.g, t.C)) : IO::zero_raw();
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                float gv[V];
                IO::unpack(gr[i], gv);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float xv[V];
                    float d[V];
                    IO::unpack(xr[i][s], xv);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        d[v] = w1[s][v] * gv[v];
                        acc[s][v] = fmaf(xv[v], gv[v], acc[s][v]);
                    }
                    if (dx != nullptr && m[i] < t.M) IO::store(dx + origin[i] + slot_offset<S>(s, t.g, t.C), d);
                }
            }
        }
    }
    if (want_w)
        block_reduce_rows<S, V>(acc, p.partial + static_cast<size_t>(blockIdx.x) * S * t.C, t.C, ln.c0, ln.cl, ln.tl,
                                t.cl, t.tl, ln.active, red);
}

// ---- single-event write, backward (fused) --------------------------------------------------
// ddz[m,c] = sum_s beta[c,s] * h[m,s,c];  partial[block][s][c] = sum_{m in block} dz[m,c] * h[m,s,c]
// (reference: `sublayer_read(grad, beta)` + `_weights_backward(grad, updates, beta)`,
//  sihc/models/sihc/sublayer_kernels.py:300-303)
template <typename T, typename W, int S, int V, int TT>
__global__ void __launch_bounds__(kMaxThreads) write_bwd1_kernel(const __grid_constant__ WriteBwd1Params p) {
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
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
        const uint32_t per_tile = t.tl * TT;
        for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
            Raw hr[TT][S];
            Raw dr[TT];
            uint32_t m[TT];
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                m[i] = tile * per_tile + i * t.tl + ln.tl;
                const bool ok = m[i] < t.M;
                const T* cell = h + cell_origin<S>(ok ? m[i] : 0u, t.g, t.C);
                dr[i] = (ok && want_w) ? IO::load_raw(dz + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
#pragma unroll
                for (int s = 0; s < S; ++s) hr[i][s] = ok ? IO::load_raw(cell + slot_offset<S>(s, t.g, t.C)) : IO::zero_raw();
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                float dv[V];
                float z[V];
                IO::unpack(dr[i], dv);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    float hv[V];
                    IO::unpack(hr[i][s], hv);
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        z[v] = s == 0 ? hv[v] * w1[0][v] : fmaf(hv[v], w1[s][v], z[v]);
                        acc[s][v] = fmaf(hv[v], dv[v], acc[s][v]);
                    }
                }
                if (ddz != nullptr && m[i] < t.M) IO::store(ddz + static_cast<size_t>(m[i]) * t.C, z);
            }
        }
    }
    if (p.partial != nullptr)
        block_reduce_rows<S, V>(acc, p.partial + static_cast<size_t>(blockIdx.x) * S * t.C, t.C, ln.c0, ln.cl, ln.tl,
                                t.cl, t.tl, ln.active, red);
}

// ---- host launchers ------------------------------------------------------------------------------
namespace {
// Defaults from a threads x tokens-per-thread sweep on B200 (n=4, width 768, 2^19 tokens, bf16).
constexpr int kReadFwdThreads = 512, kReadFwdTT = 1;
constexpr int kWriteFwdThreads = 384, kWriteFwdTT = 2;
constexpr int kReadBwdThreads = 384, kReadBwdTT = 2;
constexpr int kWriteBwdThreads = 512, kWriteBwdTT = 2;
inline int pick_tt(int dflt) { return tuning().tt > 0 ? tuning().tt : dflt; }
}  // namespace

cudaError_t launch_read_fwd(const Problem& pb, const void* x, const void* alpha, void* const* out) {
    ReadFwdParams p{};
    p.x = x; p.w = alpha; p.E = pb.E;
    for (int l = 0; l < pb.E; ++l) p.out.p[l] = out[l];
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            if (pb.E == 1)      // pb.V was chosen with vec_width_fwd by the caller; n = 8 wants two tokens per thread
                return dispatch_vec_tt<VecWidthFwd<T, S>::value>(pb.V, pick_tt(S == 8 ? 2 : kReadFwdTT), [&](auto v_, auto t_) {
                    constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                    return launch_persistent(read_fwd_kernel<T, W, S, V, TT, true>, p, pb, V, TT, kReadFwdThreads, 1, false, nullptr);
                });
            if ((tuning().stage_smem != 0) && pb.V > 1) return launch_read_fwd_stage(pb, p);
            // The stage read is limited by re-fetching each event's coefficients from L1: four tokens per thread
            // halve that traffic (E=24, n=4: 3964 -> 4598 GB/s); the packed carrier vectors of four tokens fit the
            // 168-register budget of a 384-thread block for S*V <= 32.
            return dispatch_vec_tt<VecWidth<T, S>::value>(pb.V, pick_tt(4), [&](auto v_, auto t_) {
                constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                return launch_persistent(read_fwd_kernel<T, W, S, V, TT, false>, p, pb, V, TT, TT >= 4 ? 384 : 512, 1, false, nullptr,
                                         TT >= 4 ? 384 : kMaxThreads);
            });
        });
    });
}

cudaError_t launch_write_fwd(const Problem& pb, const void* x, const void* const* dz, const void* beta, void* y) {
    WriteFwdParams p{};
    p.x = x; p.w = beta; p.y = y; p.E = pb.E;
    for (int l = 0; l < pb.E; ++l) p.dz.p[l] = dz[l];
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            if (pb.E == 1 && dz[0] != nullptr)      // pb.V was chosen with vec_width_fwd by the caller
                return dispatch_vec_tt<VecWidthFwd<T, S>::value>(pb.V, pick_tt(VecWidthFwd<T, S>::value * S >= 64 ? 1 : kWriteFwdTT), [&](auto v_, auto t_) {
                    constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                    return launch_persistent(write_fwd_kernel<T, W, S, V, TT, true>, p, pb, V, TT, kWriteFwdThreads, 1, false, nullptr);
                });
            if ((tuning().stage_smem != 0) && pb.V > 1) return launch_write_fwd_stage(pb, p);
            return dispatch_vec_tt<VecWidth<T, S>::value>(pb.V, pick_tt(kWriteFwdTT), [&](auto v_, auto t_) {
                constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                return launch_persistent(write_fwd_kernel<T, W, S, V, TT, false>, p, pb, V, TT, 512, 1, false, nullptr);
            });
        });
    });
}

cudaError_t launch_write_read(const Problem& pb, const void* x, const void* dz, const void* beta, const void* alpha_next,
                              void* y, void* z_next) {
    WriteReadParams p{};
    p.x = x; p.dz = dz; p.beta = beta; p.alpha = alpha_next; p.y = y; p.z = z_next;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int VM = VecWidth<T, S>::value;
            if (pb.V == 1) return launch_persistent(write_read_kernel<T, W, S, 1, 1>, p, pb, 1, 1, 512, 1, false, nullptr);
            // Block size x tokens per thread, measured on B200 (bf16, width 768, 65 536 / 524 288 tokens).  With packed
            // same-type coefficients: n=4 256 x 1 (6313 / 6413 GB/s; 512 x 2: 5657 / 5897), n=2 384 x 2 (6114 / 6433),
            // n=8 512 x 2 (5874 / 5933), n=16 512 x 1 (5046 / 4791).  Unpacked coefficients: 512 x 2.
            int threads = 512, tt = 2;
            if constexpr (std::is_same<T, W>::value) {
                if (S == 4) { threads = 256; tt = 1; }
                else if (S == 2) { threads = 384; tt = 2; }
                else if (S == 16) { threads = 512; tt = 1; }
            }
            if (pick_tt(tt) >= 2) return launch_persistent(write_read_kernel<T, W, S, VM, 2>, p, pb, VM, 2, threads, 1, false, nullptr);
            return launch_persistent(write_read_kernel<T, W, S, VM, 1>, p, pb, VM, 1, threads, 1, false, nullptr);
        });
    });
}

cudaError_t launch_read_bwd1(const Problem& pb, const void* x, const void* g, const void* alpha, void* dx,
                             float* partial, uint32_t* blocks) {
    ReadBwd1Params p{};
    p.x = x; p.g = g; p.w = alpha; p.dx = dx; p.partial = partial;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            return dispatch_vec_tt<VecWidth<T, S>::value>(pb.V, pick_tt(kReadBwdTT), [&](auto v_, auto t_) {
                constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                return launch_persistent(read_bwd1_kernel<T, W, S, V, TT>, p, pb, V, TT, kReadBwdThreads, 1,
                                         partial != nullptr, blocks);
            });
        });
    });
}

cudaError_t launch_write_bwd1(const Problem& pb, const void* h, const void* dz, const void* beta, void* ddz,
                              float* partial, uint32_t* blocks) {
    WriteBwd1Params p{};
    p.h = h; p.dz = dz; p.w = beta; p.ddz = ddz; p.partial = partial;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            return dispatch_vec_tt<VecWidth<T, S>::value>(pb.V, pick_tt(kWriteBwdTT), [&](auto v_, auto t_) {
                constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                return launch_persistent(write_bwd1_kernel<T, W, S, V, TT>, p, pb, V, TT, kWriteBwdThreads, 1,
                                         partial != nullptr, blocks);
            });
        });
    });
}

}  // namespace sihc
