// Stage weight-gradient reduction, its finishing pass, and the triangular kernels.
//
// Every reduction over tokens is deterministic: a block accumulates its tokens
// in registers, reduces its token lanes through shared memory in fixed order
// and writes one fp32 row set to scratch; a finishing kernel then adds the
// block rows in fixed order.  No atomics (the reference's `_weight_grad*` and
// `_triangular_gamma_grad` kernels use relaxed fp32 atomics and are not
// run-to-run reproducible: sihc/models/sihc/sublayer_kernels.py:130-177, :324-334).
#include "sihc_dispatch.cuh"

namespace sihc {

struct TriFwdParams { const void* base; ConstPtrs dz; const void* gamma; void* out; int J; Tiling t; };
struct TriBwdParams { const void* grad; ConstPtrs dz; const void* gamma; MutPtrs ddz; int has_ddz; float* partial; int J; int chunk; Tiling t; };


// ---- stage weight gradient ---------------------------------------------------------------------
// partial[block][l][s][c] = sum_{m in block} X[m,s,c] * Z_l[m,c]   for the EC events of blockIdx.z
// (reference: `_weight_grad`, sihc/models/sihc/sublayer_kernels.py:130-145).  A null Z_l leaves
// zeros (unused read output, :283).
template <typename T, int S, int V, int TT>
__global__ void __launch_bounds__(kMaxThreads) wgrad_kernel(const __grid_constant__ WGradParams p) {
    constexpr int EC = EventChunk<S, V>::value;
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    const int e0 = blockIdx.z * EC;
    const T* __restrict__ x = static_cast<const T*>(p.x) + ln.c0;
    float acc[EC * S][V];
#pragma unroll
    for (int a = 0; a < EC * S; ++a)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[a][v] = 0.f;
    if (ln.active) {
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
            Raw zr[EC][TT];
#pragma unroll
            for (int j = 0; j < EC; ++j) {
                const int l = e0 + j;
                const bool have = l < p.E && p.z.p[l] != nullptr;
                const T* __restrict__ z = have ? static_cast<const T*>(p.z.p[l]) + ln.c0 : nullptr;
#pragma unroll
                for (int i = 0; i < TT; ++i)
                    zr[j][i] = (have && m[i] < t.M) ? IO::load_raw(z + static_cast<size_t>(m[i]) * t.C) : IO::zero_raw();
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) {
#pragma unroll
                for (int s = 0; s < S; ++s) {
#pragma unroll
                    for (int j = 0; j < EC; ++j) IO::fma_raw(xr[i][s], zr[j][i], acc[j * S + s]);
                }
            }
        }
    }
    // rows of this chunk: (e0*S) .. ; rows beyond E*S are not written
    const uint32_t rows_total = static_cast<uint32_t>(p.E) * S;
    float* dst = p.partial + (static_cast<size_t>(blockIdx.x) * rows_total + static_cast<size_t>(e0) * S) * t.C;
    const int live = (p.E - e0 < EC ? p.E - e0 : EC) * S;
    // block_reduce_rows writes A rows; mask the tail chunk by reducing row by row
#pragma unroll
    for (int a = 0; a < EC * S; ++a) {
        float one[1][V];
#pragma unroll
        for (int v = 0; v < V; ++v) one[0][v] = acc[a][v];
        if (a < live)   // uniform across the block
            block_reduce_rows<1, V>(one, dst + static_cast<size_t>(a) * t.C, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl,
                                    ln.active, red);
    }
}

// ---- finishing pass ------------------------------------------------------------------------------
// out[(row / S) * C * S + c * S + row % S] = sum_{p < blocks} partial[(p * rows + row) * C + c]
// i.e. [E][S][C] block rows -> the parameter layout [E][C][S].  Fixed summation order.
__global__ void __launch_bounds__(256) finish_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                     uint32_t blocks, uint32_t rows, uint32_t C, uint32_t S) {
    __shared__ float red[8][32];
    const uint32_t lane = threadIdx.x, py = threadIdx.y;
    const size_t idx = static_cast<size_t>(blockIdx.x) * 32 + lane;     // over rows * C
    const size_t total = static_cast<size_t>(rows) * C;
    float sum = 0.f;
    if (idx < total) {
        const size_t stride = total;
        for (uint32_t q = py; q < blocks; q += 8) sum += partial[static_cast<size_t>(q) * stride + idx];
    }
    red[py][lane] = sum;
    __syncthreads();
    if (py == 0 && idx < total) {
        float s = red[0][lane];
#pragma unroll
        for (int k = 1; k < 8; ++k) s += red[k][lane];
        const uint32_t row = static_cast<uint32_t>(idx / C), c = static_cast<uint32_t>(idx % C);
        out[(static_cast<size_t>(row / S) * C + c) * S + row % S] = s;
    }
}

// ---- triangular accumulation, forward --------------------------------------------------------
// out = base + sum_{l<J} gamma[l,c] * dz_l   (reference: `_triangular`,
// sihc/models/sihc/sublayer_kernels.py:309-321).  Pure streaming: J + 2 elements per (m,c).
template <typename T, typename W, int V, int TT>
__global__ void __launch_bounds__(kMaxThreads) tri_fwd_kernel(const __grid_constant__ TriFwdParams p) {
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    if (!ln.active) return;
    const T* __restrict__ base = static_cast<const T*>(p.base) + ln.c0;
    T* __restrict__ out = static_cast<T*>(p.out) + ln.c0;
    const W* __restrict__ gamma = static_cast<const W*>(p.gamma) + ln.c0;
    const uint32_t per_tile = t.tl * TT;
    for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
        float acc[TT][V];
        size_t off[TT];
        bool ok[TT];
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            const uint32_t m = tile * per_tile + i * t.tl + ln.tl;
            ok[i] = m < t.M;
            off[i] = static_cast<size_t>(ok[i] ? m : 0u) * t.C;
            if (ok[i]) VecIO<T, V>::load(base + off[i], acc[i]);
            else {
#pragma unroll
                for (int v = 0; v < V; ++v) acc[i][v] = 0.f;
            }
        }
        int l = 0;
        for (; l + 4 <= p.J; l += 4) {      // four independent update streams in flight
            typename VecIO<T, V>::Raw d[4][TT];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const T* __restrict__ dz = static_cast<const T*>(p.dz.p[l + k]) + ln.c0;
#pragma unroll
                for (int i = 0; i < TT; ++i) d[k][i] = ok[i] ? VecIO<T, V>::load_raw(dz + off[i]) : VecIO<T, V>::zero_raw();
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float gm[1][V];
                load_coeffs<W, 1, V>(gamma + static_cast<size_t>(l + k) * t.C, gm);
#pragma unroll
                for (int i = 0; i < TT; ++i) {
                    float dv[V];
                    VecIO<T, V>::unpack(d[k][i], dv);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[i][v] = fmaf(dv[v], gm[0][v], acc[i][v]);
                }
            }
        }
        for (; l < p.J; ++l) {
            const T* __restrict__ dz = static_cast<const T*>(p.dz.p[l]) + ln.c0;
            float gm[1][V];
            load_coeffs<W, 1, V>(gamma + static_cast<size_t>(l) * t.C, gm);
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                if (ok[i]) {
                    float d[V];
                    VecIO<T, V>::load(dz + off[i], d);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[i][v] = fmaf(d[v], gm[0][v], acc[i][v]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TT; ++i)
            if (ok[i]) VecIO<T, V>::store(out + off[i], acc[i]);
    }
}

// ---- triangular accumulation, backward ------------------------------------------------------
// ddz_l = grad * gamma_l (optional); partial[block][l][c] = sum_{m in block} grad[m,c] * dz_l[m,c]
// for the JC events of blockIdx.z  (reference: `_tri_autograd`, `_triangular_gamma_grad`,
// sihc/models/sihc/sublayer_kernels.py:369-379, :324-334).
// JC = event slots per z-slice (2, 4 or 8), TT = tokens per thread; JC*TT update vectors are in flight per
// thread, so short prefixes trade unused event slots for more tokens.
// Events per z-slice (the largest the kernel is built for, and the default).  Measured on B200, bf16, both outputs:
// slices of at most 4 events with two tokens per thread beat slices of up to 8 with one token for every J >= 5
// (width 768, 65 536 tokens: J=12 5271 -> 6085, J=23 5559 -> 6034 GB/s; width 1152, 8192 tokens: J=23 4743 -> 5271).
constexpr int kTriMaxChunk = 8;
constexpr int kTriChunk = 4;
template <typename T, typename W, int V, int TT, int JC>
__global__ void __launch_bounds__(kMaxThreads) tri_bwd_kernel(const __grid_constant__ TriBwdParams p) {
    __shared__ float red[kMaxThreads * V];
    const Tiling& t = p.t;
    const Lane ln = make_lane<V>(t);
    // events [e0, e1) of this z-slice: J spread over the slices so that they differ by at most one (<= JC each)
    const int e0 = static_cast<int>(blockIdx.z) * p.J / static_cast<int>(gridDim.z);
    const int e1 = static_cast<int>(blockIdx.z + 1) * p.J / static_cast<int>(gridDim.z);
    const T* __restrict__ grad = static_cast<const T*>(p.grad) + ln.c0;
    float acc[JC][V];
#pragma unroll
    for (int a = 0; a < JC; ++a)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[a][v] = 0.f;
    if (ln.active) {
        const W* __restrict__ gamma = static_cast<const W*>(p.gamma) + ln.c0;
        const uint32_t per_tile = t.tl * TT;
        for (uint32_t tile = blockIdx.x; tile < t.ntiles; tile += gridDim.x) {
            typename VecIO<T, V>::Raw gr[TT];
            float gv[TT][V];
            size_t off[TT];
            bool ok[TT];
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                const uint32_t m = tile * per_tile + i * t.tl + ln.tl;
                ok[i] = m < t.M;
                off[i] = static_cast<size_t>(ok[i] ? m : 0u) * t.C;
                gr[i] = ok[i] ? VecIO<T, V>::load_raw(grad + off[i]) : VecIO<T, V>::zero_raw();
            }
            // issue every update load of the chunk before the first use (JC*TT vectors in flight)
            typename VecIO<T, V>::Raw dr[JC][TT];
#pragma unroll
            for (int j = 0; j < JC; ++j) {
                const int l = e0 + j;
                const bool have = l < e1 && p.partial != nullptr;
                const T* __restrict__ dz = have ? static_cast<const T*>(p.dz.p[l]) + ln.c0 : nullptr;
#pragma unroll
                for (int i = 0; i < TT; ++i)
                    dr[j][i] = (have && ok[i]) ? VecIO<T, V>::load_raw(dz + off[i]) : VecIO<T, V>::zero_raw();
            }
#pragma unroll
            for (int i = 0; i < TT; ++i) VecIO<T, V>::unpack(gr[i], gv[i]);     // for the ddz products
#pragma unroll
            for (int j = 0; j < JC; ++j) {
                const int l = e0 + j;
                if (l < e1) {
#pragma unroll
                    for (int i = 0; i < TT; ++i) VecIO<T, V>::fma_raw(gr[i], dr[j][i], acc[j]);
                    if (p.has_ddz && p.ddz.p[l] != nullptr) {
                        T* __restrict__ ddz = static_cast<T*>(p.ddz.p[l]) + ln.c0;
                        float gm[1][V];
                        load_coeffs<W, 1, V>(gamma + static_cast<size_t>(l) * t.C, gm);
#pragma unroll
                        for (int i = 0; i < TT; ++i) {
                            if (ok[i]) {
                                float r[V];
#pragma unroll
                                for (int v = 0; v < V; ++v) r[v] = gv[i][v] * gm[0][v];
                                VecIO<T, V>::store(ddz + off[i], r);
                            }
                        }
                    }
                }
            }
        }
    }
    if (p.partial != nullptr) {
        float* dst = p.partial + (static_cast<size_t>(blockIdx.x) * p.J + e0) * t.C;
        const int live = e1 - e0;
#pragma unroll
        for (int a = 0; a < JC; ++a) {
            float one[1][V];
#pragma unroll
            for (int v = 0; v < V; ++v) one[0][v] = acc[a][v];
            if (a < live)
                block_reduce_rows<1, V>(one, dst + static_cast<size_t>(a) * t.C, t.C, ln.c0, ln.cl, ln.tl, t.cl, t.tl,
                                        ln.active, red);
        }
    }
}

// ---- store-stream probe -------------------------------------------------------------------------
// Nothing but 16-byte `st.global.cs` stores over a persistent grid: the write-only bandwidth of the device, which is
// what bounds kernels whose traffic is mostly output (the 24-event stage read writes 24 of its 28 elements).
__global__ void __launch_bounds__(512) store_stream_kernel(uint4* __restrict__ dst, size_t vectors) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vectors; i += stride)
        st_stream(dst + i, make_uint4(0u, 0u, 0u, 0u));
}

cudaError_t launch_store_stream(void* dst, size_t bytes, cudaStream_t stream) {
    const int nb = occupancy_blocks(store_stream_kernel, 512);
    store_stream_kernel<<<static_cast<uint32_t>(sm_count() * nb), 512, 0, stream>>>(static_cast<uint4*>(dst), bytes / 16);
    count_launch();
    return cudaGetLastError();
}

// ---- host launchers ------------------------------------------------------------------------------
namespace {
constexpr int kTT = 2;
inline int pick_tt(int dflt) { return tuning().tt > 0 ? tuning().tt : dflt; }

template <typename F>
inline cudaError_t dispatch_tri_vec(DType dtype, int V, int tt, F&& f) {
    if (V == 1) return f(Int<1>{}, Int<1>{});
    if (dtype == kBF16) {
        if (tt >= 4) return f(Int<8>{}, Int<4>{});
        if (tt >= 2) return f(Int<8>{}, Int<2>{});
        return f(Int<8>{}, Int<1>{});
    }
    if (tt >= 4) return f(Int<4>{}, Int<4>{});
    if (tt >= 2) return f(Int<4>{}, Int<2>{});
    return f(Int<4>{}, Int<1>{});
}
}  // namespace

cudaError_t launch_wgrad(const Problem& pb, const void* carrier, const void* const* z, float* partial,
                         uint32_t* blocks) {
    WGradParams p{};
    p.x = carrier; p.partial = partial; p.E = pb.E;
    for (int l = 0; l < pb.E; ++l) p.z.p[l] = z[l];
    return dispatch_types(pb.dtype, pb.dtype, [&](auto tt_, auto) {     // weights are not read here
        using T = decltype(tt_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            return dispatch_vec_tt<VecWidth<T, S>::value>(pb.V, pick_tt(kTT), [&](auto v_, auto t_) {
                constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
                constexpr int EC = EventChunk<S, V>::value;
                const uint32_t gz = static_cast<uint32_t>((pb.E + EC - 1) / EC);
                return launch_persistent(wgrad_kernel<T, S, V, TT>, p, pb, V, TT, 512, gz, true, blocks);
            });
        });
    });
}

cudaError_t launch_finish(const float* partial, float* out, uint32_t blocks, uint32_t rows, uint32_t C, uint32_t S,
                          cudaStream_t stream) {
    const size_t total = static_cast<size_t>(rows) * C;
    const uint32_t gx = static_cast<uint32_t>((total + 31) / 32);
    finish_kernel<<<gx, dim3(32, 8), 0, stream>>>(partial, out, blocks, rows, C, S);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_tri_fwd(const Problem& pb, const void* base, const void* const* dz, const void* gamma, void* out) {
    TriFwdParams p{};
    p.base = base; p.gamma = gamma; p.out = out; p.J = pb.E;
    for (int l = 0; l < pb.E; ++l) p.dz.p[l] = dz[l];
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        return dispatch_tri_vec(pb.dtype, pb.V, pick_tt(1), [&](auto v_, auto t_) {
            constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value;
            if constexpr (V > 16 / int(sizeof(T))) return cudaErrorInvalidValue;
            else return launch_persistent(tri_fwd_kernel<T, W, V, TT>, p, pb, V, TT, 256, 1, false, nullptr);
        });
    });
}

cudaError_t launch_tri_bwd(const Problem& pb, const void* grad, const void* const* dz, const void* gamma,
                           void* const* ddz, float* partial, uint32_t* blocks) {
    TriBwdParams p{};
    p.grad = grad; p.gamma = gamma; p.partial = partial; p.J = pb.E; p.has_ddz = ddz != nullptr;
    for (int l = 0; l < pb.E; ++l) { p.dz.p[l] = dz[l]; p.ddz.p[l] = ddz ? ddz[l] : nullptr; }
    const int max_chunk = tuning().tri_chunk > 0 && tuning().tri_chunk <= kTriMaxChunk ? tuning().tri_chunk : kTriChunk;
    const uint32_t gz = static_cast<uint32_t>((pb.E + max_chunk - 1) / max_chunk);
    p.chunk = (pb.E + static_cast<int>(gz) - 1) / static_cast<int>(gz);     // largest slice, e.g. 13 events -> 4, 3, 3, 3
    const int forced_tt = tuning().tt;
    return dispatch_types(pb.dtype, pb.wdtype, [&](auto tt_, auto ww_) {
        using T = decltype(tt_); using W = decltype(ww_);
        constexpr int VF = 16 / int(sizeof(T));
        auto go = [&](auto v_, auto t_, auto j_) {
            constexpr int V = decltype(v_)::value; constexpr int TT = decltype(t_)::value; constexpr int JC = decltype(j_)::value;
            return launch_persistent(tri_bwd_kernel<T, W, V, TT, JC>, p, pb, V, TT, 512, gz, partial != nullptr, blocks);
        };
        if (pb.V == 1) return go(Int<1>{}, Int<1>{}, Int<8>{});
        if (forced_tt <= 0 && p.chunk <= 2) return go(Int<VF>{}, Int<4>{}, Int<2>{});
        if (forced_tt <= 0 && p.chunk <= 4) return go(Int<VF>{}, Int<2>{}, Int<4>{});
        return go(Int<VF>{}, Int<1>{}, Int<8>{});
    });
}

}  // namespace sihc
