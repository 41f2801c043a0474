// Shared device helpers for the SiHC routing kernels (sm_100a).
//
// Layout facts every kernel relies on (reference geometry: `_high_offsets`,
// sihc/models/sihc/sublayer_kernels.py:21-25):
//   * the NHWC carrier [B, g*KH, g*KW, C] is, without any copy, the 5-D array
//     [B*g (token rows), KH, g (tokens in the row), KW, C]; the S = KH*KW slot
//     vectors of one token are KH runs of KW*C contiguous elements, and the
//     whole cell block of one token row is one contiguous span of g*S*C elements;
//   * workspace tensors are [B*g*g tokens, C] row-major;
//   * weights are [E, C, S]: for V adjacent channels of one event the V*S
//     coefficients are contiguous, so a thread owning V channels fetches its
//     coefficients with full-width vector loads from the native layout.
//
// Thread mapping used by all streaming kernels: a block is CL channel lanes x
// TL token lanes (threadIdx.x = tl*CL + cl).  A thread owns V adjacent
// channels (one 16-byte vector in the fast path) and walks tokens
// tile*TL*TT + t*TL + tl, t < TT, over a persistent grid-stride tile loop, so
// every global access of a warp is a contiguous run of 16-byte vectors.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sihc {

constexpr int kMaxEvents = 24;
constexpr int kMaxThreads = 512;

typedef unsigned short bf16_t;   // raw bf16 storage; arithmetic is always fp32

struct ConstPtrs { const void* p[kMaxEvents]; };
struct MutPtrs { void* p[kMaxEvents]; };

// Slot grid per slot count (row-major slot numbering s = uy*KW + ux).
template <int S> struct Cell;
template <> struct Cell<2>  { static constexpr int KH = 1, KW = 2; };
template <> struct Cell<4>  { static constexpr int KH = 2, KW = 2; };
template <> struct Cell<8>  { static constexpr int KH = 2, KW = 4; };
template <> struct Cell<16> { static constexpr int KH = 4, KW = 4; };

// Block/grid decomposition computed on the host.
struct Tiling {
    uint32_t M;        // workspace tokens
    uint32_t g;        // tokens per carrier row
    uint32_t C;        // channels
    uint32_t ncv;      // channel vectors = C / V
    uint32_t cl;       // channel lanes per block
    uint32_t tl;       // token lanes per block
    uint32_t ntiles;   // token tiles of tl*TT tokens
};

// Per-thread identity inside the CL x TL block.
struct Lane {
    uint32_t cl, tl, c0;
    bool active;
};
template <int V>
__device__ __forceinline__ Lane make_lane(const Tiling& t) {
    Lane l;
    l.cl = threadIdx.x % t.cl;
    l.tl = threadIdx.x / t.cl;
    const uint32_t cv = blockIdx.y * t.cl + l.cl;
    l.active = cv < t.ncv && l.tl < t.tl;
    l.c0 = cv * V;
    return l;
}

// ---- cache-hinted vector access ------------------------------------------------
// Activations are touched exactly once per kernel.  Measured on B200 (n=4, width 768, 2^20 tokens, bf16):
// streaming STORES (st.global.cs) help, but evict-first LOADS (ld.global.cs) cost ~4 % against the
// read-only path (read fwd 6397 vs 6691 GB/s, write fwd 6285 vs 6510), so loads use ld.global.nc.
#ifndef SIHC_LOAD_MODE
#define SIHC_LOAD_MODE 1      // 0 plain, 1 ld.global.nc, 2 ld.global.cs
#endif
#ifndef SIHC_STORE_MODE
#define SIHC_STORE_MODE 1     // 0 plain, 1 st.global.cs
#endif

template <typename Q> __device__ __forceinline__ Q ld_stream(const Q* p) {
#if SIHC_LOAD_MODE == 2
    return __ldcs(p);
#elif SIHC_LOAD_MODE == 1
    return __ldg(p);
#else
    return *p;
#endif
}
template <typename Q> __device__ __forceinline__ void st_stream(Q* p, Q v) {
#if SIHC_STORE_MODE == 1
    __stcs(p, v);
#else
    *p = v;
#endif
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;   // round-to-nearest-even, first source operand lands in the upper half
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// acc += a * b for the two bf16 pairs packed in a and b, each product formed exactly and added to the fp32
// accumulator with one rounding (`fma.rn.f32.bf16`, sm_100+): the same value as fmaf(float(a), float(b), acc)
// without spending integer-pipe instructions on widening the operands first.
#ifndef SIHC_MIXED_FMA
#define SIHC_MIXED_FMA 1
#endif
__device__ __forceinline__ void fma_bf16x2(uint32_t a, uint32_t b, float& acc_lo, float& acc_hi) {
#if SIHC_MIXED_FMA
    asm("{\n\t"
        ".reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %2;\n\t"
        "mov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n\t"
        "fma.rn.f32.bf16 %1, ah, bh, %1;\n\t"
        "}"
        : "+f"(acc_lo), "+f"(acc_hi) : "r"(a), "r"(b));
#else
    acc_lo = fmaf(__uint_as_float(a << 16), __uint_as_float(b << 16), acc_lo);
    acc_hi = fmaf(__uint_as_float(a & 0xffff0000u), __uint_as_float(b & 0xffff0000u), acc_hi);
#endif
}
__device__ __forceinline__ bf16_t pack_bf16(float f) {
    bf16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}

template <typename T, int V> struct VecIO;

template <int BYTES> struct RawBits;
template <> struct RawBits<16> { typedef uint4 type; };
template <> struct RawBits<8> { typedef uint2 type; };
template <> struct RawBits<4> { typedef uint32_t type; };
template <> struct RawBits<2> { typedef unsigned short type; };

// `Raw` is the packed register image of V elements: loads are kept packed while
// they are in flight and expanded to fp32 only where they are consumed, which
// halves the registers tied up by outstanding bf16 loads.
template <int V> struct VecIO<float, V> {
    static_assert(V == 1 || V == 2 || V == 4, "fp32 vector width");
    typedef typename RawBits<4 * V>::type Raw;
    static __device__ __forceinline__ Raw load_raw(const float* p) { return ld_stream(reinterpret_cast<const Raw*>(p)); }
    // coherent load: for memory the same kernel also writes (the read-only path requires data that never changes)
    static __device__ __forceinline__ Raw load_raw_coherent(const float* p) { return *reinterpret_cast<const Raw*>(p); }
    static __device__ __forceinline__ Raw zero_raw() { return Raw(); }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[V]) {
        if constexpr (V == 4) { f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w); }
        else if constexpr (V == 2) { f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); }
        else { f[0] = __uint_as_float(r); }
    }
    static __device__ __forceinline__ void fma_raw(const Raw& a, const Raw& b, float (&acc)[V]) {   // acc += a * b
        float fa[V], fb[V];
        unpack(a, fa); unpack(b, fb);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = fmaf(fa[v], fb[v], acc[v]);
    }
    static __device__ __forceinline__ void load(const float* p, float (&f)[V]) {
        if constexpr (V == 4) { float4 q = ld_stream(reinterpret_cast<const float4*>(p)); f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w; }
        else if constexpr (V == 2) { float2 q = ld_stream(reinterpret_cast<const float2*>(p)); f[0] = q.x; f[1] = q.y; }
        else { f[0] = ld_stream(p); }
    }
    static __device__ __forceinline__ Raw pack(const float (&f)[V]) {
        if constexpr (V == 4) return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
        else if constexpr (V == 2) return make_uint2(__float_as_uint(f[0]), __float_as_uint(f[1]));
        else return __float_as_uint(f[0]);
    }
    static __device__ __forceinline__ void store_raw(float* p, const Raw& r) { st_stream(reinterpret_cast<Raw*>(p), r); }
    static __device__ __forceinline__ void store(float* p, const float (&f)[V]) {
        if constexpr (V == 4) st_stream(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
        else if constexpr (V == 2) st_stream(reinterpret_cast<float2*>(p), make_float2(f[0], f[1]));
        else st_stream(p, f[0]);
    }
};

template <int V> struct VecIO<bf16_t, V> {
    static_assert(V == 1 || V == 2 || V == 4 || V == 8, "bf16 vector width");
    typedef typename RawBits<2 * V>::type Raw;
    static __device__ __forceinline__ Raw load_raw(const bf16_t* p) { return ld_stream(reinterpret_cast<const Raw*>(p)); }
    static __device__ __forceinline__ Raw load_raw_coherent(const bf16_t* p) { return *reinterpret_cast<const Raw*>(p); }
    static __device__ __forceinline__ Raw zero_raw() { return Raw(); }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&f)[V]) {
        if constexpr (V == 8) {
            f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
            f[4] = bf16_lo(r.z); f[5] = bf16_hi(r.z); f[6] = bf16_lo(r.w); f[7] = bf16_hi(r.w);
        } else if constexpr (V == 4) {
            f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
        } else if constexpr (V == 2) {
            f[0] = bf16_lo(r); f[1] = bf16_hi(r);
        } else {
            f[0] = __uint_as_float(static_cast<uint32_t>(r) << 16);
        }
    }
    static __device__ __forceinline__ void fma_raw(const Raw& a, const Raw& b, float (&acc)[V]) {   // acc += a * b
        if constexpr (V == 8) {
            fma_bf16x2(a.x, b.x, acc[0], acc[1]); fma_bf16x2(a.y, b.y, acc[2], acc[3]);
            fma_bf16x2(a.z, b.z, acc[4], acc[5]); fma_bf16x2(a.w, b.w, acc[6], acc[7]);
        } else if constexpr (V == 4) {
            fma_bf16x2(a.x, b.x, acc[0], acc[1]); fma_bf16x2(a.y, b.y, acc[2], acc[3]);
        } else if constexpr (V == 2) {
            fma_bf16x2(a, b, acc[0], acc[1]);
        } else {
            acc[0] = fmaf(__uint_as_float(static_cast<uint32_t>(a) << 16), __uint_as_float(static_cast<uint32_t>(b) << 16), acc[0]);
        }
    }
    static __device__ __forceinline__ void load(const bf16_t* p, float (&f)[V]) {
        if constexpr (V == 8) {
            uint4 q = ld_stream(reinterpret_cast<const uint4*>(p));
            f[0] = bf16_lo(q.x); f[1] = bf16_hi(q.x); f[2] = bf16_lo(q.y); f[3] = bf16_hi(q.y);
            f[4] = bf16_lo(q.z); f[5] = bf16_hi(q.z); f[6] = bf16_lo(q.w); f[7] = bf16_hi(q.w);
        } else if constexpr (V == 4) {
            uint2 q = ld_stream(reinterpret_cast<const uint2*>(p));
            f[0] = bf16_lo(q.x); f[1] = bf16_hi(q.x); f[2] = bf16_lo(q.y); f[3] = bf16_hi(q.y);
        } else if constexpr (V == 2) {
            uint32_t q = ld_stream(reinterpret_cast<const uint32_t*>(p));
            f[0] = bf16_lo(q); f[1] = bf16_hi(q);
        } else {
            f[0] = __uint_as_float(static_cast<uint32_t>(ld_stream(p)) << 16);
        }
    }
    static __device__ __forceinline__ Raw pack(const float (&f)[V]) {      // round-to-nearest-even to storage
        if constexpr (V == 8) return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        else if constexpr (V == 4) return make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
        else if constexpr (V == 2) return pack_bf16x2(f[0], f[1]);
        else return pack_bf16(f[0]);
    }
    static __device__ __forceinline__ void store_raw(bf16_t* p, const Raw& r) { st_stream(reinterpret_cast<Raw*>(p), r); }
    static __device__ __forceinline__ void store(bf16_t* p, const float (&f)[V]) {
        if constexpr (V == 8) {
            st_stream(reinterpret_cast<uint4*>(p), make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                              pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7])));
        } else if constexpr (V == 4) {
            st_stream(reinterpret_cast<uint2*>(p), make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3])));
        } else if constexpr (V == 2) {
            st_stream(reinterpret_cast<uint32_t*>(p), pack_bf16x2(f[0], f[1]));
        } else {
            st_stream(p, pack_bf16(f[0]));
        }
    }
};

template <typename W> __device__ __forceinline__ float w_to_float(W w);
template <> __device__ __forceinline__ float w_to_float<float>(float w) { return w; }
template <> __device__ __forceinline__ float w_to_float<bf16_t>(bf16_t w) { return __uint_as_float(static_cast<uint32_t>(w) << 16); }

// Coefficients of one event for this thread's V channels: w[s][v] = Wt[c0+v][s].
// `p` points at Wt[c0][0]; the V*S values are contiguous.  The vector path
// (V > 1) requires a 16-byte aligned weight tensor; the scalar path loads
// element-wise and has no alignment requirement beyond the element size.
template <typename W, int S, int V>
__device__ __forceinline__ void load_coeffs(const W* __restrict__ p, float (&w)[S][V]) {
    constexpr int N = S * V;
    constexpr int BYTES = N * int(sizeof(W));
    if constexpr (V > 1 && BYTES % 16 == 0) {
        constexpr int NQ = BYTES / 16;
        constexpr int PER = 16 / int(sizeof(W));
        float flat[N];
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + q);
            if constexpr (sizeof(W) == 4) {
                flat[q * PER + 0] = __uint_as_float(u.x); flat[q * PER + 1] = __uint_as_float(u.y);
                flat[q * PER + 2] = __uint_as_float(u.z); flat[q * PER + 3] = __uint_as_float(u.w);
            } else {
                flat[q * PER + 0] = bf16_lo(u.x); flat[q * PER + 1] = bf16_hi(u.x);
                flat[q * PER + 2] = bf16_lo(u.y); flat[q * PER + 3] = bf16_hi(u.y);
                flat[q * PER + 4] = bf16_lo(u.z); flat[q * PER + 5] = bf16_hi(u.z);
                flat[q * PER + 6] = bf16_lo(u.w); flat[q * PER + 7] = bf16_hi(u.w);
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int s = 0; s < S; ++s) w[s][v] = flat[v * S + s];
    } else {
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int s = 0; s < S; ++s) w[s][v] = w_to_float<W>(__ldg(p + v * S + s));
    }
}

// Element offset of token m's cell origin (slot 0, channel 0) in the carrier.
template <int S>
__device__ __forceinline__ size_t cell_origin(uint32_t m, uint32_t g, uint32_t C) {
    const uint32_t wx = m % g;
    return (static_cast<size_t>(m - wx) * S + static_cast<size_t>(wx) * Cell<S>::KW) * C;
}
// Element offset of slot s relative to the cell origin.
template <int S>
__device__ __forceinline__ uint32_t slot_offset(int s, uint32_t g, uint32_t C) {
    return (static_cast<uint32_t>(s / Cell<S>::KW) * g * Cell<S>::KW + static_cast<uint32_t>(s % Cell<S>::KW)) * C;
}

// Deterministic block reduction of per-thread partial sums over the TL token
// lanes, written as one fp32 row set per block:
//   dst[(row0 + a) * C + c0 + v] = sum over token lanes of acc[a][v]
// in fixed lane order.  All threads of the block must call this.
template <int A, int V>
__device__ __forceinline__ void block_reduce_rows(float (&acc)[A][V], float* __restrict__ dst, uint32_t C,
                                                  uint32_t c0, uint32_t cl_idx, uint32_t tl_idx,
                                                  uint32_t CL, uint32_t TL, bool active, float* red) {
#pragma unroll
    for (int a = 0; a < A; ++a) {   // fully unrolled: acc must stay in registers
        if (active && tl_idx > 0) {
            float* r = red + (static_cast<size_t>(tl_idx - 1) * CL + cl_idx) * V;
#pragma unroll
            for (int v = 0; v < V; ++v) r[v] = acc[a][v];
        }
        __syncthreads();
        if (active && tl_idx == 0) {
            float sum[V];
#pragma unroll
            for (int v = 0; v < V; ++v) sum[v] = acc[a][v];
            for (uint32_t j = 0; j + 1 < TL; ++j) {
                const float* r = red + (static_cast<size_t>(j) * CL + cl_idx) * V;
#pragma unroll
                for (int v = 0; v < V; ++v) sum[v] += r[v];
            }
            float* d = dst + static_cast<size_t>(a) * C + c0;
#pragma unroll
            for (int v = 0; v < V; ++v) d[v] = sum[v];
        }
        __syncthreads();
    }
}

}  // namespace sihc
