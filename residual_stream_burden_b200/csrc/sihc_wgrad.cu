// Stage weight gradient, block-tiled:  partial[block][l][s][c] = sum_{m in block} X[m,s,c] * Z_l[m,c].
//
// `wgrad_kernel` (sihc_reduce.cu) gives each thread EC events and lets the grid's z-slices re-read the carrier once per
// EC events; those re-reads are L2 hits, but at 24 events they are 12 passes over the carrier through L2.  Here a block
// owns a channel slice (CL lanes of V channels) and ALL events: thread (lane, group) accumulates the EC events of its
// group for its lane's channels over every token the block visits.  The carrier tile of a few tokens is copied once
// per block into shared memory (`cp.async`, NST stages) and read by every event group; each thread's own Z vectors
// travel through private ring slots.  Global traffic is S + E units, and since a (lane, group) pair is unique in the
// block its accumulators ARE the block's partial sums: no block reduction.
// (reference: `_weight_grad`, sihc/models/sihc/sublayer_kernels.py:130-145; a null Z_l leaves zeros, :283)
#include "sihc_dispatch.cuh"
#include "sihc_ring.cuh"

namespace sihc {

constexpr int kWGradTileThreads = 384;        // launch bound; the `threads` knob may ask for up to this many
constexpr int kWGradTileDefaultThreads = 192; // default target: two blocks per SM overlap each other's tile barriers
constexpr int kWGradTileTokens = 4;      // tokens per stage and stages of the tile ring, unless dispatch_tile_shape
constexpr int kWGradTileStages = 3;      // picks the (8, 2) shape

template <typename T, int S, int V, int TK, int NST, bool READ = false, typename P = WGradParams>
__global__ void __launch_bounds__(READ ? kWGradTileDefaultThreads : kWGradTileThreads) wgrad_tiled_kernel(const __grid_constant__ P p) {
    constexpr int EC = EventChunk<S, V>::value;
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    constexpr int VB = int(sizeof(Raw));
    extern __shared__ __align__(16) unsigned char tile_bytes[];
    const Tiling& t = p.t;                       // t.cl channel lanes x t.tl event groups
    const Lane ln = make_lane<V>(t);             // ln.tl = event group
    const uint32_t CL = t.cl, nthreads = blockDim.x, tid = threadIdx.x;
    Raw* xs = reinterpret_cast<Raw*>(tile_bytes);                              // [NST][TK][S][CL]
    Raw* zs = xs + static_cast<size_t>(NST) * TK * S * CL;                     // [NST][TK * EC][nthreads], private slots
    const int e0 = static_cast<int>(ln.tl) * EC;
    const T* __restrict__ x = static_cast<const T*>(p.x);
    const uint32_t slice_c0 = blockIdx.y * CL * V;                             // first channel of the block's slice
    const uint32_t tile_vecs = TK * S * CL;

    auto issue = [&](uint32_t tile, int stage) {
        const bool live = tile < t.ntiles;
        // carrier tile: every thread copies its share of the TK*S*CL vectors
        for (uint32_t idx = tid; idx < tile_vecs; idx += nthreads) {
            const uint32_t lane = idx % CL, r = idx / CL, s = r % S, tok = r / S;
            const uint32_t m = tile * TK + tok;
            const bool ok = live && m < t.M && blockIdx.y * CL + lane < t.ncv;
            const T* src = x;
            if (ok) src = x + cell_origin<S>(m, t.g, t.C) + slot_offset<S>(static_cast<int>(s), t.g, t.C) + slice_c0 + lane * V;
            cp_async<VB>(xs + static_cast<size_t>(stage) * tile_vecs + idx, src, ok);
        }
        // this thread's own Z vectors
#pragma unroll
        for (int j = 0; j < EC; ++j) {
            const int l = e0 + j;
            const T* zl = (ln.active && l < p.E) ? static_cast<const T*>(p.z.p[l < p.E ? l : 0]) : nullptr;
#pragma unroll
            for (int tok = 0; tok < TK; ++tok) {
                const uint32_t m = tile * TK + tok;
                const bool ok = live && zl != nullptr && m < t.M;
                cp_async<VB>(zs + (static_cast<size_t>(stage) * TK * EC + tok * EC + j) * nthreads + tid,
                             ok ? zl + static_cast<size_t>(m) * t.C + ln.c0 : x, ok);
            }
        }
        cp_async_commit();
    };

    float acc[EC * S][V];
#pragma unroll
    for (int a = 0; a < EC * S; ++a)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[a][v] = 0.f;

    // READ: this thread also produces ddz for its EC events, from the same carrier tile: packed coefficients
    // w[l][c0..c0+V)[s] stay in registers (EC*S vectors), one output vector per event and token.
    Raw wr[READ ? EC * S : 1];
    T* outp[READ ? EC : 1];
    if constexpr (READ) {
#pragma unroll
        for (int j = 0; j < EC; ++j) {
            const int l = e0 + j;
            const bool live = ln.active && l < p.E;
            outp[j] = live && p.out.p[l] != nullptr ? static_cast<T*>(p.out.p[l]) + ln.c0 : nullptr;
            float f[S][V];
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int v = 0; v < V; ++v) f[s][v] = 0.f;
            if (live) load_coeffs<T, S, V>(static_cast<const T*>(p.w) + (static_cast<size_t>(l) * t.C + ln.c0) * S, f);
#pragma unroll
            for (int s = 0; s < S; ++s) wr[j * S + s] = IO::pack(f[s]);        // exact: the values are storage values
        }
    }

    uint32_t tile = blockIdx.x;
#pragma unroll
    for (int st = 0; st < NST - 1; ++st) issue(tile + st * gridDim.x, st);
    int stage = 0;
    for (; tile < t.ntiles; tile += gridDim.x) {
        cp_async_wait<NST - 2>();          // this thread's copies for the tile have landed
        __syncthreads();                   // ... and everyone else's; all threads are also done with the previous tile
        issue(tile + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
        const Raw* xt = xs + static_cast<size_t>(stage) * tile_vecs + ln.cl;
        const Raw* zt = zs + static_cast<size_t>(stage) * TK * EC * nthreads + tid;
#pragma unroll
        for (int tok = 0; tok < TK; ++tok) {
            Raw zr[EC];
#pragma unroll
            for (int j = 0; j < EC; ++j) zr[j] = zt[static_cast<size_t>(tok * EC + j) * nthreads];
            float rd[READ ? EC : 1][V];
            if constexpr (READ) {
#pragma unroll
                for (int j = 0; j < EC; ++j)
#pragma unroll
                    for (int v = 0; v < V; ++v) rd[j][v] = 0.f;
            }
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const Raw xr = xt[static_cast<size_t>(tok * S + s) * CL];
#pragma unroll
                for (int j = 0; j < EC; ++j) {
                    IO::fma_raw(xr, zr[j], acc[j * S + s]);
                    if constexpr (READ) IO::fma_raw(wr[j * S + s], xr, rd[j]);
                }
            }
            if constexpr (READ) {
                const uint32_t m = tile * TK + tok;
                if (m < t.M) {
#pragma unroll
                    for (int j = 0; j < EC; ++j)
                        if (outp[j] != nullptr) IO::store(outp[j] + static_cast<size_t>(m) * t.C, rd[j]);
                }
            }
        }
        stage = stage + 1 == NST ? 0 : stage + 1;
    }
    cp_async_wait<0>();
    if (!ln.active) return;
    const uint32_t rows_total = static_cast<uint32_t>(p.E) * S;
    float* dst = p.partial + static_cast<size_t>(blockIdx.x) * rows_total * t.C + ln.c0;
#pragma unroll
    for (int j = 0; j < EC; ++j) {
        if (e0 + j >= p.E) break;
#pragma unroll
        for (int s = 0; s < S; ++s) {
            float* d = dst + (static_cast<size_t>(e0 + j) * S + s) * t.C;
#pragma unroll
            for (int v = 0; v < V; ++v) d[v] = acc[j * S + s][v];
        }
    }
}

constexpr uint32_t kReadBwdTileLanes = 16;
constexpr uint32_t kReadBwdTileRowStride = 18;

// ---- one-pass stage read backward (4 slots) ---------------------------------------------------------------------------
//   dx[m,s,c]          = sum_l alpha[l,c,s] * g_l[m,c]
//   partial[b][l][s][c] = sum_{m in block b} X[m,s,c] * g_l[m,c]
// from ONE pass over X and the E gradients (2S + E elements per token and channel; the two-kernel form - the write kernel
// without carry for dx, then the weight gradient - reads the gradients twice: 2(S + E)).  The reference makes the same two
// passes (`_write_impl(..., add_x=False)` and `_weights_backward`, sihc/models/sihc/sublayer_kernels.py:280-284).
//
// A thread owns (channel lane, slot s, quarter q of the events): EQ = ceil(E/4) events of ONE slot.  Per token it reads
// its slot's carrier vector and its EQ gradient vectors from the block's shared tile (EQ + 1 reads for 2*EQ*V FMAs),
// accumulates dalpha for its (events, slot) - unique in the block, so no block reduction - and forms the partial
// sum_{l in quarter} alpha_l * g_l of dx for its slot; the four quarters of a (lane, slot) are four adjacent threads of a
// warp, so the partial is completed by a two-step reduce-scatter of shuffles (fixed order: deterministic), after which
// each of the four stores its V/4 channels.
template <typename T, int EQ, int TK, int NST>
__global__ void __launch_bounds__(256, 2) read_bwd_tiled_kernel(const __grid_constant__ WGradReadParams p) {
    constexpr int S = 4;
    constexpr int V = 16 / int(sizeof(T));
    constexpr int ROWS = S + 4 * EQ;                       // tile rows per token: carrier slots, then (padded) events
    constexpr uint32_t CL = kReadBwdTileLanes;             // channel vectors per block
    constexpr uint32_t RS = kReadBwdTileRowStride;         // row stride in vectors: the four adjacent rows a warp reads
                                                           // (its four quarters, or its four slots) fall in distinct banks
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    extern __shared__ __align__(16) unsigned char tile_bytes[];
    const Tiling& t = p.t;
    const uint32_t tid = threadIdx.x;
    const uint32_t q = tid & 3u, s = (tid >> 2) & 3u, lane = tid >> 4;
    const uint32_t cv = blockIdx.y * CL + lane;
    const bool active = cv < t.ncv;
    const uint32_t c0 = cv * V;
    Raw* tile = reinterpret_cast<Raw*>(tile_bytes);        // [NST][TK][ROWS][RS]; event l sits in row S + (l % EQ)*4 + l / EQ
    constexpr uint32_t stage_vecs = TK * ROWS * RS;
    const T* __restrict__ x = static_cast<const T*>(p.x);

    // Copy plan: per token the tile has ROWS x CL vectors; a thread copies vector `tid` and vector `tid + 256` of them, so
    // its rows, its lane and its source pointers are fixed for the whole launch.
    const uint32_t ln = tid & (CL - 1);
    const bool ln_ok = blockIdx.y * CL + ln < t.ncv;
    const size_t coff = static_cast<size_t>(blockIdx.y * CL + ln) * V;
    const T* src_row[2];
    uint32_t dst_row[2];
    bool is_x[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t row = (tid >> 4) + 16u * k;         // 0..31; rows >= ROWS do not exist
        is_x[k] = row < S;
        src_row[k] = nullptr;
        dst_row[k] = 0;
        if (row < S) {
            src_row[k] = x + slot_offset<S>(static_cast<int>(row), t.g, t.C) + coff;
            dst_row[k] = row * RS + ln;
        } else if (row < ROWS) {
            const uint32_t l = row - S;
            const T* gl = l < static_cast<uint32_t>(p.E) ? static_cast<const T*>(p.z.p[l]) : nullptr;
            src_row[k] = gl ? gl + coff : nullptr;
            dst_row[k] = (S + (l % EQ) * 4 + l / EQ) * RS + ln;
            if (gl == nullptr) dst_row[k] |= 0x80000000u;  // a row to zero-fill
        } else {
            dst_row[k] = 0xffffffffu;                      // nothing to copy
        }
    }

    __shared__ size_t origin[NST][TK];                     // carrier offset of each token's cell, for the dx stores
    auto issue = [&](uint32_t tl, int stage) {
        const bool live = tl < t.ntiles;
        Raw* sb = tile + static_cast<size_t>(stage) * stage_vecs;
        if (tid < TK) origin[stage][tid] = cell_origin<S>(tl * TK + tid, t.g, t.C);
#pragma unroll
        for (int tok = 0; tok < TK; ++tok) {
            const uint32_t m = tl * TK + tok;
            const bool ok = live && m < t.M && ln_ok;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                if (dst_row[k] == 0xffffffffu) continue;
                const bool fill = (dst_row[k] & 0x80000000u) != 0;
                const T* src = x;
                if (ok && !fill)
                    src = is_x[k] ? src_row[k] + cell_origin<S>(m, t.g, t.C) : src_row[k] + static_cast<size_t>(m) * t.C;
                cp_async<16>(sb + tok * (ROWS * RS) + (dst_row[k] & 0x7fffffffu), src, ok && !fill);
            }
        }
        cp_async_commit();
    };

    float acc[EQ][V];
    Raw ar[EQ];                                            // alpha[l][c0..c0+V)[s] of this thread's events, packed
#pragma unroll
    for (int j = 0; j < EQ; ++j) {
#pragma unroll
        for (int v = 0; v < V; ++v) acc[j][v] = 0.f;
        const uint32_t l = q * EQ + j;
        float f[V];
#pragma unroll
        for (int v = 0; v < V; ++v)
            f[v] = (active && l < static_cast<uint32_t>(p.E))
                       ? w_to_float<T>(__ldg(static_cast<const T*>(p.w) + (static_cast<size_t>(l) * t.C + c0 + v) * S + s)) : 0.f;
        ar[j] = IO::pack(f);                               // exact: the values are storage values
    }
    // the carrier gradient travels in out.p[0]; this thread's V/4 channels of its slot, relative to a cell origin
    T* __restrict__ dx_slot = static_cast<T*>(p.out.p[0]) + slot_offset<S>(static_cast<int>(s), t.g, t.C) + c0 +
                              (q & 1u) * (V / 2) + (q >> 1) * (V / 4);

    uint32_t tl = blockIdx.x;
#pragma unroll
    for (int st = 0; st < NST - 1; ++st) issue(tl + st * gridDim.x, st);
    int stage = 0;
    for (; tl < t.ntiles; tl += gridDim.x) {
        cp_async_wait<NST - 2>();
        __syncthreads();
        issue(tl + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
        const Raw* tb = tile + static_cast<size_t>(stage) * stage_vecs + lane;
#pragma unroll
        for (int tok = 0; tok < TK; ++tok) {
            const Raw* tr = tb + tok * (ROWS * RS);
            const Raw xr = tr[s * RS];
            float part[V];
#pragma unroll
            for (int v = 0; v < V; ++v) part[v] = 0.f;
#pragma unroll
            for (int j = 0; j < EQ; ++j) {
                const Raw gr = tr[(S + j * 4 + q) * RS];
                IO::fma_raw(xr, gr, acc[j]);
                IO::fma_raw(ar[j], gr, part);
            }
            // reduce-scatter over the four quarters: (q0 + q1) + (q2 + q3) for every channel, each thread ending up with
            // V/4 of the V sums
            float half[V / 2], mine[V / 4];
#pragma unroll
            for (int k = 0; k < V / 2; ++k) {
                const float send = (q & 1u) ? part[k] : part[k + V / 2];
                const float keep = (q & 1u) ? part[k + V / 2] : part[k];
                half[k] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
            }
#pragma unroll
            for (int k = 0; k < V / 4; ++k) {
                const float send = (q & 2u) ? half[k] : half[k + V / 4];
                const float keep = (q & 2u) ? half[k + V / 4] : half[k];
                mine[k] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
            }
            const uint32_t m = tl * TK + tok;
            if (active && m < t.M)
                VecIO<T, V / 4>::store(dx_slot + origin[stage][tok], mine);
        }
        stage = stage + 1 == NST ? 0 : stage + 1;
    }
    cp_async_wait<0>();
    if (!active || p.partial == nullptr) return;
    const uint32_t rows_total = static_cast<uint32_t>(p.E) * S;
    float* dst = p.partial + static_cast<size_t>(blockIdx.x) * rows_total * t.C + c0;
#pragma unroll
    for (int j = 0; j < EQ; ++j) {
        const uint32_t l = q * EQ + j;
        if (l >= static_cast<uint32_t>(p.E)) break;
        float* d = dst + (static_cast<size_t>(l) * S + s) * t.C;
#pragma unroll
        for (int v = 0; v < V; ++v) d[v] = acc[j][v];
    }
}

// Shape of the tile ring: (tokens per stage, stages).  What matters is how many tokens of copies a block keeps in
// flight, (stages - 1) x tokens: 8 is the optimum and 16 collapses (the threads stall issuing copies into a full
// memory queue instead of computing).  Measured on B200, bf16, 4 slots, 65 536 tokens, width 768, GB/s:
//   24 events: (4,3) two blocks per SM 4690, (8,2) one block 5027, (8,3) 3292, (4,2) 4131, (2,3) 4201
//   16 events: (4,3) 4569, (8,2) 3216, (4,2) 4233
// and at 8192 tokens, width 1152: 24 events 3924 vs 4128, 16 events 3626 vs 2812; 8 slots, 24 events: 2288 vs 2490.
// So twelve event groups take (8,2) and fewer take (4,3); the `tokens_per_thread` knob (4 or 8) forces one of them.
template <typename F> cudaError_t dispatch_tile_shape(uint32_t groups, F&& f) {
    const int forced = tuning().tt;
    const bool wide = forced == 8 || (forced != kWGradTileTokens && groups >= 12);
    if (wide) return f(std::integral_constant<int, 8>{}, std::integral_constant<int, 2>{});
    return f(std::integral_constant<int, kWGradTileTokens>{}, std::integral_constant<int, kWGradTileStages>{});
}

namespace {
template <bool READ, typename P>
cudaError_t launch_tiled(const Problem& pb, P& p, uint32_t* blocks) {
    return dispatch_types(pb.dtype, pb.dtype, [&](auto tt_, auto) {
        using T = decltype(tt_);
        return dispatch_slots(pb.S, [&](auto s_) {
            constexpr int S = decltype(s_)::value;
            constexpr int V = VecWidth<T, S>::value;
            constexpr int EC = EventChunk<S, V>::value;
            if constexpr (V * int(sizeof(T)) < 4) return cudaErrorInvalidValue;
            else return dispatch_tile_shape(static_cast<uint32_t>((pb.E + EC - 1) / EC), [&](auto tk_, auto nst_) {
                constexpr int TK = decltype(tk_)::value;
                constexpr int NST = decltype(nst_)::value;
                auto kernel = wgrad_tiled_kernel<T, S, V, TK, NST, READ, P>;
                const uint32_t ncv = pb.C / V;
                const uint32_t groups = static_cast<uint32_t>((pb.E + EC - 1) / EC);
                // channel lanes: what the block's threads and 200 KB of shared memory leave per event group, split evenly
                // over blockIdx.y (a lane costs NST*TK vectors for each of its S carrier slots and EC*groups event slots).
                // 192 threads = 16 lanes at 24 events (measured on B200, 4 slots, width 768, with three 4-token stages:
                // 384 threads 4485, 256 4489, 192 4703, 128 3247 GB/s; with two 8-token stages: 384 4060, 256 3606,
                // 192 5048; 16 events, three 4-token stages: 384 4404, 256 3774, 192 4563).
                constexpr size_t kMaxDynamic = 200 * 1024;
                const size_t vb = static_cast<size_t>(V) * sizeof(T);
                const size_t per_lane = NST * TK * vb * (static_cast<size_t>(S) + static_cast<size_t>(EC) * groups);
                uint32_t block_threads = kWGradTileDefaultThreads;
                const uint32_t limit = READ ? kWGradTileDefaultThreads : kWGradTileThreads;
                if (tuning().threads > 0) block_threads = static_cast<uint32_t>(tuning().threads) < limit ? static_cast<uint32_t>(tuning().threads) : limit;
                if (block_threads < groups) block_threads = groups;
                uint32_t max_cl = block_threads / groups;
                if (max_cl > kMaxDynamic / per_lane) max_cl = static_cast<uint32_t>(kMaxDynamic / per_lane);
                if (max_cl < 1) return cudaErrorInvalidConfiguration;
                const uint32_t gy = (ncv + max_cl - 1) / max_cl;
                const uint32_t cl = (ncv + gy - 1) / gy;
                const uint32_t threads = cl * groups;
                if (threads > limit) return cudaErrorInvalidConfiguration;
                const size_t smem = per_lane * cl;
                if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kMaxDynamic)) return e;
                Tiling& t = p.t;
                t.M = pb.M; t.g = pb.g; t.C = pb.C; t.ncv = ncv; t.cl = cl; t.tl = groups;
                t.ntiles = (pb.M + TK - 1) / TK;
                int nb = cached_occupancy(reinterpret_cast<const void*>(kernel), static_cast<int>(threads), smem);
                const int cap = tuning().rbps > 0 ? tuning().rbps : 2;
                if (nb > cap) nb = cap;
                if (nb < 1) nb = 1;
                uint32_t gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / gy;
                const uint32_t bound = partial_blocks_bound(pb.M);
                if (gx > bound) gx = bound;
                if (gx < 1) gx = 1;
                if (gx > t.ntiles) gx = t.ntiles;
                if (blocks) *blocks = gx;
                kernel<<<dim3(gx, gy, 1), threads, smem, pb.stream>>>(p);
                count_launch();
                return cudaGetLastError();
            });
        });
    });
}
}  // namespace

cudaError_t launch_wgrad_tiled(const Problem& pb, const void* carrier, const void* const* z, float* partial,
                               uint32_t* blocks) {
    WGradParams p{};
    p.x = carrier; p.partial = partial; p.E = pb.E;
    for (int l = 0; l < pb.E; ++l) p.z.p[l] = z[l];
    return launch_tiled<false>(pb, p, blocks);
}

// Fewest events at which one pass beats the two kernels (B200, bf16, 4 slots; ms one pass / two kernels):
//   write backward  E=4: 0.386 / 0.285   E=6: 0.089 / 0.098 (8192 x 1152)   E=8: 0.389 / 0.473, 0.092 / 0.116   E=12: 0.517 / 0.679
//   read backward   E=4: 0.457 / 0.294   E=8: 0.548 / 0.474, 0.116 / 0.115                     E=12: 0.576 / 0.674, 0.127 / 0.159
// (65 536 tokens x 768 unless noted).  The "one_pass_min_events" knob overrides both.
constexpr int kOnePassMinEventsWrite = 8;
constexpr int kOnePassMinEventsRead = 12;
static int one_pass_min_events(int builtin) { return tuning().one_pass_min_events > 0 ? tuning().one_pass_min_events : builtin; }

bool wgrad_tiled_read_applies(const Problem& pb) {
    return pb.V > 1 && pb.S == 4 && pb.E >= one_pass_min_events(kOnePassMinEventsWrite) && pb.E >= 2 && pb.dtype == pb.wdtype &&
           tuning().wgrad_tiled != 0;
}

cudaError_t launch_wgrad_tiled_read(const Problem& pb, const void* carrier, const void* const* z, const void* beta,
                                    void* const* ddz, float* partial, uint32_t* blocks) {
    WGradReadParams p{};
    p.x = carrier; p.partial = partial; p.E = pb.E; p.w = beta;
    for (int l = 0; l < pb.E; ++l) { p.z.p[l] = z[l]; p.out.p[l] = ddz[l]; }
    return launch_tiled<true>(pb, p, blocks);
}

bool read_bwd_tiled_applies(const Problem& pb) {
    return pb.V > 1 && pb.S == 4 && pb.E >= one_pass_min_events(kOnePassMinEventsRead) && pb.E >= 2 && pb.dtype == pb.wdtype && tuning().wgrad_tiled != 0 &&
           tuning().one_pass_adjoints != 0;
}

cudaError_t launch_read_bwd_tiled(const Problem& pb, const void* carrier, const void* const* g, const void* alpha, void* dx,
                                  float* partial, uint32_t* blocks) {
    WGradReadParams p{};
    p.x = carrier; p.partial = partial; p.E = pb.E; p.w = alpha; p.out.p[0] = dx;
    for (int l = 0; l < pb.E; ++l) p.z.p[l] = g[l];
    return dispatch_types(pb.dtype, pb.dtype, [&](auto tt_, auto) {
        using T = decltype(tt_);
        constexpr int V = 16 / int(sizeof(T));
        constexpr int TK = 4, NST = 3;
        auto go = [&](auto eq_) {
            constexpr int EQ = decltype(eq_)::value;
            auto kernel = read_bwd_tiled_kernel<T, EQ, TK, NST>;
            const uint32_t ncv = pb.C / V, cl = kReadBwdTileLanes;
            const uint32_t gy = (ncv + cl - 1) / cl;
            const size_t smem = static_cast<size_t>(NST) * TK * (4 + 4 * EQ) * kReadBwdTileRowStride * 16;
            if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024)) return e;
            Tiling& t = p.t;
            t.M = pb.M; t.g = pb.g; t.C = pb.C; t.ncv = ncv; t.cl = cl; t.tl = 16;
            t.ntiles = (pb.M + TK - 1) / TK;
            int nb = cached_occupancy(reinterpret_cast<const void*>(kernel), 256, smem);
            const int cap = tuning().rbps > 0 ? tuning().rbps : 2;
            if (nb > cap) nb = cap;
            if (nb < 1) nb = 1;
            uint32_t gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(nb) / gy;
            const uint32_t bound = partial_blocks_bound(pb.M);
            if (gx > bound) gx = bound;
            if (gx < 1) gx = 1;
            if (gx > t.ntiles) gx = t.ntiles;
            if (blocks) *blocks = gx;
            kernel<<<dim3(gx, gy, 1), 256, smem, pb.stream>>>(p);
            count_launch();
            return cudaGetLastError();
        };
        static_assert(kMaxEvents <= 24, "the widest instantiation covers 4 x 6 events");
        if (pb.E <= 4) return go(std::integral_constant<int, 1>{});
        if (pb.E <= 8) return go(std::integral_constant<int, 2>{});
        if (pb.E <= 12) return go(std::integral_constant<int, 3>{});
        if (pb.E <= 16) return go(std::integral_constant<int, 4>{});
        if (pb.E <= 20) return go(std::integral_constant<int, 5>{});
        return go(std::integral_constant<int, 6>{});
    });
}

}  // namespace sihc
