// Gradient of the whole triangular coefficient matrix of a stage in ONE pass:
//     dgamma[i, j, c] = sum_m g_i[m, c] * dz_j[m, c]        for j < i < E
// where g_i is the gradient that reached event i's accumulated read and dz_j is event j's update.
//
// The per-event form (`tri_bwd_kernel`, and the reference's `_triangular_gamma_grad`,
// sihc/models/sihc/sublayer_kernels.py:324-334, launched once per event by `_tri_gamma_backward`, :355-361)
// re-reads the prefix dz_0..dz_{i-1} for every i: about E*E/2 workspace tensors per stage.  Here every g_i and
// dz_j is read exactly once (2(E-1) tensors) and all E(E-1)/2 products are formed from a token tile held in
// shared memory.
//
// Work split: rows r = i-1 and columns j of the lower triangle (j <= r) are cut into 4 x 4 blocks; a thread
// owns one block for V = 4 adjacent channels: 16 products per token from 8 shared-memory vectors, 64 fp32
// accumulators.  A thread block is (lower-triangle 4x4 blocks) x (CL channel lanes); the tile of TK tokens of
// all 2(E-1) tensors for the block's CL*V channels is copied once per block by `cp.async` (16-byte pieces, NST
// stages) and read by every 4x4 block.  A (4x4 block, lane) pair is unique in the thread block, so a thread's
// accumulators ARE the block's partial sums: no reduction inside the block, one fp32 row set per thread block
// in scratch, and a fixed-order finishing pass over the thread blocks (deterministic, no atomics).  Diagonal
// 4x4 blocks compute 16 products and keep the 10 with j <= r.
#include "sihc_dispatch.cuh"
#include "sihc_ring.cuh"

namespace sihc {

constexpr int kTriGammaBlock = 4;            // rows and columns of a thread's block of the coefficient matrix
constexpr int kTriGammaV = 4;                // channels per thread
constexpr int kTriGammaMaxThreads = 384;

struct TriGammaParams {
    ConstPtrs g;        // g[i], i in 1..E-1 (entry 0 unused); null = that read was not used: zero row
    ConstPtrs dz;       // dz[j], j in 0..E-2
    float* partial;     // [gridDim.x][n(n+1)/2][C], n = E-1, pair (r, j) at r(r+1)/2 + j
    int E;
    Tiling t;           // t.cl = channel lanes, t.tl = number of 4x4 blocks, t.ntiles = token tiles of TK
};

template <typename T, int TK, int NST>
__global__ void __launch_bounds__(kTriGammaMaxThreads) tri_dgamma_kernel(const __grid_constant__ TriGammaParams p) {
    constexpr int V = kTriGammaV, B = kTriGammaBlock;
    typedef VecIO<T, V> IO;
    typedef typename IO::Raw Raw;
    extern __shared__ __align__(16) unsigned char tile_bytes[];
    const Tiling& t = p.t;
    const int n = p.E - 1;                       // rows r = i-1 in [0,n), columns j in [0,n)
    const int nb = (n + B - 1) / B;              // 4x4 blocks per side
    const int rows = 2 * nb * B;                 // tile rows: nb*B (padded) g rows, then nb*B dz rows
    const uint32_t CL = t.cl, tid = threadIdx.x, nthreads = blockDim.x;
    const uint32_t lane = tid % CL, blk = tid / CL;
    // block index -> (br, bc) with bc <= br, numbered row by row
    int br = 0;
    while ((br + 1) * (br + 2) / 2 <= static_cast<int>(blk)) ++br;
    const int bc = static_cast<int>(blk) - br * (br + 1) / 2;
    const uint32_t cv = blockIdx.y * CL + lane;
    const bool active = cv < t.ncv && blk < t.tl;
    const uint32_t row_vecs = CL;                                    // Raw vectors per tile row
    const uint32_t row_bytes = CL * V * sizeof(T);
    const uint32_t chunks_per_row = row_bytes / 16;
    const size_t block_c0 = static_cast<size_t>(blockIdx.y) * CL * V;  // first channel of the block's slice
    const uint32_t chan_bytes_left = t.C > block_c0 ? static_cast<uint32_t>((t.C - block_c0) * sizeof(T)) : 0u;

    // Copy plan.  A tile is TK tokens x `rows` rows of `chunks_per_row` 16-byte pieces.  Which (row, piece) pairs
    // a thread copies is the same for every token and every tile, so the pair's shared-memory offset and global
    // row pointer are worked out once (KD pairs in registers; shapes with more pairs per thread - few threads,
    // wide rows - fall back to computing them per copy).  Rows that are padding or belong to an unused read have
    // no source: the whole ring is zeroed once and those rows are never written again.
    constexpr int KD = 4;
    const uint32_t per_token = static_cast<uint32_t>(rows) * chunks_per_row;
    auto source_of = [&](uint32_t row) -> const unsigned char* {
        const int k = static_cast<int>(row) < nb * B ? static_cast<int>(row) : static_cast<int>(row) - nb * B;
        if (k >= n) return nullptr;
        return static_cast<const unsigned char*>(static_cast<int>(row) < nb * B ? p.g.p[k + 1] : p.dz.p[k]);
    };
    uint32_t plan_dst[KD];
    const unsigned char* plan_src[KD];
#pragma unroll
    for (int k = 0; k < KD; ++k) {
        const uint32_t idx = tid + static_cast<uint32_t>(k) * nthreads;
        plan_dst[k] = 0; plan_src[k] = nullptr;
        if (idx < per_token) {
            const uint32_t ck = idx % chunks_per_row, row = idx / chunks_per_row;
            const unsigned char* base = source_of(row);
            if (base != nullptr && ck * 16 < chan_bytes_left) {
                plan_dst[k] = row * row_bytes + ck * 16;
                plan_src[k] = base + block_c0 * sizeof(T) + ck * 16;
            }
        }
    }
    for (uint32_t i = tid * 16; i < static_cast<uint32_t>(NST) * TK * rows * row_bytes; i += nthreads * 16)
        *reinterpret_cast<uint4*>(tile_bytes + i) = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const size_t token_stride = static_cast<size_t>(t.C) * sizeof(T);
    const uint32_t token_bytes = static_cast<uint32_t>(rows) * row_bytes;

    auto issue = [&](uint32_t tile, int stage) {
        const bool live = tile < t.ntiles;
        unsigned char* dst0 = tile_bytes + static_cast<size_t>(stage) * TK * token_bytes;
#pragma unroll
        for (int tok = 0; tok < TK; ++tok) {
            const uint32_t m = tile * TK + tok;
            const bool ok = live && m < t.M;            // past the end: zero-fill, so stale tokens never count twice
            const size_t goff = static_cast<size_t>(ok ? m : 0u) * token_stride;
#pragma unroll
            for (int k = 0; k < KD; ++k)
                if (plan_src[k] != nullptr) cp_async<16>(dst0 + tok * token_bytes + plan_dst[k], plan_src[k] + goff, ok);
            for (uint32_t idx = tid + KD * nthreads; idx < per_token; idx += nthreads) {       // rare wide shapes
                const uint32_t ck = idx % chunks_per_row, row = idx / chunks_per_row;
                const unsigned char* base = source_of(row);
                if (base != nullptr && ck * 16 < chan_bytes_left)
                    cp_async<16>(dst0 + tok * token_bytes + row * row_bytes + ck * 16,
                                 base + block_c0 * sizeof(T) + ck * 16 + goff, ok);
            }
        }
        cp_async_commit();
    };

    float acc[B * B][V];
#pragma unroll
    for (int a = 0; a < B * B; ++a)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[a][v] = 0.f;

    uint32_t tile = blockIdx.x;
#pragma unroll
    for (int st = 0; st < NST - 1; ++st) issue(tile + st * gridDim.x, st);
    int stage = 0;
    const uint32_t g_row0 = static_cast<uint32_t>(br * B), d_row0 = static_cast<uint32_t>(nb * B + bc * B);
    for (; tile < t.ntiles; tile += gridDim.x) {
        cp_async_wait<NST - 2>();
        __syncthreads();                   // everyone's copies for this tile have landed; previous tile fully consumed
        issue(tile + (NST - 1) * gridDim.x, stage == 0 ? NST - 1 : stage - 1);
        if (active) {
            const Raw* tb = reinterpret_cast<const Raw*>(tile_bytes + static_cast<size_t>(stage) * TK * rows * row_bytes) + lane;
#pragma unroll
            for (int tok = 0; tok < TK; ++tok) {
                const Raw* tr = tb + static_cast<size_t>(tok) * rows * row_vecs;
                Raw gv[B], dv[B];
#pragma unroll
                for (int a = 0; a < B; ++a) {
                    gv[a] = tr[(g_row0 + a) * row_vecs];
                    dv[a] = tr[(d_row0 + a) * row_vecs];
                }
#pragma unroll
                for (int a = 0; a < B; ++a)
#pragma unroll
                    for (int b = 0; b < B; ++b) IO::fma_raw(gv[a], dv[b], acc[a * B + b]);
            }
        }
        stage = stage + 1 == NST ? 0 : stage + 1;
    }
    cp_async_wait<0>();
    if (!active) return;
    const size_t pairs = static_cast<size_t>(n) * (n + 1) / 2;
    float* dst = p.partial + static_cast<size_t>(blockIdx.x) * pairs * t.C + static_cast<size_t>(cv) * V;
#pragma unroll
    for (int a = 0; a < B; ++a) {
        const int r = br * B + a;
        if (r >= n) continue;
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int j = bc * B + b;
            if (j > r) continue;                 // above the diagonal (or a padded column: j <= r < n)
            float* d = dst + (static_cast<size_t>(r) * (r + 1) / 2 + j) * t.C;
#pragma unroll
            for (int v = 0; v < V; ++v) d[v] = acc[a * B + b][v];
        }
    }
}

// dgamma[i][j][c] = j < i ? sum_{q < blocks} partial[q][(i-1) i / 2 + j][c] : 0   (fixed summation order)
__global__ void __launch_bounds__(256) tri_dgamma_finish_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                                uint32_t blocks, int E, uint32_t C) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;      // over E*E*C
    const size_t total = static_cast<size_t>(E) * E * C;
    if (idx >= total) return;
    const uint32_t c = static_cast<uint32_t>(idx % C);
    const int ij = static_cast<int>(idx / C), i = ij / E, j = ij % E;
    float sum = 0.f;
    if (j < i) {
        const size_t n = static_cast<size_t>(E) - 1;
        const size_t pairs = n * (n + 1) / 2;
        const size_t row = static_cast<size_t>(i - 1) * i / 2 + j;
        for (uint32_t q = 0; q < blocks; ++q) sum += partial[(static_cast<size_t>(q) * pairs + row) * C + c];
    }
    out[idx] = sum;
}

namespace {
constexpr int kTriGammaTokens = 4, kTriGammaStages = 3;
constexpr size_t kTriGammaMaxSmem = 200 * 1024;
struct TriGammaShape { uint32_t cl, gy, threads, nblk; size_t smem; };
inline TriGammaShape tri_gamma_shape(int E, uint32_t ncv, size_t esize) {
    const int n = E - 1, nb = (n + kTriGammaBlock - 1) / kTriGammaBlock;
    TriGammaShape s;
    s.nblk = static_cast<uint32_t>(nb * (nb + 1) / 2);
    const size_t per_lane = static_cast<size_t>(kTriGammaStages) * kTriGammaTokens * (2 * nb * kTriGammaBlock) *
                            kTriGammaV * esize;
    uint32_t cl = 64;               // a power of two >= 8: tile rows are whole 16-byte pieces (cl * V * esize % 16 == 0)
    while (cl > 8 && (cl * s.nblk > static_cast<uint32_t>(kTriGammaMaxThreads) || per_lane * cl > kTriGammaMaxSmem)) cl >>= 1;
    s.cl = cl;
    s.gy = (ncv + cl - 1) / cl;
    s.threads = cl * s.nblk;
    s.smem = per_lane * cl;
    return s;
}
// Thread blocks along the token axis: one wave of resident blocks (a 336-thread block of the 24-event case holds
// 64 accumulators per thread, so one block fits per SM; smaller stages fit two).  The count must not depend on the
// element type (the scratch is sized without it), so the resident-block estimate is the register budget only.
inline uint32_t tri_gamma_blocks(const TriGammaShape& s, uint32_t M) {
    int per_sm = s.threads * 144u <= 32768u ? 2 : 1;
    if (tuning().rbps > 0) per_sm = tuning().rbps;
    uint32_t gx = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(per_sm) / s.gy;
    const uint32_t ntiles = (M + kTriGammaTokens - 1) / kTriGammaTokens;
    if (gx < 1) gx = 1;
    if (gx > ntiles) gx = ntiles;
    return gx;
}
}  // namespace

// Vector path only: C % 4 == 0 and 16-byte aligned rows (checked by the caller).
size_t tri_dgamma_workspace_bytes(int E, uint32_t M, uint32_t C, size_t esize) {
    if (E < 2) return 0;
    const TriGammaShape s = tri_gamma_shape(E, C / kTriGammaV, esize);
    const size_t n = static_cast<size_t>(E) - 1;
    return static_cast<size_t>(tri_gamma_blocks(s, M)) * (n * (n + 1) / 2) * C * sizeof(float);
}

cudaError_t launch_tri_dgamma(const Problem& pb, const void* const* g, const void* const* dz, float* partial,
                              float* dgamma) {
    const int E = pb.E;
    cudaError_t err = cudaSuccess;
    uint32_t gx = 0;
    if (E >= 2) {
        TriGammaParams p{};
        for (int l = 0; l < E; ++l) { p.g.p[l] = g[l]; p.dz.p[l] = dz[l]; }
        p.partial = partial; p.E = E;
        const uint32_t ncv = pb.C / kTriGammaV;
        const TriGammaShape s = tri_gamma_shape(E, ncv, pb.dtype == kBF16 ? 2 : 4);
        gx = tri_gamma_blocks(s, pb.M);
        Tiling& t = p.t;
        t.M = pb.M; t.g = 1; t.C = pb.C; t.ncv = ncv; t.cl = s.cl; t.tl = s.nblk;
        t.ntiles = (pb.M + kTriGammaTokens - 1) / kTriGammaTokens;
        if (s.smem > kTriGammaMaxSmem || s.threads > static_cast<uint32_t>(kTriGammaMaxThreads)) return cudaErrorInvalidConfiguration;
        err = dispatch_types(pb.dtype, pb.dtype, [&](auto tt_, auto) {
            using T = decltype(tt_);
            auto kernel = tri_dgamma_kernel<T, kTriGammaTokens, kTriGammaStages>;
            size_t smem = s.smem;
            // Two stages of eight tokens instead of three of four (4/3 of the ring bytes) once a thread block holds
            // six or more 4x4 blocks of the matrix.  Measured on B200, bf16, GB/s of the 2(E-1) tensors read:
            // 24 events, 65 536 tokens x 768: 2058 -> 2391; 8192 x 1152: 2001 -> 2308; 16 events 2569 -> 2906;
            // 12 events 3660 -> 4086; but 8 events (three 4x4 blocks, 192 threads) 4345 -> 3083.
            // The `tokens_per_thread` knob forces a shape: 4 = (4 tokens, 3 stages), 8 = (8, 2), 12 = (8, 3), 16 = (16, 2).
            const int forced = tuning().tt;
            const bool wide = forced == 8 || (forced != kTriGammaTokens && forced != 12 && forced != 16 && s.nblk >= 6);
            auto use = [&](auto k, int tokens, int stages) {
                const size_t need = s.smem * static_cast<size_t>(tokens * stages) / (kTriGammaTokens * kTriGammaStages);
                if (need > kTriGammaMaxSmem) return false;
                kernel = k;
                t.ntiles = (pb.M + tokens - 1) / tokens;
                smem = need;
                if (gx > t.ntiles) gx = t.ntiles;
                return true;
            };
            if (forced == 12) use(tri_dgamma_kernel<T, 8, 3>, 8, 3);
            else if (forced == 16) use(tri_dgamma_kernel<T, 16, 2>, 16, 2);
            else if (wide) use(tri_dgamma_kernel<T, 2 * kTriGammaTokens, kTriGammaStages - 1>, 8, 2);
            if (cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kTriGammaMaxSmem)) return e;
            kernel<<<dim3(gx, s.gy, 1), s.threads, smem, pb.stream>>>(p);
            count_launch();
            return cudaGetLastError();
        });
        if (err != cudaSuccess) return err;
    }
    const size_t total = static_cast<size_t>(E) * E * pb.C;
    tri_dgamma_finish_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, pb.stream>>>(partial, dgamma, gx, E, pb.C);
    count_launch();
    return cudaGetLastError();
}

}  // namespace sihc
