// Internal host-side interface between the C ABI (sihc_capi.cu) and the kernel
// translation units.  Not part of the public ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sihc_common.cuh"

namespace sihc {

enum DType { kF32 = 0, kBF16 = 1 };

// Tunable launch parameters (defaults chosen from measurements on B200).
struct Tuning {
    int threads = 0;        // target threads per block (0: per-kernel default)
    int tt = 0;             // tokens per thread per tile (0: per-kernel default)
    int bps = 0;            // blocks per SM cap for streaming kernels (0: occupancy)
    int rbps = 0;           // blocks per SM for kernels that emit partial sums (0: default 2)
    int maxvec_bytes = 0;   // cap on the vector width in bytes (0: 16)
    int ring = -1;          // stages of the async-copy ring in the fused single-event adjoints (-1: default, 0: off)
    int min_block_tokens = 0;   // fewest tokens a partial-sum block should own (0: default)
    int stage_budget_kb = 0;    // shared-memory budget of the staged-coefficient kernels in KB (0: default 35)
    int tri_chunk = 0;          // events per z-slice of the triangular backward (0: default)
    int wgrad_tiled = -1;       // stage weight gradient: 1 block-tiled kernel, 0 per-thread kernel (-1: default)
    int token_lanes = 0;        // fused literal adjoint: fewest token lanes per block (0: default 4 or 6)
    int one_pass_adjoints = -1; // stage read/write backward: 0 two kernels, otherwise one pass where it applies
    int one_pass_min_events = 0; // fewest events for the one-pass forms; <= 0: 8 (write backward) and 12 (read backward)
    int half_vectors = -1;      // fused literal adjoint: 1 half-width vectors and twice the threads, 0 full width, -1 default
    int stage_smem = -1;        // stage read/write coefficients: 1 staged in shared memory, 0 re-read from L1,
                                // -1 default (staged whenever the vector path applies)
};
Tuning& tuning();
int sm_count();
void count_launch(int n = 1);

// Problem description after validation.
struct Problem {
    DType dtype, wdtype;
    int E;              // events (or active prefix for triangular)
    int S;              // slots (0 for triangular)
    uint32_t M, g, C;
    int V;              // channels per thread chosen by the C ABI from size/alignment
    cudaStream_t stream;
};

// Upper bound on the number of partial-sum blocks a reduction kernel will use.
uint32_t partial_blocks_bound(uint32_t M);

cudaError_t launch_read_fwd(const Problem& pb, const void* x, const void* alpha, void* const* out);
cudaError_t launch_write_fwd(const Problem& pb, const void* x, const void* const* dz, const void* beta, void* y);
// Literal inference step: y = x + beta*dz (rounded), z_next = read(y, alpha_next); y may alias x.
cudaError_t launch_write_read(const Problem& pb, const void* x, const void* dz, const void* beta, const void* alpha_next,
                              void* y, void* z_next);
// Fused single-event adjoints; `partial` receives [P][S][C] fp32 rows, *blocks = P.
cudaError_t launch_read_bwd1(const Problem& pb, const void* x, const void* g, const void* alpha, void* dx,
                             float* partial, uint32_t* blocks);
cudaError_t launch_write_bwd1(const Problem& pb, const void* h, const void* dz, const void* beta, void* ddz,
                              float* partial, uint32_t* blocks);
// Same contracts, loads staged through a per-thread cp.async ring in shared memory (vector path only).
cudaError_t launch_read_bwd1_ring(const Problem& pb, const void* x, const void* g, const void* alpha, void* dx,
                                  float* partial, uint32_t* blocks, int stages, int threads);
cudaError_t launch_write_bwd1_ring(const Problem& pb, const void* h, const void* dz, const void* beta, void* ddz,
                                   float* partial, uint32_t* blocks, int stages, int threads);
struct ReadFwdParams { const void* x; const void* w; MutPtrs out; int E; Tiling t; };
struct WriteFwdParams { const void* x; ConstPtrs dz; const void* w; void* y; int E; Tiling t; };
// Stage (multi-event) read / write with the block's coefficient slice staged once in shared memory.
cudaError_t launch_read_fwd_stage(const Problem& pb, ReadFwdParams& p);
cudaError_t launch_write_fwd_stage(const Problem& pb, WriteFwdParams& p);
struct WriteReadParams { const void* x; const void* dz; const void* beta; const void* alpha; void* y; void* z; Tiling t; };
struct ReadBwd1Params { const void* x; const void* g; const void* w; void* dx; float* partial; Tiling t; };
struct WriteBwd1Params { const void* h; const void* dz; const void* w; void* ddz; float* partial; Tiling t; };
// Multi-event weight gradient partials: [P][E][S][C].
struct WGradParams { const void* x; ConstPtrs z; float* partial; int E; Tiling t; };
// The tiled weight gradient with the write's other adjoint in the same pass: ddz[l][m,c] = sum_s w[l,c,s] * x[m,s,c].
struct WGradReadParams { const void* x; ConstPtrs z; float* partial; int E; Tiling t; const void* w; MutPtrs out; };
// Events handled per pass over the carrier by the stage weight-gradient kernel.
template <int S, int V> struct EventChunk {
    static constexpr int raw = 64 / (S * V);
    static constexpr int value = raw < 1 ? 1 : (raw > 8 ? 8 : raw);
};
// The same partials from a block-tiled kernel: the carrier tile is staged once per block in shared memory and shared by
// the threads that own different events (sihc_wgrad.cu).  Vector path only.
cudaError_t launch_wgrad_tiled(const Problem& pb, const void* carrier, const void* const* z, float* partial,
                               uint32_t* blocks);
// Whether the one-pass form below serves this problem (vector path, 4 slots, >= 16 events, weights in the tensor dtype).
bool wgrad_tiled_read_applies(const Problem& pb);
// One pass over the carrier gradient for BOTH adjoints of the stage write: the dbeta partials of launch_wgrad_tiled and
// ddz[l] = sum_s beta[l,c,s] * h[m,s,c] (null ddz[l] skipped): S + 2E elements instead of 2(S + E).
cudaError_t launch_wgrad_tiled_read(const Problem& pb, const void* carrier, const void* const* z, const void* beta,
                                    void* const* ddz, float* partial, uint32_t* blocks);
cudaError_t launch_wgrad(const Problem& pb, const void* carrier, const void* const* z, float* partial,
                         uint32_t* blocks);
// out[(row / S) * C * S + c * S + row % S] = sum_p partial[(p * rows + row) * C + c]
cudaError_t launch_finish(const float* partial, float* out, uint32_t blocks, uint32_t rows, uint32_t C,
                          uint32_t S, cudaStream_t stream);
cudaError_t launch_tri_fwd(const Problem& pb, const void* base, const void* const* dz, const void* gamma, void* out);
// Partials [P][J][C]; ddz may be null.
cudaError_t launch_tri_bwd(const Problem& pb, const void* grad, const void* const* dz, const void* gamma,
                           void* const* ddz, float* partial, uint32_t* blocks);

// Fused backward of the literal step (sihc_literal.cu); `partial` receives [P][2S][C] rows (dalpha_next, then dbeta).
cudaError_t launch_write_read_bwd(const Problem& pb, const void* h, const void* gz, const void* y, const void* dz,
                                  const void* beta, const void* alpha_next, void* hh, void* ddz, float* partial,
                                  uint32_t* blocks);

// One pass over the carrier and the E gradients for BOTH adjoints of the stage read (4 slots, 12..24 events, weights in
// the tensor dtype): dx = sum_l alpha_l * g_l and the dalpha partials: 2S + E elements instead of 2(S + E).
bool read_bwd_tiled_applies(const Problem& pb);
cudaError_t launch_read_bwd_tiled(const Problem& pb, const void* carrier, const void* const* g, const void* alpha, void* dx,
                                  float* partial, uint32_t* blocks);

// Whole-stage coefficient gradient dgamma[i][j][c] = sum_m g_i * dz_j (j < i; zero elsewhere), [E][E][C] fp32, from one
// pass over the E-1 recorded gradients and E-1 updates (sihc_trigamma.cu).  Needs C * element size % 16 == 0 and
// 16-byte aligned tensors.  g[0] and dz[E-1] are not read; a null g[i] gives a zero row.
size_t tri_dgamma_workspace_bytes(int E, uint32_t M, uint32_t C, size_t esize);
cudaError_t launch_tri_dgamma(const Problem& pb, const void* const* g, const void* const* dz, float* partial,
                              float* dgamma);

// Measurement aid: write `bytes` of zeros with the same 16-byte streaming stores the kernels use (sihc_reduce.cu).
cudaError_t launch_store_stream(void* dst, size_t bytes, cudaStream_t stream);

// ---- shared launch plumbing -------------------------------------------------------------------
struct BlockShape { uint32_t cl, tl, gy, threads; };

inline BlockShape block_shape(uint32_t ncv, int target_threads, int max_threads = kMaxThreads) {
    BlockShape b;
    const uint32_t target = static_cast<uint32_t>(target_threads);
    const uint32_t limit = static_cast<uint32_t>(max_threads);      // the kernel's __launch_bounds__
    if (ncv <= limit) { b.cl = ncv; b.gy = 1; }
    else { b.cl = 256; b.gy = (ncv + 255) / 256; }
    uint32_t tl = (target + b.cl / 2) / b.cl;
    if (tl < 1) tl = 1;
    while (tl > 1 && tl * b.cl > limit) --tl;
    b.tl = tl;
    b.threads = b.cl * b.tl;
    return b;
}

// Resident blocks per SM of `kernel` at this block size / dynamic shared memory (cached per device,
// kernel address, block size and shared-memory size; defined in sihc_capi.cu).
int cached_occupancy(const void* kernel, int threads, size_t dynamic_smem);
// Raise the kernel's dynamic shared-memory limit once per device.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);

template <typename K>
inline int occupancy_blocks(K kernel, int threads) {
    return cached_occupancy(reinterpret_cast<const void*>(kernel), threads, 0);
}

}  // namespace sihc
