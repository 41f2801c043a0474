/*
 * sihc_b200 — C ABI of the B200 (sm_100a) SiHC hyper-connection routing library.
 *
 * This is the drop-in boundary for the reference's fused routing operators.
 * Every entry point is plain C: raw device pointers, sizes, a CUDA stream passed
 * as `void*` (a `cudaStream_t`), and an `int` status.  The library allocates no
 * memory, keeps no per-call state, never synchronises the device and launches
 * only on the stream it is given, so it may be called from the autograd worker
 * thread, from compiled graphs and under stream capture.
 *
 * Geometry shared by all carrier operators (reference: `_high_offsets`,
 * sihc/models/sihc/sublayer_kernels.py:21-25 and `_geometry`, :180-193):
 *   carrier  X  : NHWC, packed, [batch, grid*kh, grid*kw, channels]
 *   workspace z : packed, [batch, grid*grid, channels]
 *   weights     : packed, [events, channels, slots], slots = kh*kw
 *   token m = (b, wy, wx) owns carrier pixels (wy*kh+uy, wx*kw+ux); slot s = uy*kw+ux.
 * Supported cells: (kh,kw) in {(1,2),(2,2),(2,4),(4,4)}  -> slots in {2,4,8,16}.
 * The reference supports (2,2) and (4,4) only; the others are this library's extension.
 *
 * dtype codes: SIHC_F32 = 0, SIHC_BF16 = 1.  `dtype` is the storage type of the
 * carrier and workspace tensors; `wdtype` is the storage type of the weight
 * tensor (alpha / beta / gamma) and must be `dtype` or SIHC_F32.  All arithmetic
 * accumulates in fp32 and rounds once when storing.
 *
 * Pointer arrays (`const void* const*`) are HOST arrays of `events` device
 * pointers; they are copied by value into the kernel parameters (the analogue
 * of the reference's tuple-of-pointers kernels).
 *
 * Status: 0 success; negative = invalid argument (see sihc_status_string);
 * positive = a cudaError_t reported by the launch.
 */
#ifndef SIHC_B200_H_
#define SIHC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SIHC_F32 0
#define SIHC_BF16 1
#define SIHC_MAX_EVENTS 24

#define SIHC_OK 0
#define SIHC_ERR_NULL (-1)        /* a required pointer is null */
#define SIHC_ERR_DTYPE (-2)       /* unsupported dtype / wdtype combination */
#define SIHC_ERR_EVENTS (-3)      /* events outside 1..SIHC_MAX_EVENTS */
#define SIHC_ERR_CELL (-4)        /* (kh,kw) not a supported cell */
#define SIHC_ERR_SHAPE (-5)       /* non-positive or overflowing batch/grid/channels */
#define SIHC_ERR_WORKSPACE (-6)   /* workspace missing, misaligned or too small */
#define SIHC_ERR_ALIGN (-7)       /* a tensor pointer is not aligned to its element size */
#define SIHC_ERR_CAPACITY (-8)    /* size beyond a built-in fixed capacity */

/* Library ABI version (bumped on any signature change). */
int sihc_version(void);

/* Human-readable text for a status returned by any entry point. */
const char* sihc_status_string(int status);

/*
 * Stage read, forward.  out[l][m,c] = sum_s alpha[l,c,s] * X[m,s,c]  for l < events.
 * Replaces `sublayer_read` + `_read` / `_read_bf16_mma`
 * (sihc/models/sihc/sublayer_kernels.py:219-232, :28-79) and, with events == 1,
 * `read_torch` (sihc/bench/fusion_controls.py:14-20).
 */
int sihc_read_fwd(const void* x, const void* alpha, void* const* out, int events,
                  int64_t batch, int grid, int kh, int kw, int channels,
                  int dtype, int wdtype, void* stream);

/*
 * Stage write, forward.  y[m,s,c] = (x ? x[m,s,c] : 0) + sum_l beta[l,c,s] * dz[l][m,c].
 * Replaces `sublayer_write` / `_write_impl` + `_write` / `_write_bf16_mma`
 * (sihc/models/sihc/sublayer_kernels.py:246-258, :290-292, :82-127); `x == NULL`
 * is the reference's `add_x=False` (the read's carrier gradient, :284); events == 1
 * is `write_torch` (sihc/bench/fusion_controls.py:23-31).  `y` must not alias `x`.
 */
int sihc_write_fwd(const void* x, const void* const* dz, const void* beta, void* y, int events,
                   int64_t batch, int grid, int kh, int kw, int channels,
                   int dtype, int wdtype, void* stream);

/*
 * Literal (unfused-schedule) step for inference: write one event into the carrier and read the next
 * event from the result, in one pass over the carrier.
 *   y[m,s,c]      = x[m,s,c] + beta[c,s] * dz[m,c]        (rounded to `dtype`)
 *   z_next[m,c]   = sum_s alpha_next[c,s] * y[m,s,c]      (computed from the rounded y)
 * `beta` and `alpha_next` are [channels, slots].  Replaces the pair
 * `carrier = write_torch(carrier, [dz], [beta]); z = read_torch(carrier, alpha_next)` of the reference's
 * literal schedule (sihc/bench/fusion_controls.py:64, :80; research/tests/test_sublayer_kernels.py:216-226)
 * and gives the same values, moving 2*slots+2 elements per token and channel instead of 3*slots+2.
 * `y` may be `x` (in-place carrier update: the carrier is then read with coherent loads, every element by the
 * thread that rewrites it); any other overlap of `y` with an input is not allowed.  Forward only.
 */
int sihc_write_read_fwd(const void* x, const void* dz, const void* beta, const void* alpha_next,
                        void* y, void* z_next, int64_t batch, int grid, int kh, int kw, int channels,
                        int dtype, int wdtype, void* stream);

/* Scratch bytes for sihc_write_read_bwd. */
size_t sihc_write_read_bwd_workspace_bytes(int64_t batch, int grid, int kh, int kw, int channels, int dtype);

/*
 * Backward of sihc_write_read_fwd, fused: with h = dL/dy and gz = dL/dz_next,
 *   hh[m,s,c]          = h[m,s,c] + alpha_next[c,s] * gz[m,c]       (gradient w.r.t. x; rounded to `dtype`)
 *   ddz[m,c]           = sum_s beta[c,s] * hh[m,s,c]                 (from the unrounded hh)
 *   dweights[0][c,s]   = sum_m y[m,s,c] * gz[m,c]                    (dalpha_next, fp32)
 *   dweights[1][c,s]   = sum_m dz[m,c] * hh[m,s,c]                   (dbeta, fp32)
 * in one pass: 3*slots+3 elements per token and channel.  `y` is the carrier the forward call produced.  It is what
 * differentiating the reference's literal schedule step `write_torch` -> `read_torch`
 * (sihc/bench/fusion_controls.py:14-31, :64, :80) yields, which the reference leaves to autograd over separate
 * operators.  `h` NULL = no gradient reaches y from later events (zero); `gz` NULL = the next read was unused
 * (hh = h, dalpha_next = 0; `y` is then not read); `hh`, `ddz`, `dweights` may each be NULL to skip that output;
 * `hh` may be `h` (in place).  `dweights` is [2, channels, slots] fp32.  Deterministic reduction as in sihc_read_bwd.
 */
int sihc_write_read_bwd(const void* h, const void* gz, const void* y, const void* dz, const void* beta,
                        const void* alpha_next, void* hh, void* ddz, float* dweights, void* workspace,
                        size_t workspace_bytes, int64_t batch, int grid, int kh, int kw, int channels,
                        int dtype, int wdtype, void* stream);

/*
 * Bytes of scratch the two backward entry points below need for `events` events
 * on this geometry (per-block partial sums of the weight gradients).  The
 * scratch needs no initialisation and holds nothing between calls.
 * The size depends on the launch parameters in force ("partial_blocks_per_sm" and
 * "min_block_tokens" of sihc_tune): size the scratch and make the call under the same
 * settings, or the call returns SIHC_ERR_WORKSPACE.  The same holds for
 * sihc_tri_workspace_bytes.
 */
size_t sihc_wgrad_workspace_bytes(int events, int64_t batch, int grid, int kh, int kw,
                                  int channels, int dtype);

/*
 * Stage read, backward (both adjoints in one call).
 *   dx[m,s,c]       = sum_l alpha[l,c,s] * g[l][m,c]
 *   dalpha[l,c,s]   = sum_m X[m,s,c] * g[l][m,c]          (fp32, [events,channels,slots])
 * Replaces `_read_backward` (sihc/models/sihc/sublayer_kernels.py:280-284), i.e.
 * `_write_impl(..., add_x=False)` plus `_weights_backward` (:261-273) with its
 * `_weight_grad*` kernels (:130-177).  A NULL entry g[l] is an unused read output:
 * it adds nothing to dx and leaves dalpha[l] exactly zero (the reference
 * materialises zeros, :283).  `dx` or `dalpha` may be NULL to skip that output.
 * The reduction over tokens is deterministic (no atomics): fixed per-block
 * partials in `workspace`, then a fixed-order finishing pass.
 * With 4 slots, 12 or more events, weights in the tensor dtype and both outputs wanted,
 * one kernel produces dx and the dalpha partials from a single pass over x and the
 * gradients (2*slots + events elements per token and channel; the two-kernel form, and
 * the reference, read the gradients twice).  dx is then summed per quarter of the events
 * and combined in a fixed order: deterministic, equal to the two-kernel form to fp32
 * rounding of the sum.
 */
int sihc_read_bwd(const void* x, const void* const* g, const void* alpha, void* dx, float* dalpha,
                  void* workspace, size_t workspace_bytes, int events,
                  int64_t batch, int grid, int kh, int kw, int channels,
                  int dtype, int wdtype, void* stream);

/*
 * sihc_read_bwd for callers that cannot allocate device memory.  No counterpart in
 * the reference (its operators allocate their scratch with torch.zeros).
 *
 * Same inputs, outputs and results as sihc_read_bwd, but without the workspace
 * arguments: the partial sums go to a fixed SIHC_STATIC_SCRATCH_BYTES array built
 * into the library (held by every GPU that loads the library until the process
 * exits).  Meant for hosts whose device memory is fully planned at start-up (fixed
 * arenas, frozen memory maps) and for threads that must never trigger the implicit
 * device synchronisation of cudaMalloc / cudaFree.  It calls no allocating routine.
 *   - Returns SIHC_ERR_CAPACITY, before launching anything, when
 *     sihc_wgrad_workspace_bytes(...) for the case exceeds SIHC_STATIC_SCRATCH_BYTES
 *     (single event, 4 slots, 768 channels needs 3.6 MB; the limit is 16 MiB).
 *   - The first call on each device does a one-time set-up: it looks up the array's
 *     device address (cudaGetSymbolAddress, with that device current).  Make that first
 *     call before any stream capture is started on the device.  The sentence at the top
 *     of this header about compiled graphs and stream capture is not extended to this
 *     entry point.
 *   - One array per device is shared by all calls: calls that can overlap on the GPU
 *     race and must be serialised by the caller.  The array keeps the previous call's
 *     partial sums; they are never read (every row is rewritten before use).
 */
#define SIHC_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int sihc_read_bwd_static(const void* x, const void* const* g, const void* alpha, void* dx, float* dalpha,
                         int events, int64_t batch, int grid, int kh, int kw, int channels,
                         int dtype, int wdtype, void* stream);

/*
 * Stage write, backward w.r.t. the updates and beta (the carrier gradient of the
 * write is `h` itself and needs no kernel).
 *   ddz[l][m,c]     = sum_s beta[l,c,s] * h[m,s,c]
 *   dbeta[l,c,s]    = sum_m dz[l][m,c] * h[m,s,c]         (fp32, [events,channels,slots])
 * Replaces `_write_backward` (sihc/models/sihc/sublayer_kernels.py:300-303), i.e.
 * `sublayer_read(grad, beta)` plus `_weights_backward(grad, updates, beta)`.
 * `ddz` (the array) or `dbeta` may be NULL to skip that output.
 * With 4 slots, 8 or more events, weights in the tensor dtype and both outputs wanted,
 * one kernel produces ddz and the dbeta partials from a single pass over h and the updates
 * (slots + 2*events elements per token and channel); ddz is bit-identical to the two-kernel
 * form, and so is dbeta from 16 events up (below, the two-kernel form sums in another order).
 */
int sihc_write_bwd(const void* h, const void* const* dz, const void* beta, void* const* ddz,
                   float* dbeta, void* workspace, size_t workspace_bytes, int events,
                   int64_t batch, int grid, int kh, int kw, int channels,
                   int dtype, int wdtype, void* stream);

/*
 * Triangular accumulation, forward.  out = base + sum_{l<active} gamma[l,c] * dz[l].
 * `tokens` = batch*grid*grid rows of `channels`; gamma is [active, channels] in `gdtype`.
 * Replaces `sublayer_triangular` + `_triangular`
 * (sihc/models/sihc/sublayer_kernels.py:337-352, :309-321) and `triangular_torch`
 * (sihc/bench/fusion_controls.py:34-38).  active in 1..SIHC_MAX_EVENTS.
 */
int sihc_tri_fwd(const void* base, const void* const* dz, const void* gamma, void* out, int active,
                 int64_t tokens, int channels, int dtype, int gdtype, void* stream);

/* Scratch bytes for sihc_tri_bwd's deterministic dgamma reduction. */
size_t sihc_tri_workspace_bytes(int active, int64_t tokens, int channels, int dtype);

/*
 * Triangular accumulation, backward.
 *   ddz[l]       = grad * gamma[l]        (fp32 product, one rounding)   if ddz != NULL
 *   dgamma[l,c]  = sum_m grad[m,c] * dz[l][m,c]   (fp32, [active,channels]) if dgamma != NULL
 * Replaces `_tri_autograd` / `_tri_gamma_backward` + `_triangular_gamma_grad`
 * (sihc/models/sihc/sublayer_kernels.py:369-379, :355-361, :324-334).
 */
int sihc_tri_bwd(const void* grad, const void* const* dz, const void* gamma, void* const* ddz,
                 float* dgamma, void* workspace, size_t workspace_bytes, int active,
                 int64_t tokens, int channels, int dtype, int gdtype, void* stream);

/* Scratch bytes for sihc_tri_dgamma. */
size_t sihc_tri_dgamma_workspace_bytes(int events, int64_t tokens, int channels, int dtype);

/*
 * Gradient of a whole stage's triangular coefficients in one pass.
 *   dgamma[i,j,c] = sum_m g[i][m,c] * dz[j][m,c]   for j < i < events;  0 elsewhere   (fp32, [events,events,channels])
 * g[i] is the gradient that reached event i's accumulated read (g[0] is not read; a NULL g[i] is a read that was
 * never used and gives a zero row), dz[j] is event j's update (dz[events-1] is not read).  Every tensor is read once:
 * 2(events-1) workspace tensors instead of the events^2/2 of one `_tri_gamma_backward` + `_triangular_gamma_grad`
 * call per event (sihc/models/sihc/sublayer_kernels.py:355-361, :324-334), which this replaces for a stage whose
 * backward is scheduled as a whole.  Deterministic (per-block partial sums in `workspace`, fixed-order finish).
 */
int sihc_tri_dgamma(const void* const* g, const void* const* dz, float* dgamma, void* workspace,
                    size_t workspace_bytes, int events, int64_t tokens, int channels, int dtype, void* stream);

/*
 * Benchmark-only knob: override a launch parameter by name; never needed for
 * correct results.  Process-global and not thread-safe.  "partial_blocks_per_sm" and
 * "min_block_tokens" change what sihc_*_workspace_bytes return: do not change them
 * between sizing a workspace and the call that uses it.
 *   "threads", "tokens_per_thread", "blocks_per_sm", "partial_blocks_per_sm",
 *   "max_vector_bytes", "min_block_tokens", "stage_budget_kb" (KB of shared memory
 *   for a block's coefficient slice), "tri_chunk" (events per grid slice of the
 *   triangular backward, 1..8), "token_lanes" (fewest token lanes per block of the fused literal
 *   adjoint): value <= 0 restores the default.
 *   "ring_stages" (0 = register-staged single-event adjoints, 3..8 = async-copy ring),
 *   "stage_smem" (0 = stage coefficients from L1, 1 = from shared memory),
 *   "wgrad_tiled" (0 = per-thread, 1 = block-tiled stage weight gradient),
 *   "one_pass_adjoints" (0 = stage read/write backward always as two kernels),
 *   "one_pass_min_events" (fewest events for which they run as one pass; <= 0 restores the defaults,
 *   8 for the write backward and 12 for the read backward),
 *   "half_vectors" (fused literal adjoint: 1 = half-width vectors and twice the channel lanes): a negative
 *   value restores the per-kernel default ("ring_default" / "stage_smem_default"
 *   with any value do the same).
 * Returns 0, or SIHC_ERR_NULL for an unknown name.  (Counterpart of the
 * reference's `SIHC_*` environment tile overrides, sihc/models/sihc/kernels.py:19-23.)
 */
int sihc_tune(const char* name, int value);

/*
 * Measurement aid, no counterpart in the reference: fill `bytes` (a multiple of 16, `dst` 16-byte aligned) with zeros
 * using the 16-byte streaming stores of the routing kernels and nothing else.  Its bandwidth is the device's
 * write-only rate, the bound for operators whose traffic is mostly output (a 24-event stage read writes 24 of its
 * 28 elements per token and channel).
 */
int sihc_probe_store_stream(void* dst, size_t bytes, void* stream);

/* Number of kernel launches this library has issued in this process (for benches). */
uint64_t sihc_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SIHC_B200_H_ */
