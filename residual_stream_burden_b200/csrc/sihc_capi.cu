// C ABI of the SiHC routing library: argument validation, vector-width
// selection from sizes and pointer alignment, and the composition of kernels
// behind each entry point.  Declarations and the reference symbols each entry
// point replaces are in include/sihc_b200.h.
#include "sihc_b200.h"

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <tuple>

#include "sihc_dispatch.cuh"

namespace sihc {

Tuning& tuning() {
    static Tuning t;
    return t;
}

int sm_count() {
    static std::atomic<int> cached[64];     // zero-initialised; concurrent first calls all store the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

namespace {
std::mutex g_cache_mutex;
std::map<std::tuple<int, const void*, int, size_t>, int> g_occupancy;
std::set<std::pair<int, const void*>> g_smem_raised;
int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    return dev;
}
}  // namespace

int cached_occupancy(const void* kernel, int threads, size_t dynamic_smem) {
    const auto key = std::make_tuple(current_device(), kernel, threads, dynamic_smem);
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    auto it = g_occupancy.find(key);
    if (it != g_occupancy.end()) return it->second;
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, threads, dynamic_smem) != cudaSuccess || nb < 1) nb = 1;
    g_occupancy[key] = nb;
    return nb;
}

cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
    const auto key = std::make_pair(current_device(), kernel);
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    if (g_smem_raised.count(key)) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e == cudaSuccess) g_smem_raised.insert(key);
    return e;
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

uint32_t partial_blocks_bound(uint32_t M) {
    const int cap = tuning().rbps > 0 ? tuning().rbps : 2;
    uint32_t by_sm = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(cap);
    const uint32_t per = tuning().min_block_tokens > 0 ? static_cast<uint32_t>(tuning().min_block_tokens) : 32u;
    uint32_t by_tokens = (M + per - 1) / per;      // a block should own at least this many tokens
    if (by_tokens < 1) by_tokens = 1;
    return by_sm < by_tokens ? by_sm : by_tokens;
}

namespace {

// Async-copy ring defaults for the fused single-event adjoints, from a stages x threads sweep on B200
// (2^20 tokens, width 768 and 1152, bf16): three stages win everywhere they win at all; deeper rings lose
// DRAM locality.  read bwd: n=4 6447 vs 6416 GB/s (width 1152: 6436 vs 6215), n=8 6194 vs 5347, n=2 loses.
// write bwd: n=4 6710 vs 5879, n=8 6608 vs 5849, n=2 6789 (4 stages) vs 6714.
// Stage weight gradient.  The block-tiled kernel reads the carrier once instead of once per two events (through L2)
// and wins where the events are many; measured on B200, bf16, 4 slots, per-thread -> tiled GB/s: E=24 width 768
// 3906 -> 4487, E=16 width 1152 3774 -> 4480; but E=12 4329 -> 3568, E=8 4836 -> 4307, and 2 / 8 / 16 slots at E=12
// 5875 -> 2870, 2334 -> 2205, 1393 -> 1031.  With 192-thread blocks and the tile ring shaped per event count
// (sihc_wgrad.cu) the tiled form gives, at 65 536 tokens and width 768, E=24 5048 and E=16 4563 (per-thread 3877 /
// 4087); at 8192 tokens and width 1152, E=24 4137 and E=16 3641 (per-thread 3147 / 3271); E=12 stays a draw (4475 vs
// 4333, 3142 vs 3339).  8 slots at 24 events: 1906 -> 2488.  wgrad_tiled = 1 / 0 forces one form on the vector path.
inline cudaError_t stage_wgrad(const Problem& pb, const void* carrier, const void* const* z, float* partial, uint32_t* blocks) {
    const int forced = tuning().wgrad_tiled;
    const bool tiled = forced >= 0 ? forced != 0 : ((pb.S == 4 && pb.E >= 16) || (pb.S == 8 && pb.E >= 24));
    if (pb.V > 1 && tiled) return launch_wgrad_tiled(pb, carrier, z, partial, blocks);
    return launch_wgrad(pb, carrier, z, partial, blocks);
}
inline int read_bwd_ring_stages(int S) { const int t = tuning().ring; return t >= 0 ? t : (S >= 4 ? 3 : 0); }
inline int write_bwd_ring_stages(int S) { const int t = tuning().ring; return t >= 0 ? t : (S >= 4 ? 3 : 4); }
constexpr int kReadBwdRingThreads = 256, kWriteBwdRingThreads = 384;

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline size_t esize(int dtype) { return dtype == SIHC_BF16 ? 2 : 4; }

int check_types(int dtype, int wdtype) {
    if (dtype != SIHC_F32 && dtype != SIHC_BF16) return SIHC_ERR_DTYPE;
    if (wdtype != dtype && wdtype != SIHC_F32) return SIHC_ERR_DTYPE;
    return SIHC_OK;
}

int slots_of(int kh, int kw) {
    if (kh == 1 && kw == 2) return 2;
    if (kh == 2 && kw == 2) return 4;
    if (kh == 2 && kw == 4) return 8;
    if (kh == 4 && kw == 4) return 16;
    return 0;
}

// Validate the carrier geometry and fill everything of Problem but V.
int make_problem(Problem& pb, int events, int64_t batch, int grid, int kh, int kw, int channels, int dtype,
                 int wdtype, void* stream) {
    if (int st = check_types(dtype, wdtype)) return st;
    if (events < 1 || events > SIHC_MAX_EVENTS) return SIHC_ERR_EVENTS;
    const int S = slots_of(kh, kw);
    if (S == 0) return SIHC_ERR_CELL;
    if (batch < 1 || grid < 1 || channels < 1) return SIHC_ERR_SHAPE;
    const int64_t tokens = batch * grid * grid;
    if (grid > 65535 || tokens >= (int64_t(1) << 31) || channels > (1 << 24)) return SIHC_ERR_SHAPE;
    // the kernels keep a slot's offset inside its cell row block in 32 bits: (kh-1) carrier rows + one cell row
    const int64_t slot_span = (static_cast<int64_t>(kh - 1) * grid * kw + kw) * channels;
    if (slot_span >= (int64_t(1) << 32)) return SIHC_ERR_SHAPE;
    pb.dtype = static_cast<DType>(dtype);
    pb.wdtype = static_cast<DType>(wdtype);
    pb.E = events; pb.S = S;
    pb.M = static_cast<uint32_t>(tokens); pb.g = static_cast<uint32_t>(grid); pb.C = static_cast<uint32_t>(channels);
    pb.V = 1;
    pb.stream = static_cast<cudaStream_t>(stream);
    return SIHC_OK;
}

// Tracks the widest vector access every pointer of a call allows.
struct VecChoice {
    int full;           // candidate channels per thread
    size_t ebytes;
    bool ok = true;
    bool elem_ok = true;
    VecChoice(int full_, size_t ebytes_, uint32_t C) : full(full_), ebytes(ebytes_) {
        const int cap = tuning().maxvec_bytes;
        if (cap > 0 && static_cast<size_t>(full) * ebytes > static_cast<size_t>(cap)) ok = false;
        if (C % static_cast<uint32_t>(full) != 0) ok = false;
    }
    void act(const void* p) {            // activation tensor (may be null = absent)
        if (!p) return;
        if (!aligned(p, ebytes)) elem_ok = false;
        if (!aligned(p, static_cast<size_t>(full) * ebytes)) ok = false;
    }
    void weight(const void* p, size_t wbytes) {
        if (!p) return;
        if (!aligned(p, wbytes)) elem_ok = false;
        if (!aligned(p, 16)) ok = false;
    }
    int V() const { return ok ? full : 1; }
};

int status_of(cudaError_t e) { return e == cudaSuccess ? SIHC_OK : static_cast<int>(e); }

int check_workspace(const void* ws, size_t have, size_t need) {
    if (need == 0) return SIHC_OK;
    if (ws == nullptr || !aligned(ws, 16) || have < need) return SIHC_ERR_WORKSPACE;
    return SIHC_OK;
}

}  // namespace
}  // namespace sihc

using namespace sihc;

extern "C" {

int sihc_version(void) { return 2; }

const char* sihc_status_string(int status) {
    switch (status) {
        case SIHC_OK: return "ok";
        case SIHC_ERR_NULL: return "a required pointer is null";
        case SIHC_ERR_DTYPE: return "unsupported dtype (fp32/bf16 activations; weights in the activation dtype or fp32)";
        case SIHC_ERR_EVENTS: return "event count outside 1..24";
        case SIHC_ERR_CELL: return "unsupported slot grid (kh,kw); supported: (1,2) (2,2) (2,4) (4,4)";
        case SIHC_ERR_SHAPE: return "batch, grid and channels must be positive, tokens must fit 31 bits and one cell row block 32 bits";
        case SIHC_ERR_WORKSPACE: return "workspace missing, not 16-byte aligned, or smaller than sihc_*_workspace_bytes";
        case SIHC_ERR_ALIGN: return "a tensor pointer is not aligned to its element size";
        case SIHC_ERR_CAPACITY: return "size exceeds the fixed capacity of this entry point";
        default: break;
    }
    if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
    return "unknown status";
}

int sihc_tune(const char* name, int value) {
    if (!name) return SIHC_ERR_NULL;
    Tuning& t = tuning();
    const int tri = value < 0 ? -1 : value;      // three-state knobs: a negative value restores the per-kernel default
    if (value < 0) value = 0;
    if (!std::strcmp(name, "threads")) t.threads = value;
    else if (!std::strcmp(name, "tokens_per_thread")) t.tt = value;
    else if (!std::strcmp(name, "blocks_per_sm")) t.bps = value;
    else if (!std::strcmp(name, "partial_blocks_per_sm")) t.rbps = value;
    else if (!std::strcmp(name, "max_vector_bytes")) t.maxvec_bytes = value;
    else if (!std::strcmp(name, "ring_stages")) t.ring = tri;            // 0 = register-staged kernels
    else if (!std::strcmp(name, "ring_default")) t.ring = -1;            // back to the per-kernel default
    else if (!std::strcmp(name, "min_block_tokens")) t.min_block_tokens = value;
    else if (!std::strcmp(name, "stage_budget_kb")) t.stage_budget_kb = value;
    else if (!std::strcmp(name, "tri_chunk")) t.tri_chunk = value;
    else if (!std::strcmp(name, "wgrad_tiled")) t.wgrad_tiled = tri;    // 1 block-tiled, 0 per-thread weight gradient
    else if (!std::strcmp(name, "half_vectors")) t.half_vectors = tri;
    else if (!std::strcmp(name, "one_pass_adjoints")) t.one_pass_adjoints = tri;
    else if (!std::strcmp(name, "one_pass_min_events")) t.one_pass_min_events = value;
    else if (!std::strcmp(name, "token_lanes")) t.token_lanes = value;
    else if (!std::strcmp(name, "stage_smem")) t.stage_smem = tri;
    else if (!std::strcmp(name, "stage_smem_default")) t.stage_smem = -1;
    else return SIHC_ERR_NULL;
    return SIHC_OK;
}

uint64_t sihc_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int sihc_probe_store_stream(void* dst, size_t bytes, void* stream) {
    if (!dst) return SIHC_ERR_NULL;
    if (!aligned(dst, 16) || bytes % 16 != 0) return SIHC_ERR_ALIGN;
    if (bytes == 0) return SIHC_OK;
    return status_of(launch_store_stream(dst, bytes, static_cast<cudaStream_t>(stream)));
}

int sihc_read_fwd(const void* x, const void* alpha, void* const* out, int events, int64_t batch, int grid, int kh,
                  int kw, int channels, int dtype, int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, events, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!x || !alpha || !out) return SIHC_ERR_NULL;
    VecChoice vc(events == 1 ? vec_width_fwd(pb.dtype, pb.S) : vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(x); vc.weight(alpha, esize(wdtype));
    bool any = false;
    for (int l = 0; l < events; ++l) { vc.act(out[l]); any = any || out[l]; }
    if (!any) return SIHC_ERR_NULL;
    if (events == 1 && !out[0]) return SIHC_ERR_NULL;
    if (!vc.elem_ok) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    return status_of(launch_read_fwd(pb, x, alpha, out));
}

int sihc_write_fwd(const void* x, const void* const* dz, const void* beta, void* y, int events, int64_t batch,
                   int grid, int kh, int kw, int channels, int dtype, int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, events, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!dz || !beta || !y) return SIHC_ERR_NULL;
    VecChoice vc(events == 1 && dz[0] ? vec_width_fwd(pb.dtype, pb.S) : vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(x); vc.act(y); vc.weight(beta, esize(wdtype));
    for (int l = 0; l < events; ++l) vc.act(dz[l]);
    if (!vc.elem_ok) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    return status_of(launch_write_fwd(pb, x, dz, beta, y));
}

int sihc_write_read_fwd(const void* x, const void* dz, const void* beta, const void* alpha_next, void* y, void* z_next,
                        int64_t batch, int grid, int kh, int kw, int channels, int dtype, int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, 1, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!x || !dz || !beta || !alpha_next || !y || !z_next) return SIHC_ERR_NULL;
    VecChoice vc(vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(x); vc.act(dz); vc.act(y); vc.act(z_next);
    vc.weight(beta, esize(wdtype)); vc.weight(alpha_next, esize(wdtype));
    if (!vc.elem_ok) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    return status_of(launch_write_read(pb, x, dz, beta, alpha_next, y, z_next));
}

size_t sihc_write_read_bwd_workspace_bytes(int64_t batch, int grid, int kh, int kw, int channels, int dtype) {
    return 2 * sihc_wgrad_workspace_bytes(1, batch, grid, kh, kw, channels, dtype);      // two row sets per block
}

int sihc_write_read_bwd(const void* h, const void* gz, const void* y, const void* dz, const void* beta,
                        const void* alpha_next, void* hh, void* ddz, float* dweights, void* workspace,
                        size_t workspace_bytes, int64_t batch, int grid, int kh, int kw, int channels, int dtype,
                        int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, 1, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!beta || !alpha_next) return SIHC_ERR_NULL;
    if (gz && dweights && !y) return SIHC_ERR_NULL;          // dalpha_next needs the carrier
    if (dweights && !dz) return SIHC_ERR_NULL;               // dbeta needs the update
    if (!hh && !ddz && !dweights) return SIHC_OK;
    VecChoice vc(vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(h); vc.act(gz); vc.act(y); vc.act(dz); vc.act(hh); vc.act(ddz);
    vc.weight(beta, esize(wdtype)); vc.weight(alpha_next, esize(wdtype));
    if (!vc.elem_ok || (dweights && !aligned(dweights, 4))) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    if (dweights)
        if (int st = check_workspace(workspace, workspace_bytes, sihc_write_read_bwd_workspace_bytes(batch, grid, kh, kw, channels, dtype))) return st;
    float* partial = dweights ? static_cast<float*>(workspace) : nullptr;
    uint32_t blocks = 0;
    cudaError_t e = launch_write_read_bwd(pb, h, gz, y, dz, beta, alpha_next, hh, ddz, partial, &blocks);
    if (e == cudaSuccess && dweights)     // rows 0..S-1 -> dweights[0] (dalpha_next), rows S..2S-1 -> dweights[1] (dbeta)
        e = launch_finish(partial, dweights, blocks, 2u * pb.S, pb.C, pb.S, pb.stream);
    return status_of(e);
}

size_t sihc_wgrad_workspace_bytes(int events, int64_t batch, int grid, int kh, int kw, int channels, int dtype) {
    Problem pb;
    if (make_problem(pb, events, batch, grid, kh, kw, channels, dtype, dtype, nullptr)) return 0;
    return static_cast<size_t>(partial_blocks_bound(pb.M)) * static_cast<size_t>(events) * pb.S * pb.C * sizeof(float);
}

int sihc_read_bwd(const void* x, const void* const* g, const void* alpha, void* dx, float* dalpha, void* workspace,
                  size_t workspace_bytes, int events, int64_t batch, int grid, int kh, int kw, int channels,
                  int dtype, int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, events, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!x || !g || !alpha) return SIHC_ERR_NULL;
    if (!dx && !dalpha) return SIHC_OK;
    VecChoice vc(vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(x); vc.act(dx); vc.weight(alpha, esize(wdtype));
    bool any = false;
    for (int l = 0; l < events; ++l) { vc.act(g[l]); any = any || g[l]; }
    if (!vc.elem_ok || (dalpha && !aligned(dalpha, 4))) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    const size_t carrier_bytes = static_cast<size_t>(pb.M) * pb.S * pb.C * esize(dtype);
    const size_t wbytes = static_cast<size_t>(events) * pb.C * pb.S * sizeof(float);
    if (!any) {   // no output of the read was used
        cudaError_t e = cudaSuccess;
        if (dx) e = cudaMemsetAsync(dx, 0, carrier_bytes, pb.stream);
        if (e == cudaSuccess && dalpha) e = cudaMemsetAsync(dalpha, 0, wbytes, pb.stream);
        return status_of(e);
    }
    if (dalpha) {
        const size_t need = sihc_wgrad_workspace_bytes(events, batch, grid, kh, kw, channels, dtype);
        if (int st = check_workspace(workspace, workspace_bytes, need)) return st;
    }
    float* partial = dalpha ? static_cast<float*>(workspace) : nullptr;
    uint32_t blocks = 0;
    cudaError_t e;
    const int ring = read_bwd_ring_stages(pb.S);
    if (events == 1 && ring > 0 && pb.V > 1) {
        e = launch_read_bwd1_ring(pb, x, g[0], alpha, dx, partial, &blocks, ring, kReadBwdRingThreads);
    } else if (events == 1) {
        e = launch_read_bwd1(pb, x, g[0], alpha, dx, partial, &blocks);
    } else if (dx && dalpha && read_bwd_tiled_applies(pb)) {
        // both adjoints from one pass over x and the gradients: 2S + E elements ("one_pass_adjoints" = 0 restores two kernels)
        e = launch_read_bwd_tiled(pb, x, g, alpha, dx, partial, &blocks);
    } else {
        e = cudaSuccess;
        if (dx) e = launch_write_fwd(pb, nullptr, g, alpha, dx);
        if (e == cudaSuccess && dalpha) e = stage_wgrad(pb, x, g, partial, &blocks);
    }
    if (e == cudaSuccess && dalpha)
        e = launch_finish(partial, dalpha, blocks, static_cast<uint32_t>(events) * pb.S, pb.C, pb.S, pb.stream);
    return status_of(e);
}

int sihc_write_bwd(const void* h, const void* const* dz, const void* beta, void* const* ddz, float* dbeta,
                   void* workspace, size_t workspace_bytes, int events, int64_t batch, int grid, int kh, int kw,
                   int channels, int dtype, int wdtype, void* stream) {
    Problem pb;
    if (int st = make_problem(pb, events, batch, grid, kh, kw, channels, dtype, wdtype, stream)) return st;
    if (!h || !beta) return SIHC_ERR_NULL;
    if (dbeta && !dz) return SIHC_ERR_NULL;
    bool want_ddz = false;
    if (ddz) for (int l = 0; l < events; ++l) want_ddz = want_ddz || ddz[l];
    if (!want_ddz && !dbeta) return SIHC_OK;
    VecChoice vc(vec_width(pb.dtype, pb.S), esize(dtype), pb.C);
    vc.act(h); vc.weight(beta, esize(wdtype));
    for (int l = 0; l < events; ++l) {
        if (dbeta) { if (!dz[l]) return SIHC_ERR_NULL; vc.act(dz[l]); }
        if (ddz) vc.act(ddz[l]);
    }
    if (!vc.elem_ok || (dbeta && !aligned(dbeta, 4))) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    if (dbeta) {
        const size_t need = sihc_wgrad_workspace_bytes(events, batch, grid, kh, kw, channels, dtype);
        if (int st = check_workspace(workspace, workspace_bytes, need)) return st;
    }
    float* partial = dbeta ? static_cast<float*>(workspace) : nullptr;
    uint32_t blocks = 0;
    cudaError_t e;
    const int ring = write_bwd_ring_stages(pb.S);
    if (events == 1 && ring > 0 && pb.V > 1) {
        e = launch_write_bwd1_ring(pb, h, dbeta ? dz[0] : nullptr, beta, want_ddz ? ddz[0] : nullptr, partial, &blocks, ring,
                                   kWriteBwdRingThreads);
    } else if (events == 1) {
        e = launch_write_bwd1(pb, h, dbeta ? dz[0] : nullptr, beta, want_ddz ? ddz[0] : nullptr, partial, &blocks);
    } else if (want_ddz && dbeta && wgrad_tiled_read_applies(pb) && tuning().one_pass_adjoints != 0) {
        // both adjoints from one pass over h: S + 2E elements ("one_pass_adjoints" = 0 restores the two-kernel form)
        e = launch_wgrad_tiled_read(pb, h, dz, beta, ddz, partial, &blocks);
    } else {
        e = cudaSuccess;
        if (want_ddz) e = launch_read_fwd(pb, h, beta, ddz);
        if (e == cudaSuccess && dbeta) e = stage_wgrad(pb, h, dz, partial, &blocks);
    }
    if (e == cudaSuccess && dbeta)
        e = launch_finish(partial, dbeta, blocks, static_cast<uint32_t>(events) * pb.S, pb.C, pb.S, pb.stream);
    return status_of(e);
}

static int make_tri_problem(Problem& pb, int active, int64_t tokens, int channels, int dtype, int gdtype, void* stream) {
    if (int st = check_types(dtype, gdtype)) return st;
    if (active < 1 || active > SIHC_MAX_EVENTS) return SIHC_ERR_EVENTS;
    if (tokens < 1 || channels < 1 || tokens >= (int64_t(1) << 31) || channels > (1 << 24)) return SIHC_ERR_SHAPE;
    pb.dtype = static_cast<DType>(dtype);
    pb.wdtype = static_cast<DType>(gdtype);
    pb.E = active; pb.S = 0;
    pb.M = static_cast<uint32_t>(tokens); pb.g = 1; pb.C = static_cast<uint32_t>(channels);
    pb.V = 1;
    pb.stream = static_cast<cudaStream_t>(stream);
    return SIHC_OK;
}

int sihc_tri_fwd(const void* base, const void* const* dz, const void* gamma, void* out, int active, int64_t tokens,
                 int channels, int dtype, int gdtype, void* stream) {
    Problem pb;
    if (int st = make_tri_problem(pb, active, tokens, channels, dtype, gdtype, stream)) return st;
    if (!base || !dz || !gamma || !out) return SIHC_ERR_NULL;
    VecChoice vc(vec_width(pb.dtype, 0), esize(dtype), pb.C);
    vc.act(base); vc.act(out); vc.weight(gamma, esize(gdtype));
    // gamma rows are C elements apart: vector loads need every row 16-byte aligned
    if ((static_cast<size_t>(pb.C) * esize(gdtype)) % 16 != 0) vc.ok = false;
    for (int l = 0; l < active; ++l) { if (!dz[l]) return SIHC_ERR_NULL; vc.act(dz[l]); }
    if (!vc.elem_ok) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    return status_of(launch_tri_fwd(pb, base, dz, gamma, out));
}

size_t sihc_tri_workspace_bytes(int active, int64_t tokens, int channels, int dtype) {
    Problem pb;
    if (make_tri_problem(pb, active, tokens, channels, dtype, dtype, nullptr)) return 0;
    return static_cast<size_t>(partial_blocks_bound(pb.M)) * static_cast<size_t>(active) * pb.C * sizeof(float);
}

int sihc_tri_bwd(const void* grad, const void* const* dz, const void* gamma, void* const* ddz, float* dgamma,
                 void* workspace, size_t workspace_bytes, int active, int64_t tokens, int channels, int dtype,
                 int gdtype, void* stream) {
    Problem pb;
    if (int st = make_tri_problem(pb, active, tokens, channels, dtype, gdtype, stream)) return st;
    if (!grad || !gamma) return SIHC_ERR_NULL;
    if (dgamma && !dz) return SIHC_ERR_NULL;
    bool want_ddz = false;
    if (ddz) for (int l = 0; l < active; ++l) want_ddz = want_ddz || ddz[l];
    if (!want_ddz && !dgamma) return SIHC_OK;
    VecChoice vc(vec_width(pb.dtype, 0), esize(dtype), pb.C);
    vc.act(grad); vc.weight(gamma, esize(gdtype));
    if ((static_cast<size_t>(pb.C) * esize(gdtype)) % 16 != 0) vc.ok = false;
    for (int l = 0; l < active; ++l) {
        if (dgamma) { if (!dz[l]) return SIHC_ERR_NULL; vc.act(dz[l]); }
        if (ddz) vc.act(ddz[l]);
    }
    if (!vc.elem_ok || (dgamma && !aligned(dgamma, 4))) return SIHC_ERR_ALIGN;
    pb.V = vc.V();
    if (dgamma) {
        const size_t need = sihc_tri_workspace_bytes(active, tokens, channels, dtype);
        if (int st = check_workspace(workspace, workspace_bytes, need)) return st;
    }
    float* partial = dgamma ? static_cast<float*>(workspace) : nullptr;
    uint32_t blocks = 0;
    const void* no_dz[SIHC_MAX_EVENTS] = {};
    cudaError_t e = launch_tri_bwd(pb, grad, dz ? dz : no_dz, gamma, want_ddz ? ddz : nullptr, partial, &blocks);
    if (e == cudaSuccess && dgamma)
        e = launch_finish(partial, dgamma, blocks, static_cast<uint32_t>(active), pb.C, 1, pb.stream);
    return status_of(e);
}

size_t sihc_tri_dgamma_workspace_bytes(int events, int64_t tokens, int channels, int dtype) {
    Problem pb;
    if (make_tri_problem(pb, events, tokens, channels, dtype, dtype, nullptr)) return 0;
    if (events < 2) return 0;
    // the larger of the one-pass kernel's scratch and the per-event form's (used when vector access is not possible)
    const size_t one_pass = tri_dgamma_workspace_bytes(events, pb.M, pb.C, esize(dtype));
    const size_t per_event = sihc_tri_workspace_bytes(events - 1, tokens, channels, dtype);
    return one_pass > per_event ? one_pass : per_event;
}

int sihc_tri_dgamma(const void* const* g, const void* const* dz, float* dgamma, void* workspace, size_t workspace_bytes,
                    int events, int64_t tokens, int channels, int dtype, void* stream) {
    Problem pb;
    if (int st = make_tri_problem(pb, events, tokens, channels, dtype, dtype, stream)) return st;
    if (!g || !dz || !dgamma) return SIHC_ERR_NULL;
    if (!aligned(dgamma, 4)) return SIHC_ERR_ALIGN;
    bool vec = (static_cast<size_t>(pb.C) * esize(dtype)) % 16 == 0;
    for (int l = 0; l < events; ++l) {
        if (l + 1 < events) { if (!dz[l]) return SIHC_ERR_NULL; if (!aligned(dz[l], esize(dtype))) return SIHC_ERR_ALIGN; vec = vec && aligned(dz[l], 16); }
        if (l > 0 && g[l]) { if (!aligned(g[l], esize(dtype))) return SIHC_ERR_ALIGN; vec = vec && aligned(g[l], 16); }
    }
    if (tuning().maxvec_bytes > 0 && tuning().maxvec_bytes < 16) vec = false;
    if (events >= 2)
        if (int st = check_workspace(workspace, workspace_bytes, sihc_tri_dgamma_workspace_bytes(events, tokens, channels, dtype))) return st;
    float* partial = static_cast<float*>(workspace);
    if (vec) {
        pb.V = 4;
        return status_of(launch_tri_dgamma(pb, g, dz, partial, dgamma));
    }
    // scalar path: one per-event reduction per row of the matrix, rows of unused reads and the upper triangle stay zero
    cudaError_t e = cudaMemsetAsync(dgamma, 0, static_cast<size_t>(events) * events * pb.C * sizeof(float), pb.stream);
    for (int i = 1; i < events && e == cudaSuccess; ++i) {
        if (!g[i]) continue;
        Problem row = pb;
        row.E = i; row.V = 1;
        uint32_t blocks = 0;
        e = launch_tri_bwd(row, g[i], dz, dz[0], nullptr, partial, &blocks);     // no ddz: the coefficients are not read
        if (e == cudaSuccess)
            e = launch_finish(partial, dgamma + static_cast<size_t>(i) * events * pb.C, blocks, static_cast<uint32_t>(i), pb.C, 1, pb.stream);
    }
    return status_of(e);
}

}  // extern "C"
