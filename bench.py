"""Benchmark of the SiHC read/write path: fused hyper-connection read + write, forward and backward.

One "step" = one pass of the hot path over one batch of synthetic input:
    read fwd -> write fwd -> read bwd (dX + dalpha) -> write bwd (ddz + dbeta)
on a single connection event (the op-level definition of the headline metric,
"SiHC read/write fwd+bwd HBM GB/s").  Bytes are ALGORITHMIC bytes: per token and
channel element, read fwd S+1, write fwd 2S+1, read bwd 2S+1, write bwd S+2
(total 6S+5 elements of the activation dtype).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Under torchrun (N > 1) every rank runs the same per-GPU workload on its own
shard of the batch (weak scaling) and the small weight gradients are
all-reduced over NCCL inside the step, as in data-parallel training.

``--impl reference`` times the CPU restatement of the reference's unfused
PyTorch path (the oracle) on the host cores; it is the only place besides the
``cpu_baseline`` leg where this file executes anything under ``oracle/``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CELLS = {2: (1, 2), 4: (2, 2), 8: (2, 4), 16: (4, 4)}


def shutdown_group():
    """Leave the process group.  The result line is already printed when this runs; should the teardown of the
    collective library ever block (it waits for every captured graph that holds its collectives to be destroyed),
    a timer ends this process after a minute instead of leaving the job's GPUs occupied."""
    import gc
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return
    sys.stdout.flush()
    timer = threading.Timer(60.0, os._exit, args=(0,))
    timer.daemon = True
    timer.start()
    gc.collect()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    timer.cancel()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--slots", type=int, default=4, help="streams per token n (2/4/8/16)")
    ap.add_argument("--channels", type=int, default=768)
    ap.add_argument("--log2-tokens", type=int, default=20, help="batch x tokens per GPU = 2**this")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--workload", default="op", choices=["op", "stage_ops", "sihc_b_fwd", "sihc_xl_train", "sihc_xl_sample"],
                    help="op: the read/write path itself (headline); the others time the SiHC models around it")
    ap.add_argument("--no-models", action="store_true", help="skip the model-level figures added to the op line")
    ap.add_argument("--sample-steps", type=int, default=50)
    ap.add_argument("--events", type=int, default=24, help="events per stage for --workload stage_ops")
    ap.add_argument("--no-compile", action="store_true",
                    help="run the models' torch sublayers eagerly instead of under torch.compile")
    ap.add_argument("--train-impl", default="graph", choices=["graph", "compiled_ddp"],
                    help="SiHC-XL training step: this package's single-graph step, or whole-model compile + DDP")
    ap.add_argument("--train-schedule", default="literal", choices=["stage", "literal"],
                    help="single-graph step: the literal recurrence (fused write+read step and its fused adjoint; fewest "
                         "bytes at n = 4) or the reference's factored stages with the stage-scoped backward")
    ap.add_argument("--bucket-mb", type=int, default=256, help="gradient bucket size of the single-graph step")
    ap.add_argument("--no-overlap-optimizer", dest="overlap_optimizer", action="store_false",
                    help="single-graph step: one AdamW update after backward instead of per-bucket updates on the side "
                         "stream right after each bucket's all-reduce")
    ap.add_argument("--no-shard-optimizer", dest="shard_optimizer", action="store_false",
                    help="single-graph step: every rank updates all parameters after an all-reduce instead of 1/N of them "
                         "between a reduce-scatter and an all-gather")
    ap.add_argument("--sweep-slots", default="2,4,8", help="n values of --sweep")
    ap.add_argument("--sweep-channels", default="768,1152", help="widths of --sweep")
    ap.add_argument("--sweep-log2", default="12-20", help="range lo-hi of log2(tokens) of --sweep")
    ap.add_argument("--sweep", action="store_true",
                    help="bandwidth sweep over n in {2,4,8}, width in {768,1152}, tokens 2^12..2^20: one JSON line per point")
    return ap.parse_args()


def algorithmic_units(slots: int) -> dict:
    return {"read_fwd": slots + 1, "write_fwd": 2 * slots + 1, "read_bwd": 2 * slots + 1, "write_bwd": slots + 2}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def recorded_traffic_ratio(stage, slots, channels, dtype_name, library_version):
    """(DRAM bytes / algorithmic bytes, source) for one hot-path stage from the tracked ncu record, or (None, why)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None, "no profiles/dram_traffic.json"
    if rec.get("library_version") != library_version:
        return None, f"record is for library version {rec.get('library_version')}, this is {library_version}"
    key = f"single_event/n{slots}/c{channels}/{dtype_name}"
    entry = rec.get("cases", {}).get(key, {}).get(stage)
    if not entry:
        return None, f"no record for {key}/{stage}"
    return float(entry["dram_over_algorithmic"]), f"{entry['source']} ({entry['kernel']}), scaled by tokens"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()           # the exact child we started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        clocks, reasons, mx = [], set(), None
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(clocks)}


def make_inputs(batch, grid, slots, channels, dtype, device, seed=0):
    kh, kw = CELLS[slots]
    gen = torch.Generator(device=device).manual_seed(seed)

    def randn(*shape, mean=0.0, std=1.0):
        t = torch.empty(*shape, device=device, dtype=dtype)
        return t.normal_(mean, std, generator=gen)

    return dict(
        x=randn(batch, grid * kh, grid * kw, channels),
        dz=randn(batch, grid * grid, channels),
        gz=randn(batch, grid * grid, channels),
        gy=randn(batch, grid * kh, grid * kw, channels),
        alpha=randn(1, channels, slots, mean=1.0 / slots, std=0.02),
        beta=randn(1, channels, slots, mean=1.0 / slots, std=0.02),
    )


# ------------------------------------------------------------------------------------------ ours
class DevicePath:
    """The four hot-path launches on resident tensors, straight through the C ABI."""

    def __init__(self, inp, batch, grid, slots, channels, dtype):
        from residual_stream_burden_b200 import _lib
        self.lib, self._lib = _lib.lib, _lib
        self.inp = inp
        kh, kw = CELLS[slots]
        self.geom = (batch, grid, kh, kw, channels)
        self.dt = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
        dev = inp["x"].device
        self.z = torch.empty_like(inp["dz"])
        self.y = torch.empty_like(inp["x"])
        self.dx = torch.empty_like(inp["x"])
        self.ddz = torch.empty_like(inp["dz"])
        # both weight gradients are written by the kernels straight into ONE flat fp32 buffer, so that the
        # data-parallel exchange is a single all-reduce with no packing copies
        self.wgrads = torch.empty(2, 1, channels, slots, device=dev, dtype=torch.float32)
        self.dalpha, self.dbeta = self.wgrads[0], self.wgrads[1]
        nbytes = self.lib.sihc_wgrad_workspace_bytes(1, batch, grid, kh, kw, channels, self.dt)
        self.ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        pa = _lib.ptr_array
        self.p_z, self.p_dz = pa([self.z.data_ptr()]), pa([inp["dz"].data_ptr()])
        self.p_gz, self.p_ddz = pa([inp["gz"].data_ptr()]), pa([self.ddz.data_ptr()])
        self.stream = torch.cuda.current_stream().cuda_stream

    def read_fwd(self):
        i = self.inp
        self._lib.check(self.lib.sihc_read_fwd(i["x"].data_ptr(), i["alpha"].data_ptr(), self.p_z, 1, *self.geom,
                                               self.dt, self.dt, self.stream), "read_fwd")

    def write_fwd(self):
        i = self.inp
        self._lib.check(self.lib.sihc_write_fwd(i["x"].data_ptr(), self.p_dz, i["beta"].data_ptr(), self.y.data_ptr(),
                                                1, *self.geom, self.dt, self.dt, self.stream), "write_fwd")

    def read_bwd(self):
        i = self.inp
        self._lib.check(self.lib.sihc_read_bwd(i["x"].data_ptr(), self.p_gz, i["alpha"].data_ptr(), self.dx.data_ptr(),
                                               self.dalpha.data_ptr(), self.ws.data_ptr(), self.ws.numel(), 1,
                                               *self.geom, self.dt, self.dt, self.stream), "read_bwd")

    def write_bwd(self):
        i = self.inp
        self._lib.check(self.lib.sihc_write_bwd(i["gy"].data_ptr(), self.p_dz, i["beta"].data_ptr(), self.p_ddz,
                                                self.dbeta.data_ptr(), self.ws.data_ptr(), self.ws.numel(), 1,
                                                *self.geom, self.dt, self.dt, self.stream), "write_bwd")

    STAGES = ("read_fwd", "write_fwd", "read_bwd", "write_bwd")


def run_e2e(args, batch, grid, slots, channels, dtype, device, steps):
    """The same step through the public autograd API with HOST buffers.

    The per-GPU batch is streamed in chunks: each chunk's inputs are copied from
    pinned host memory, the four passes run through ``sihc_read`` / ``sihc_write``
    and autograd, and every result is copied back to pinned host memory.  Three
    CUDA streams (copy-in, kernels, copy-out) keep both PCIe directions and the
    GPU busy at once.
    """
    import residual_stream_burden_b200 as R
    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)   # side streams are intended here
    kh, kw = CELLS[slots]
    chunk = min(batch, 128)
    nchunks = (batch + chunk - 1) // chunk
    gen = torch.Generator().manual_seed(1)
    ibits = torch.int16 if dtype == torch.bfloat16 else torch.int32
    # random bit patterns of positive finite values in [2^-31, 1): cheap to generate for GBs of pinned memory
    lo, hi = (0x3000, 0x3F80) if dtype == torch.bfloat16 else (0x30000000, 0x3F800000)

    def host(*shape):
        t = torch.empty(*shape, dtype=dtype).pin_memory()
        t.view(ibits).random_(lo, hi, generator=gen)
        return t

    carrier, work = (chunk, grid * kh, grid * kw, channels), (chunk, grid * grid, channels)
    NB = 3                                                         # chunks in flight: copy-in / compute / copy-out
    h_in = dict(x=host(*carrier), dz=host(*work), gz=host(*work), gy=host(*carrier))
    h_out = [dict(z=host(*work), y=host(*carrier), dx=host(*carrier), ddz=host(*work)) for _ in range(NB)]
    h_dw = torch.empty(2, channels, slots, dtype=dtype).pin_memory()
    alpha = torch.full((channels, slots), 1.0 / slots, device=device, dtype=dtype).requires_grad_()
    beta = torch.full((channels, slots), 1.0, device=device, dtype=dtype).requires_grad_()
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=device) for _ in range(3))
    d_in = [{k: torch.empty_like(v, device=device) for k, v in h_in.items()} for _ in range(NB)]
    sums = torch.zeros(2, channels, slots, device=device, dtype=torch.float32)
    esize = h_in["x"].element_size()
    h2d = sum(v.numel() for v in h_in.values()) * esize * nchunks
    d2h = (sum(v.numel() for v in h_out[0].values()) * nchunks + h_dw.numel()) * esize

    def step():
        # three engines busy at once: H2D of chunk k+1, kernels of chunk k, D2H of chunk k-1
        main_stream = torch.cuda.current_stream()
        for s in (s_in, s_cmp, s_out):
            s.wait_stream(main_stream)
        with torch.cuda.stream(s_cmp):
            sums.zero_()
        in_free = [None] * NB       # event: kernels have consumed input buffer b
        out_free = [None] * NB      # event: D2H of host buffer b has finished
        for ci in range(nchunks):
            b = ci % NB
            buf, out = d_in[b], h_out[b]
            with torch.cuda.stream(s_in):
                if in_free[b] is not None:
                    s_in.wait_event(in_free[b])
                for k in h_in:
                    buf[k].copy_(h_in[k], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                x = buf["x"].detach().requires_grad_()
                dz = buf["dz"].detach().requires_grad_()
                z = R.sihc_read(x, alpha)
                y = R.sihc_write(x, dz, beta)
                dx, da = torch.autograd.grad(z, (x, alpha), buf["gz"])
                ddz, db = torch.autograd.grad(y, (dz, beta), buf["gy"])
                sums[0].add_(da)
                sums[1].add_(db)
                in_free[b] = torch.cuda.Event()
                in_free[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(in_free[b])
                if out_free[b] is not None:
                    s_out.wait_event(out_free[b])
                for name, t in (("z", z), ("y", y), ("dx", dx), ("ddz", ddz)):
                    t.record_stream(s_out)
                    out[name].copy_(t, non_blocking=True)
                out_free[b] = torch.cuda.Event()
                out_free[b].record(s_out)
        for s in (s_in, s_cmp, s_out):
            main_stream.wait_stream(s)
        h_dw.copy_(sums.to(dtype), non_blocking=True)

    step()
    torch.cuda.synchronize()
    for out in h_out[:min(NB, nchunks)]:        # the streamed results are real numbers, not Inf/NaN patterns
        assert all(bool(torch.isfinite(t.float()).all()) for t in out.values()), "non-finite end-to-end result"
    assert bool(torch.isfinite(h_dw.float()).all())
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    seconds = (time.perf_counter() - t0) / steps
    return seconds, h2d, d2h, chunk


# ------------------------------------------------------------------------------------------ sweep
def run_sweep(args, device, rank, world):
    """Forward (read+write) and backward (read bwd + write bwd) bandwidth for every point of the sweep.

    Small points fit in the 126 MB L2, so each point rotates over enough independent buffer sets that
    the data touched between two uses of a set exceeds 512 MB; GB/s is always algorithmic bytes / time.
    """
    import torch.distributed as dist
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    esize = 2 if dtype == torch.bfloat16 else 4
    peak, peak_kind = load_peaks()
    grid = 16
    lo, hi = (int(v) for v in args.sweep_log2.split("-"))
    for slots in (int(v) for v in args.sweep_slots.split(",")):
        for channels in (int(v) for v in args.sweep_channels.split(",")):
            for log2m in range(lo, hi + 1):
                tokens = 1 << log2m
                batch = tokens // (grid * grid)
                units = algorithmic_units(slots)
                set_bytes = (4 * slots + 4) * tokens * channels * esize       # x, gy, y, dx + dz, gz, z, ddz
                nsets = max(1, min(64, -(-(512 << 20) // set_bytes)))
                paths = []
                for k in range(nsets):
                    inp = make_inputs(batch, grid, slots, channels, dtype, device, seed=k)
                    paths.append(DevicePath(inp, batch, grid, slots, channels, dtype))
                reps = max(3, min(50, (1 << 22) // tokens))

                def timed(names):
                    """ms per pass over `names`.  The launches of one rotation over the buffer sets are captured
                    in a CUDA graph and the graph is replayed: at the small points a pass is a few 10 us of GPU work
                    and would otherwise be bound by the host's launch calls, not by the kernels."""
                    for pth in paths:                                            # warm-up: every set once
                        for n in names:
                            getattr(pth, n)()
                    torch.cuda.synchronize()
                    side = torch.cuda.Stream()
                    for pth in paths:
                        pth.stream = side.cuda_stream
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        for pth in paths:
                            for n in names:
                                getattr(pth, n)()
                    for pth in paths:
                        pth.stream = torch.cuda.current_stream().cuda_stream
                    rounds = max(1, -(-reps // nsets))
                    graph.replay()
                    torch.cuda.synchronize()
                    if world > 1:
                        dist.barrier()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(rounds):
                        graph.replay()
                    b.record()
                    torch.cuda.synchronize()
                    ms = a.elapsed_time(b) / (rounds * nsets)
                    del graph
                    if world > 1:
                        t = torch.tensor([ms], device=device)
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                        ms = float(t.item())
                    return ms

                fwd_ms = timed(("read_fwd", "write_fwd"))
                bwd_ms = timed(("read_bwd", "write_bwd"))
                unit = tokens * channels * esize
                fwd = world * (units["read_fwd"] + units["write_fwd"]) * unit / fwd_ms / 1e6
                bwd = world * (units["read_bwd"] + units["write_bwd"]) * unit / bwd_ms / 1e6
                tot = world * sum(units.values()) * unit / (fwd_ms + bwd_ms) / 1e6
                if rank == 0:
                    print(json.dumps({"sweep": True, "n": slots, "channels": channels, "log2_tokens": log2m,
                                      "n_gpus": world, "dtype": args.dtype, "buffer_sets": nsets, "launch": "cuda graph",
                                      "fwd_ms": round(fwd_ms, 4), "bwd_ms": round(bwd_ms, 4),
                                      "fwd_GBs": round(fwd, 1), "bwd_GBs": round(bwd, 1), "fwd_bwd_GBs": round(tot, 1),
                                      "frac_of_peak": round(tot / world / peak, 4), "peak": peak,
                                      "peak_source": peak_kind}), flush=True)
                del paths
                torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------------ stage ops
def run_stage_ops(args, device, steps, warmup):
    """The multi-event stage operators one by one on SiHC-B's stage shapes (the SiHC-B forward configuration: batch 256,
    256 tokens, n=4, width 768, E=24 events): read(E), triangular(E-1), write(E) and their backward calls, plus the
    literal schedule's fused step and its fused adjoint, the one-pass stage coefficient gradient and the device's
    write-only bandwidth.  GB/s are algorithmic bytes (read S+E, write 2S+E, triangular J+2, read bwd 2S+E and
    write bwd S+2E where one pass produces both adjoints (4 slots; >= 12 and >= 8 events) else 2(S+E) as two kernels, triangular bwd
    2J+1, literal step 2S+2, its adjoint 3S+3, stage dgamma 2(E-1)) over the CUDA-event time of the C ABI call; `value` is the six factored-stage operators as a set.  The reference's own
    Triton operators are timed on the same tensors as a labelled comparator."""
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    esize = 2 if dtype == torch.bfloat16 else 4
    S, C, E, g = args.slots, args.channels, args.events, 16
    kh, kw = CELLS[S]
    tokens = 1 << min(args.log2_tokens, 16)
    B = tokens // 256
    gen = torch.Generator(device=device).manual_seed(0)

    def rnd(*shape, std=1.0, mean=0.0):
        return torch.empty(*shape, device=device, dtype=dtype).normal_(mean, std, generator=gen)

    x, gy, y = rnd(B, g * kh, g * kw, C), rnd(B, g * kh, g * kw, C), torch.empty(B, g * kh, g * kw, C, device=device, dtype=dtype)
    dz = [rnd(B, 256, C) for _ in range(E)]
    out = [torch.empty(B, 256, C, device=device, dtype=dtype) for _ in range(E)]
    w = rnd(E, C, S, std=0.02, mean=1.0 / S)
    gam = rnd(E, C, std=0.05)
    dw = torch.empty(E, C, S, device=device, dtype=torch.float32)
    dgam = torch.empty(E, C, device=device, dtype=torch.float32)
    nbytes = max(lib.sihc_wgrad_workspace_bytes(E, B, g, kh, kw, C, code), lib.sihc_tri_workspace_bytes(E, tokens, C, code),
                 lib.sihc_tri_dgamma_workspace_bytes(E, tokens, C, code), 16)
    dgam_full = torch.empty(E, E, C, device=device, dtype=torch.float32)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    st = torch.cuda.current_stream().cuda_stream
    pa = _lib.ptr_array
    p_dz, p_out = pa([t.data_ptr() for t in dz]), pa([t.data_ptr() for t in out])
    geom = (B, g, kh, kw, C, code, code, st)
    J = E - 1 if E > 1 else 1
    ops = {
        "read_fwd": (lambda: lib.sihc_read_fwd(x.data_ptr(), w.data_ptr(), p_out, E, *geom), S + E),
        "triangular_fwd": (lambda: lib.sihc_tri_fwd(out[0].data_ptr(), p_dz, gam.data_ptr(), y.data_ptr(), J, tokens, C, code, code, st), J + 2),
        "write_fwd": (lambda: lib.sihc_write_fwd(x.data_ptr(), p_dz, w.data_ptr(), y.data_ptr(), E, *geom), 2 * S + E),
        # one pass (S+2E, 2S+E) where the weight-gradient kernel also produces the other adjoint (4 slots; write from 8
        # events, read from 12), else two kernels
        "write_bwd": (lambda: lib.sihc_write_bwd(gy.data_ptr(), p_dz, w.data_ptr(), p_out, dw.data_ptr(), ws.data_ptr(), ws.numel(), E, *geom),
                      S + 2 * E if (S == 4 and E >= 8) else 2 * (S + E)),
        "triangular_bwd": (lambda: lib.sihc_tri_bwd(out[0].data_ptr(), p_dz, gam.data_ptr(), p_out, dgam.data_ptr(), ws.data_ptr(), ws.numel(), J, tokens, C, code, code, st), 2 * J + 1),
        "read_bwd": (lambda: lib.sihc_read_bwd(x.data_ptr(), p_dz, w.data_ptr(), y.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), E, *geom),
                     2 * S + E if (S == 4 and E >= 12) else 2 * (S + E)),
    }
    # literal schedule: one event's write fused with the next read (2S+2) and the fused adjoint of that step (3S+3)
    dw2 = torch.empty(2, C, S, device=device, dtype=torch.float32)
    ws_lit = torch.empty(max(lib.sihc_write_read_bwd_workspace_bytes(B, g, kh, kw, C, code), 16), dtype=torch.uint8, device=device)
    hh = torch.empty_like(x)
    ops["literal_step_fwd"] = (lambda: lib.sihc_write_read_fwd(x.data_ptr(), dz[0].data_ptr(), w[0].data_ptr(), w[1 % E].data_ptr(),
                                                               y.data_ptr(), out[0].data_ptr(), *geom), 2 * S + 2)
    ops["literal_step_bwd"] = (lambda: lib.sihc_write_read_bwd(gy.data_ptr(), dz[1 % E].data_ptr(), y.data_ptr(), dz[0].data_ptr(),
                                                               w[0].data_ptr(), w[1 % E].data_ptr(), hh.data_ptr(), out[1 % E].data_ptr(),
                                                               dw2.data_ptr(), ws_lit.data_ptr(), ws_lit.numel(), *geom), 3 * S + 3)
    if E > 1:       # whole-stage coefficient gradient of the stage-scoped backward: every tensor read once
        ops["stage_dgamma"] = (lambda: lib.sihc_tri_dgamma(p_out, p_dz, dgam_full.data_ptr(), ws.data_ptr(), ws.numel(), E, tokens, C, code, st), 2 * (E - 1))
    peak, peak_kind = load_peaks()
    res = {}
    launches0 = _lib.launch_count()
    # write-only bandwidth of the device (16-byte streaming stores, 1 GiB): the bound for mostly-output operators
    probe = torch.empty(1 << 30, dtype=torch.uint8, device=device)
    for _ in range(3):
        _lib.check(lib.sihc_probe_store_stream(probe.data_ptr(), probe.numel(), st), "store stream")
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(10):
        lib.sihc_probe_store_stream(probe.data_ptr(), probe.numel(), st)
    b.record()
    torch.cuda.synchronize()
    store_gbs = probe.numel() * 10 / a.elapsed_time(b) / 1e6
    del probe
    for name, (fn, units) in ops.items():
        for _ in range(warmup):
            _lib.check(fn(), name)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        gbs = units * tokens * C * esize / ms / 1e6
        res[name] = {"ms": round(ms, 4), "units": units, "GB/s": round(gbs, 1), "frac": round(gbs / peak, 4)}
    # headline of this workload: the six operators of one factored stage as a set; the other entries are reported per op
    stage_set = ("read_fwd", "triangular_fwd", "write_fwd", "write_bwd", "triangular_bwd", "read_bwd")
    total_ms = sum(res[k]["ms"] for k in stage_set)
    total_units = sum(res[k]["units"] for k in stage_set)
    value = total_units * tokens * C * esize / total_ms / 1e6
    comparators = reference_triton_comparator(x, gy, dz, out, w, gam, J, steps, warmup,
                                              {k: v[1] for k, v in ops.items() if k in ("read_fwd", "triangular_fwd", "write_fwd", "write_bwd",
                                                                                       "triangular_bwd", "read_bwd")},
                                              tokens * C * esize)
    print(json.dumps({"metric": "sihc_stage_ops_bandwidth", "value": round(value, 1), "unit": "GB/s", "n_gpus": 1,
                      "steps": steps, "warmup": warmup, "ms_per_step": round(total_ms, 4), "higher_is_better": True,
                      "dtype": args.dtype, "data": "synthetic",
                      "config": {"workload": f"stage operators, E={E} events, n={S}, width {C}, {tokens} tokens"},
                      "peak": peak, "peak_source": peak_kind, "store_stream_GBs": round(store_gbs, 1), "ops": res,
                      "comparators": comparators,
                      "gpu_launches": int(_lib.launch_count() - launches0)}))


def reference_triton_comparator(x, gy, dz, out, w, gam, J, steps, warmup, units, unit_bytes):
    """The reference's own Triton operators (sihc/models/sihc/sublayer_kernels.py:219-379, unmodified copy under
    ``oracle/_ref``) timed on the same tensors, same GPU, same method, as a labelled comparator.  Each backward is
    the call sequence of the reference's autograd formula, run eagerly (its triangular backward leaves the per-edge
    products to torch, which Inductor would fuse in a compiled model).  Their GB/s use the same byte counts as this library's
    operators, so the ratio of the two is the ratio of times.  Skipped, with the reason, when the copy is absent,
    the shape is outside what the reference supports (8/12/16/24 events, 4/16 slots) or Triton cannot compile."""
    label = "reference Triton operators (sihc/models/sihc/sublayer_kernels.py), same tensors"
    from oracle.make_ref import ref_path
    path = ref_path()
    E, S = w.shape[0], w.shape[2]
    if path is None:
        return {"what": label, "skipped": "oracle/_ref is absent"}
    if E not in (8, 12, 16, 24) or S not in (4, 16):
        return {"what": label, "skipped": f"the reference has no {E}-event / {S}-slot operator"}
    try:
        if path not in sys.path:
            sys.path.insert(0, path)
        import sihc.models.sihc.sublayer_kernels as sk
        g0, gj = out[0], gam[:J].contiguous()
        calls = {
            "read_fwd": lambda: sk.sublayer_read(x, w),
            "triangular_fwd": lambda: sk.sublayer_triangular(g0, dz[:J], gj),
            "write_fwd": lambda: sk.sublayer_write(x, dz, w),
            "write_bwd": lambda: (sk.sublayer_read(gy, w), sk._weights_backward(gy, dz, w)),
            "triangular_bwd": lambda: (sk._tri_gamma_backward(g0, dz[:J], gj),
                                       [(g0.float() * gj[i].float()).to(g0.dtype) for i in range(J)]),
            "read_bwd": lambda: (sk._write_impl(x, dz, w, False), sk._weights_backward(x, dz, w)),
        }
        res = {}
        for name, fn in calls.items():
            for _ in range(max(warmup, 3)):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            res[name] = {"ms": round(ms, 4), "GB/s": round(units[name] * unit_bytes / ms / 1e6, 1)}
        return {"what": label, "triton": __import__("triton").__version__, "ops": res,
                "ms_total": round(sum(v["ms"] for v in res.values()), 4)}
    except Exception as exc:                                       # noqa: BLE001
        return {"what": label, "skipped": repr(exc)[:300]}


# ------------------------------------------------------------------------------------------ models
def time_device(fn, steps, warmup, world, device):
    """W untimed + K timed calls, CUDA events on the current stream, barrier on both sides, max over ranks."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def model_workload(kind, device, rank, world, local_rank, steps, warmup, sample_steps=50, compile_model=True,
                   train_impl="graph", bucket_mb=256, overlap_optimizer=True, train_schedule="literal", shard_optimizer=True):
    """SiHC-B forward (batch 256), SiHC-XL training step (batch 32 per GPU, DDP) or SiHC-XL Heun sampling
    (batch 256 per GPU, CFG 2.4 on [0.1, 0.9]); bf16 autocast over fp32 parameters, synthetic N(0,1) images,
    random-init weights with opened gates.  Inputs start in pinned host memory every step.

    As in the reference's own benchmark (compile, then DDP: sihc/bench/fusion_profile.py:113-195) the model runs
    under ``torch.compile(fullgraph=True, mode="reduce-overhead")``; that fuses the torch sublayers' elementwise
    glue (norms, modulation, RoPE, gates) and replays each pass as a CUDA graph, routing launches included.  The routing operators stay opaque ``sihc_b200::*`` custom ops inside the graph: every read,
    write and triangular step is this package's CUDA kernel either way."""
    from residual_stream_burden_b200 import _lib
    from residual_stream_burden_b200.model import sample_heun, sihc_b, sihc_xl, velocity_training_batch
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.manual_seed(1234 + rank)
    gen = torch.Generator().manual_seed(rank)
    launches0 = _lib.launch_count()
    torch.cuda.reset_peak_memory_stats(device)
    if kind == "sihc_b_fwd":
        batch = 256
        model = sihc_b().to(device).eval()
        model.open_gates()
        model.inference_schedule = "literal"        # n = 4: fused write+read steps move fewer bytes than the factored stage
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):     # one eager pass: counts this
            model(torch.randn(2, 3, 256, 256, device=device), torch.rand(2, device=device),  # library's launches
                  torch.zeros(2, dtype=torch.long, device=device))              # (graph replays are not counted)
        per_step_launches = _lib.launch_count() - launches0
        net = torch.compile(model, fullgraph=True, mode="reduce-overhead") if compile_model else model
        x_host = torch.randn(batch, 3, 256, 256, generator=gen).pin_memory()
        t = torch.rand(batch, device=device)
        y = torch.randint(0, 1000, (batch,), device=device)

        def step():
            torch.compiler.cudagraph_mark_step_begin()
            x = x_host.to(device, non_blocking=True)
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                out = net(x, t, y)
            return float(out.float().abs().mean())          # device -> host read of a scalar

        ms = time_device(step, steps, warmup, world, device)
        name = "SiHC-B forward, 12 blocks x 768, n=4, batch 256 per GPU, bf16 autocast, literal fused write+read schedule"
    elif kind == "sihc_xl_train" and train_impl == "graph":
        # The whole step - forward, loss, backward, bucketed gradient all-reduce on a side stream, fused AdamW - as
        # ONE hand-captured CUDA graph; stages run the stage-scoped backward; only the torch sublayers are compiled.
        from residual_stream_burden_b200.train import TrainStep
        batch = 32
        model = sihc_xl().to(device)
        model.open_gates()
        trainer = TrainStep(model, batch, lr=2e-4, betas=(0.9, 0.95), weight_decay=0.0, compile_model=compile_model,
                            bucket_mb=bucket_mb, overlap_optimizer=overlap_optimizer, schedule=train_schedule,
                            shard_optimizer=shard_optimizer)
        x_host = torch.randn(batch, 3, 256, 256, generator=gen).pin_memory()
        y = torch.randint(0, 1000, (batch,), device=device)
        trainer.step(x_host, y)                     # first eager pass: compiles the sublayers
        torch.cuda.synchronize()
        launches0 = _lib.launch_count()
        trainer.step(x_host, y)                     # second eager pass: counts this library's launches per step
        torch.cuda.synchronize()
        per_step_launches = _lib.launch_count() - launches0

        def step():
            return float(trainer.step(x_host, y))           # H2D copy of the images, graph replay, D2H read of the loss

        try:
            ms = time_device(step, steps, warmup, world, device)
            assert trainer.graph is not None
        finally:
            trainer.close()        # the graph holds captured collectives: it must be gone before the group is destroyed
        name = ("SiHC-XL training step, 28 blocks x 1152, n=4, stages 8+12+8, batch 32 per GPU, bf16 autocast + fp32 AdamW, "
                "one CUDA graph per step (%s, gradient all-reduce in %d MB buckets under backward%s)"
                % ("factored stages with the stage-scoped backward" if train_schedule == "stage"
                   else "literal schedule: fused write+read step and its fused adjoint",
                   bucket_mb, (", per-bucket AdamW on the side stream" + (" on this rank's 1/N of every parameter "
                               "(reduce-scatter, update, all-gather)" if shard_optimizer and world > 1 else ""))
                   if overlap_optimizer else ""))
    elif kind == "sihc_xl_train":
        batch = 32
        model = sihc_xl().to(device)
        model.open_gates()
        with torch.autocast("cuda", dtype=torch.bfloat16):                      # one eager forward+backward: counts
            model(torch.randn(2, 3, 256, 256, device=device), torch.rand(2, device=device),   # this library's launches
                  torch.zeros(2, dtype=torch.long, device=device)).float().mean().backward()
        model.zero_grad(set_to_none=True)
        per_step_launches = _lib.launch_count() - launches0
        net = torch.compile(model, fullgraph=True, mode="reduce-overhead") if compile_model else model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP
            # 512 MB buckets: the compiled backward is one autograd node, so every gradient becomes ready at its
            # end and the default 25 MB buckets turn into ~110 back-to-back latency-bound all-reduces
            # (measured on 2 x B200: 85.4 ms per step with 25 MB buckets, 66.7 ms with 512 MB, 62.0 ms on one GPU)
            net = DDP(net, device_ids=[local_rank], gradient_as_bucket_view=True, bucket_cap_mb=512)
        opt = torch.optim.AdamW(model.parameters(), lr=2e-4, betas=(0.9, 0.95), weight_decay=0.0, fused=True)
        x_host = torch.randn(batch, 3, 256, 256, generator=gen).pin_memory()
        y = torch.randint(0, 1000, (batch,), device=device)

        def step():
            torch.compiler.cudagraph_mark_step_begin()
            x = x_host.to(device, non_blocking=True)
            z, t, v = velocity_training_batch(x)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                pred = net(z, t, y)
            loss = (pred.float() - v).square().mean()
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return float(loss.detach())                     # device -> host read of the loss

        ms = time_device(step, steps, warmup, world, device)
        name = ("SiHC-XL training step, 28 blocks x 1152, n=4, stages 8+12+8, batch 32 per GPU, bf16 autocast + fp32 AdamW, "
                "whole-model torch.compile + DistributedDataParallel (the reference trainer's arrangement)")
    else:
        batch = 256
        model = sihc_xl().to(device).eval()
        model.open_gates()
        model.inference_schedule = "literal"
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            model(torch.randn(2, 3, 256, 256, device=device), torch.rand(2, device=device),
                  torch.zeros(2, dtype=torch.long, device=device))
        per_step_launches = (_lib.launch_count() - launches0) * 2 * (2 * sample_steps - 1)   # two forwards per guided evaluation
        net = torch.compile(model, fullgraph=True, mode="reduce-overhead") if compile_model else model
        y = torch.randint(0, 1000, (batch,), device=device)

        def step():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                img = sample_heun(net, y, steps=sample_steps, cfg_scale=2.4, interval=(0.1, 0.9))
            return float(img.float().abs().mean())

        ms = time_device(step, steps, warmup, world, device)
        name = f"SiHC-XL Heun sampling, {sample_steps} steps, CFG 2.4 on [0.1,0.9], batch 256 per GPU, bf16 autocast, literal fused write+read schedule"
    if not (kind == "sihc_xl_train" and train_impl == "graph"):
        name += ", torch.compile (CUDA graphs) around the torch sublayers" if compile_model else ", eager"
    elif not compile_model:
        name += ", sublayers not compiled"
    res = {"workload": name, "img_per_s": round(world * batch / (ms * 1e-3), 2),
           "img_per_s_per_gpu": round(batch / (ms * 1e-3), 2), "ms_per_step": round(ms, 3),
           "steps": steps, "warmup": warmup, "global_batch": world * batch, "routing_launches_per_step": per_step_launches,
           "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 2**30, 2)}
    del model
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------ CPU
def cpu_path(slots):
    """``(read, write, kind)`` of the unfused eager path on the host: the reference's own ``read_torch`` /
    ``write_torch`` (sihc/bench/fusion_controls.py:14-31) from the unmodified copy under ``oracle/_ref`` when it is
    there and defines this cell (square cells only), else the oracle's restatement of them."""
    from oracle.make_ref import ref_path
    path = ref_path()
    if path is not None and slots in (4, 16):
        if path not in sys.path:
            sys.path.insert(0, path)
        from sihc.bench import fusion_controls as fc
        return fc.read_torch, fc.write_torch, "reference"
    from oracle import sihc_oracle as O
    return O.read, O.write, "port"


def cpu_step_factory(batch, grid, slots, channels, dtype):
    """The reference's unfused eager path on the host: read_torch/write_torch + autograd."""
    read, write, kind = cpu_path(slots)
    inp = make_inputs(batch, grid, slots, channels, dtype, torch.device("cpu"))

    def step():
        x = inp["x"].clone().requires_grad_()
        alpha = inp["alpha"][0].clone().requires_grad_()
        beta = inp["beta"][0].clone().requires_grad_()
        dz = inp["dz"].clone().requires_grad_()
        z = read(x, alpha)
        y = write(x, [dz], [beta])
        torch.autograd.grad(z, (x, alpha), inp["gz"])
        torch.autograd.grad(y, (dz, beta), inp["gy"])

    return step, kind


def time_cpu(batch, grid, slots, channels, dtype, reps, warm=1):
    """Seconds per pass of the host path with every host thread, and which implementation ran."""
    torch.set_num_threads(os.cpu_count() or 1)
    step, kind = cpu_step_factory(batch, grid, slots, channels, dtype)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    return (time.perf_counter() - t0) / reps, kind


def main():
    args = parse_args()
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    esize = 2 if dtype == torch.bfloat16 else 4
    slots, channels, grid = args.slots, args.channels, 16
    tokens = 1 << args.log2_tokens
    batch = max(1, tokens // (grid * grid))
    tokens = batch * grid * grid
    units = algorithmic_units(slots)
    step_bytes = sum(units.values()) * tokens * channels * esize
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    workload = (f"SiHC read+write fwd+bwd, single event, n={slots} streams, width {channels}, "
                f"batch x tokens = 2^{args.log2_tokens} per GPU ({batch} x {grid * grid}), {args.dtype}")
    config = {"workload": workload, "slots": slots, "channels": channels, "tokens_per_gpu": tokens,
              "l2": "inputs larger than L2 (no flush needed)", "parallelism": f"dp{world}"}

    if args.impl == "reference":
        if rank != 0:
            return
        cores = os.cpu_count() or 1
        sample_batch = min(batch, 256)
        sample_tokens = sample_batch * grid * grid
        for _ in range(max(0, min(args.warmup, 1))):
            time_cpu(sample_batch, grid, slots, channels, dtype, 1, warm=0)
        sec, kind = time_cpu(sample_batch, grid, slots, channels, dtype, max(1, min(args.steps, 10)), warm=0)
        gbs = sum(units.values()) * sample_tokens * channels * esize / sec / 1e9
        sample = (f"{sample_batch} images ({sample_tokens} tokens) of the workload per step, torch eager on CPU, "
                  + ("the reference's read_torch / write_torch + autograd" if kind == "reference"
                     else "the oracle's restatement of read_torch / write_torch + autograd"))
        line = {"impl": "reference", "metric": "sihc_read_write_fwd_bwd_bandwidth", "value": gbs, "unit": "GB/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype,
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from residual_stream_burden_b200 import _lib

    if args.sweep:
        run_sweep(args, device, rank, world)
        if world > 1:
            shutdown_group()
        return
    if args.workload == "stage_ops":
        if rank == 0:
            run_stage_ops(args, device, args.steps, max(args.warmup, 3))
        if world > 1:
            shutdown_group()
        return
    if args.workload != "op":
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        # one sampling pass is already 2*steps-1 guided evaluations (198 forwards): one warm-up pass is enough there
        warm = max(args.warmup, 1) if args.workload == "sihc_xl_sample" else max(args.warmup, 3)
        res = model_workload(args.workload, device, rank, world, local_rank, args.steps, warm,
                             args.sample_steps, not args.no_compile, args.train_impl, args.bucket_mb,
                             args.overlap_optimizer, args.train_schedule, args.shard_optimizer)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            print(json.dumps({"metric": args.workload + "_throughput", "value": res["img_per_s"], "unit": "img/s",
                              "n_gpus": world, "steps": args.steps, "warmup": warm,
                              "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                              "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": res["workload"], "global_batch": res["global_batch"],
                                         "parallelism": f"dp{world}"},
                              "gpu_launches": res["routing_launches_per_step"] * args.steps,
                              "peak_mem_gb": res["peak_mem_gb"], "clocks": clocks}))
        if world > 1:
            shutdown_group()
        return

    from residual_stream_burden_b200.dist import allreduce_weight_grads
    inp = make_inputs(batch, grid, slots, channels, dtype, device, seed=rank)
    path = DevicePath(inp, batch, grid, slots, channels, dtype)

    def step(events=None):
        for k, name in enumerate(DevicePath.STAGES):
            if events is not None:
                events[k][0].record()
            getattr(path, name)()
            if events is not None:
                events[k][1].record()
        if world > 1:       # data-parallel exchange of the small weight gradients: one NCCL all-reduce
            allreduce_weight_grads([path.wgrads])

    # The clock sampler (nvidia-smi, 100 ms period) needs a few hundred ms to deliver its first line, longer
    # than the timed region itself.  It is started first and the GPU is kept under the same load until it has
    # reported three samples (bounded, single GPU only; these passes are not warm-up steps and are not counted);
    # then come exactly W warm-up steps and K timed steps.  Its record covers all of it.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_wait = time.perf_counter()
    while (rank == 0 and world == 1 and sampler.proc is not None and len(sampler.samples) < 3
           and time.perf_counter() - t_wait < 3.0):
        step()
        torch.cuda.synchronize()
    warmup = max(args.warmup, 3)           # the timing rules ask for at least three
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    per_kernel = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(4)]
                  for _ in range(args.steps)]
    launches0 = _lib.launch_count()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(args.steps):
        step(per_kernel[k])
    end.record()
    torch.cuda.synchronize()
    launches = _lib.launch_count() - launches0
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    kernel_ms = {name: statistics.mean(ev[k][0].elapsed_time(ev[k][1]) for ev in per_kernel)
                 for k, name in enumerate(DevicePath.STAGES)}
    peak, peak_kind = load_peaks()
    kernels = {}
    for name in DevicePath.STAGES:
        nbytes = units[name] * tokens * channels * esize
        gbs = nbytes / (kernel_ms[name] * 1e-3) / 1e9
        kernels[name] = {"ms": round(kernel_ms[name], 4), "GB/s": round(gbs, 1), "frac": round(gbs / peak, 4)}
    dominant = max(DevicePath.STAGES, key=lambda n: kernel_ms[n])
    dom_bytes = units[dominant] * tokens * channels * esize
    achieved = dom_bytes / (kernel_ms[dominant] * 1e-3) / 1e9
    # DRAM traffic per launch is not measured in this run: it is the ncu figure (dram__bytes_read.sum +
    # dram__bytes_write.sum over algorithmic bytes) recorded in profiles/dram_traffic.json for this kernel and
    # configuration, scaled to this launch (traffic is proportional to tokens); null when the record is for
    # another library version or configuration.
    ncu_ratio, ncu_source = recorded_traffic_ratio(dominant, slots, channels, args.dtype, _lib.lib.sihc_version())
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_source": f"{peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": dom_bytes,
                "traffic": int(dom_bytes * ncu_ratio) if ncu_ratio else None,
                "traffic_source": ncu_source,
                "all_kernels": kernels, "step_frac_of_peak": round(value / world / peak, 4)}

    # The legs below add to the headline line.  On one GPU a failure in one of them is recorded in its place and
    # the line is still printed.  With several ranks a rank-local failure (out of memory, a compile error) must
    # not be swallowed: the other ranks would wait for it inside a collective on their GPUs, so the exception
    # propagates, this process exits non-zero and the launcher ends the whole job at once.
    e2e = None
    if not args.no_e2e:
        try:
            sec, h2d, d2h, chunk = run_e2e(args, batch, grid, slots, channels, dtype, device, args.e2e_steps)
            err = None
        except Exception as exc:                                   # noqa: BLE001
            if world > 1:
                raise
            sec, h2d, d2h, chunk, err = float("inf"), 0, 0, 0, repr(exc)[:300]
        if world > 1:
            t = torch.tensor([sec], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        if sec == float("inf"):
            e2e = {"value": None, "unit": "GB/s", "error": err or "failed on another rank"}
        else:
            e2e = {"value": round(world * step_bytes / sec / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": d2h, "ms_per_step": round(sec * 1e3, 2),
                   "api": "sihc_read / sihc_write + torch.autograd, pinned host buffers, chunks of %d images" % chunk}

    cpu = None
    if rank == 0 and not args.no_cpu and world == 1:
        sample_batch = min(batch, 256)                 # about ten seconds of CPU work in total
        sec, kind = time_cpu(sample_batch, grid, slots, channels, dtype, reps=5)
        sample_tokens = sample_batch * grid * grid
        cpu = {"value": round(sum(units.values()) * sample_tokens * channels * esize / sec / 1e9, 3), "unit": "GB/s",
               "cores": os.cpu_count() or 1, "kind": kind,
               "sample": f"{sample_batch} images ({sample_tokens} tokens) of the workload, torch eager on CPU, "
                         f"{sec * 1e3:.0f} ms per pass"}

    models = None
    if not args.no_models:
        # second half of the headline metric: the models around the path, same process, same GPUs
        del path, inp
        torch.cuda.empty_cache()
        cm = not args.no_compile
        models = {}
        for kind in (("sihc_xl_train", "sihc_b_fwd") if world == 1 else ("sihc_xl_train",)):
            try:
                models[kind] = model_workload(kind, device, rank, world, local_rank, 20, 8, 50, cm,
                                              args.train_impl, args.bucket_mb, args.overlap_optimizer,
                                              args.train_schedule, args.shard_optimizer)
            except Exception as exc:                               # noqa: BLE001
                if world > 1:
                    raise                                          # see above: never leave the peers waiting
                models[kind] = {"error": repr(exc)[:300]}
                torch.cuda.empty_cache()

    if rank == 0:
        line = {"metric": "sihc_read_write_fwd_bwd_bandwidth", "value": round(value, 1), "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "config": config,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
                "clocks": clocks, "models": models}
        print(json.dumps(line))
    if world > 1:
        shutdown_group()


if __name__ == "__main__":
    main()
