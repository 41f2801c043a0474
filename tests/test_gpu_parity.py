"""CUDA kernels vs the CPU oracle and the reference-generated golden fixtures.

Everything here goes through the C ABI (ctypes) of the in-tree library, either
directly or via the ``sihc_b200::*`` operators.  Tolerances:
  * fp32: relative L2 <= 1e-5 and elementwise atol = rtol = 2e-4 (the reference's
    own bound, research/tests/test_sublayer_kernels.py:33-36);
  * bf16 storage with fp32 accumulation: relative L2 <= 2e-2 and elementwise
    atol 0.025 / rtol 0.03.
"""

import pytest
import torch

from conftest import load_golden, regenerate_op_inputs
from oracle import sihc_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def R():
    import residual_stream_burden_b200 as pkg
    return pkg


def close(actual, expected, dtype, what=""):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == e.shape, (what, a.shape, e.shape)
    rel = (a - e).norm() / e.norm().clamp_min(1e-12)
    assert rel <= (1e-5 if dtype == torch.float32 else 2e-2), (what, float(rel))
    atol, rtol = (2e-4, 2e-4) if dtype == torch.float32 else (0.025, 0.03)
    torch.testing.assert_close(a, e, atol=atol, rtol=rtol, msg=lambda m: f"{what}: {m}")


def run_all(R, x, alpha, beta, dz, gz, gy):
    """Forward and every gradient of the stage read and write through the public ops."""
    xd, ad, bd = (t.to(DEV).requires_grad_() for t in (x, alpha, beta))
    dzd = [t.to(DEV).requires_grad_() for t in dz]
    z = R.sublayer_read(xd, ad)
    dx_read, dalpha = torch.autograd.grad(z, (xd, ad), [t.to(DEV) for t in gz])
    y = R.sublayer_write(xd, dzd, bd)
    dx_write, dbeta, *ddz = torch.autograd.grad(y, (xd, bd, *dzd), gy.to(DEV))
    return dict(z=torch.stack(z), y=y, dx_read=dx_read, dalpha=dalpha, dx_write=dx_write, dbeta=dbeta,
                ddz=torch.stack(ddz))


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
@pytest.mark.parametrize("case", ["tails_s4_e24", "tails_s16_e16", "vec_s4_e8"])
def test_golden_op_cases(R, case, tag):
    meta, t = load_golden(f"{case}_{tag}")
    dtype = getattr(torch, meta["dtype"])
    got = run_all(R, t["x"], t["alpha"], t["beta"], list(t["dz"].unbind(0)), list(t["gz"].unbind(0)), t["gy"])
    for key in ("z", "y", "dx_read", "dalpha", "dx_write", "dbeta", "ddz"):
        close(got[key], t[key], dtype, f"{case}_{tag}:{key}")
    assert torch.equal(got["dx_write"].cpu(), t["gy"])


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_golden_config1_seed0(R, tag):
    """The standalone-op configuration: batch 4, 256 tokens, n=4, width 768, seed 0, all outputs and gradients."""
    meta, t = load_golden(f"cfg1_{tag}")
    dtype = getattr(torch, meta["dtype"])
    stride = meta["sample_stride"]
    inp = regenerate_op_inputs(meta)
    assert torch.equal(inp["x"].flatten()[::stride], t["x_sample"])
    # single-event public API (autograd.Function path)
    xd = inp["x"].to(DEV).requires_grad_()
    ad = inp["alpha"][0].to(DEV).requires_grad_()
    bd = inp["beta"][0].to(DEV).requires_grad_()
    dzd = inp["dz"][0].to(DEV).requires_grad_()
    z = R.sihc_read(xd, ad)
    dx_read, dalpha = torch.autograd.grad(z, (xd, ad), inp["gz"][0].to(DEV))
    y = R.sihc_write(xd, dzd, bd)
    dx_write, dbeta, ddz = torch.autograd.grad(y, (xd, bd, dzd), inp["gy"].to(DEV))
    got = dict(z=z, y=y, dx_read=dx_read, dalpha=dalpha, dx_write=dx_write, dbeta=dbeta, ddz=ddz)
    for key, val in got.items():
        close(val.flatten()[::stride], t[key], dtype, f"cfg1_{tag}:{key}")
    # and the whole tensors against the oracle
    close(z, O.read(inp["x"], inp["alpha"][0]), dtype, "z full")
    close(y, O.write(inp["x"], [inp["dz"][0]], inp["beta"]), dtype, "y full")
    odx, oda = O.read_backward(inp["x"], [inp["gz"][0]], inp["alpha"], acc=torch.float64)
    oddz, odb = O.write_backward(inp["gy"], [inp["dz"][0]], inp["beta"], acc=torch.float64)
    close(dx_read, odx, dtype, "dx full")
    close(ddz, oddz[0], dtype, "ddz full")
    close(dalpha, oda[0].to(dtype), dtype, "dalpha full")
    close(dbeta, odb[0].to(dtype), dtype, "dbeta full")


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
@pytest.mark.parametrize("case", ["tri_a3", "tri_a23"])
def test_golden_triangular(R, case, tag):
    meta, t = load_golden(f"{case}_{tag}")
    dtype = getattr(torch, meta["dtype"])
    base = t["base"].to(DEV).requires_grad_()
    ups = [u.to(DEV).requires_grad_() for u in t["updates"].unbind(0)]
    gamma = t["gamma"].to(DEV).requires_grad_()
    out = R.sublayer_triangular(base, ups, gamma)
    dbase, dgamma, *ddz = torch.autograd.grad(out, (base, gamma, *ups), t["grad"].to(DEV))
    close(out, t["out"], dtype, "out")           # fused multiply-add here, mul then add there
    close(torch.stack(ddz), t["ddz"], dtype, "ddz")
    close(dgamma, t["dgamma"], t["gamma"].dtype, "dgamma")
    assert torch.equal(dbase.cpu(), t["grad"])


CASES = [
    # slots, batch, grid, channels, events, dtype, weights fp32?
    (2, 2, 5, 64, 1, torch.bfloat16, False),
    (2, 3, 3, 37, 3, torch.float32, False),
    (4, 2, 16, 768, 1, torch.bfloat16, True),
    (4, 5, 9, 1152, 2, torch.bfloat16, False),
    (4, 3, 7, 67, 24, torch.bfloat16, False),
    (4, 1, 16, 100, 12, torch.float32, False),
    (8, 2, 6, 128, 1, torch.bfloat16, False),
    (8, 2, 5, 36, 5, torch.float32, False),
    (16, 2, 4, 64, 1, torch.bfloat16, False),
    (16, 3, 11, 67, 16, torch.bfloat16, True),
    (16, 1, 16, 256, 8, torch.float32, False),
    (4, 9, 16, 768, 16, torch.bfloat16, False),
    (4, 1, 4, 3200, 3, torch.bfloat16, False),       # 400 channel vectors: wider than a 384-thread block
    (4, 2, 16, 1152, 24, torch.bfloat16, True),
]


@pytest.mark.parametrize("slots,b,g,c,events,dtype,wf32", CASES)
def test_random_shapes_vs_oracle(R, slots, b, g, c, events, dtype, wf32):
    torch.manual_seed(1000 + slots * 37 + c + events)
    kh, kw = O.cell_shape(slots)
    wdtype = torch.float32 if wf32 else dtype
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots)).to(wdtype)
    beta = (1.0 + 0.05 * torch.randn(events, c, slots)).to(wdtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * kh, g * kw, c).to(dtype)
    got = run_all(R, x, alpha, beta, dz, gz, gy)
    close(got["z"], torch.stack(O.multi_read(x, alpha)), dtype, "z")
    close(got["y"], O.write(x, dz, beta), dtype, "y")
    odx, oda = O.read_backward(x, gz, alpha, acc=torch.float64)
    oddz, odb = O.write_backward(gy, dz, beta, acc=torch.float64)
    close(got["dx_read"], odx, dtype, "dx_read")
    close(got["ddz"], torch.stack(oddz), dtype, "ddz")
    close(got["dalpha"], oda.to(wdtype), wdtype, "dalpha")
    close(got["dbeta"], odb.to(wdtype), wdtype, "dbeta")
    assert got["dalpha"].dtype == wdtype and got["dbeta"].dtype == wdtype


def test_packed_layout_contract_and_unused_reads(R):
    # research/tests/test_sublayer_kernels.py:111-123
    x = torch.randn(1, 16, 16, 37, device=DEV, requires_grad=True)
    a = torch.randn(16, 37, 16, device=DEV, requires_grad=True)
    with pytest.raises(ValueError, match="contiguous|packed"):
        R.sublayer_read(x.transpose(1, 2), a)
    base = R.sublayer_read(x, a)
    padded = torch.randn(2, 18, 37, device=DEV)
    bad = padded[:, 2:]
    with pytest.raises(ValueError, match="contiguous|packed"):
        R.sublayer_triangular(bad, [bad], torch.ones(1, 37, device=DEV))
    base[0].sum().backward()
    assert torch.count_nonzero(a.grad[1:]) == 0
    assert torch.count_nonzero(a.grad[0]) > 0
    xo, ao = x.detach().cpu(), a.detach().cpu()
    odx, oda = O.read_backward(xo, [torch.ones(1, 16, 37)] + [None] * 15, ao)
    close(x.grad, odx, torch.float32, "dx with unused outputs")
    close(a.grad, oda, torch.float32, "dalpha with unused outputs")


def test_error_contract(R):
    x = torch.randn(2, 8, 8, 16, device=DEV)
    a = torch.randn(4, 16, 4, device=DEV)
    with pytest.raises(ValueError):
        R.sublayer_read(x, a[:, :8].contiguous())                      # channel mismatch
    with pytest.raises(ValueError):
        R.sublayer_read(x, torch.randn(4, 16, 3, device=DEV))          # unsupported slot count
    with pytest.raises(ValueError):
        R.sublayer_read(x, torch.randn(25, 16, 4, device=DEV))         # too many events
    with pytest.raises(ValueError):
        R.sublayer_read(x.half(), a.half())                            # unsupported dtype
    with pytest.raises(ValueError):
        R.sublayer_read(x.cpu(), a.cpu())                              # not CUDA: no CPU fallback
    with pytest.raises(ValueError):
        R.sublayer_write(x, [torch.randn(2, 16, 16, device=DEV)] * 3, a)   # one update per event
    with pytest.raises(ValueError):
        R.sublayer_write(x, [torch.randn(2, 15, 16, device=DEV)] * 4, a)   # wrong token count
    with pytest.raises(ValueError):
        R.sublayer_triangular(torch.randn(2, 16, 16, device=DEV), [], torch.ones(0, 16, device=DEV))
    with pytest.raises(ValueError):
        R.blockwise_read(x, a)                                         # block-wise needs 8 or 12 events


def test_weight_gradients_are_deterministic(R):
    torch.manual_seed(5)
    x = torch.randn(8, 32, 32, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    a = (0.25 + 0.02 * torch.randn(1, 256, 4, device=DEV)).to(torch.bfloat16).requires_grad_()
    g = torch.randn(8, 256, 256, device=DEV, dtype=torch.bfloat16)
    runs = []
    for _ in range(3):
        z = R.sublayer_read(x, a)
        runs.append(torch.autograd.grad(z, (x, a), [g]))
    for dx, da in runs[1:]:
        assert torch.equal(dx, runs[0][0]) and torch.equal(da, runs[0][1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("events,slots", [(16, 4), (24, 4), (8, 16)])
def test_stage_recurrence_matches_literal_carrier(R, events, slots, dtype):
    """read -> triangular -> write staged == literal dense recurrence, all gradients
    (research/tests/test_sublayer_kernels.py:76-108; oracle in place of the CUDA einsum)."""
    torch.manual_seed(92)
    k = int(slots ** 0.5)
    x = torch.randn(2, 4 * k, 4 * k, 37).to(dtype)
    alpha = (torch.randn(events, 37, slots) * 0.07).to(dtype)
    beta = (torch.randn(events, 37, slots) * 0.07).to(dtype)
    xd, ad, bd = (t.to(DEV).requires_grad_() for t in (x, alpha, beta))
    base = R.sublayer_read(xd, ad)
    gamma = (ad[:, None] * bd[None, :]).sum(-1)
    updates = []
    for i in range(events):
        z = base[i] if i == 0 else R.sublayer_triangular(base[i], updates, gamma[i, :i].contiguous())
        updates.append((0.05 * z.tanh()).contiguous())
    out = R.sublayer_write(xd, updates, bd)
    xr, ar, br = (t.clone().requires_grad_() for t in (x, alpha, beta))
    ref = O.literal_stage(xr, ar, br, [lambda z: 0.05 * z.tanh()] * events)
    upstream = (torch.randn(out.shape) * 0.1).to(dtype)
    ga = torch.autograd.grad(out, (xd, ad, bd), upstream.to(DEV))
    gr = torch.autograd.grad(ref, (xr, ar, br), upstream)
    atol, rtol = (2e-4, 2e-4) if dtype == torch.float32 else (0.025, 0.03)
    torch.testing.assert_close(out.cpu(), ref, atol=atol, rtol=rtol)
    for a, b in zip(ga, gr):
        torch.testing.assert_close(a.cpu(), b, atol=atol, rtol=rtol)
        rel = (a.cpu().float() - b.float()).norm() / b.float().norm().clamp_min(1e-8)
        assert rel < (0.035 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("active", [1, 3, 8, 23, 24])
def test_triangular_tails_and_mixed_gamma(R, dtype, active):
    torch.manual_seed(583)
    base = torch.randn(3, 49, 67).to(dtype)
    ups = [torch.randn(3, 49, 67).to(dtype) for _ in range(active)]
    gamma = torch.randn(active, 67) * 0.05                     # fp32 gamma with a bf16 workspace is allowed
    grad = torch.randn(3, 49, 67).to(dtype)
    bd = base.to(DEV).requires_grad_()
    ud = [u.to(DEV).requires_grad_() for u in ups]
    gd = gamma.to(DEV).requires_grad_()
    out = R.sublayer_triangular(bd, ud, gd)
    dbase, dgamma, *ddz = torch.autograd.grad(out, (bd, gd, *ud), grad.to(DEV))
    close(out, O.triangular(base, ups, gamma), dtype, "out")
    oddz, odg = O.triangular_backward(grad, ups, gamma, acc=torch.float64)
    close(torch.stack(ddz), torch.stack(oddz), dtype, "ddz")
    close(dgamma, odg.float(), torch.float32, "dgamma")
    assert torch.equal(dbase.cpu(), grad)


def test_large_size_properties(R):
    """Size-independent properties at a size the oracle would take minutes on:
    adjointness <read(x), g> == <x, read^T(g)>, linearity, and write(x, dz, 0*beta) == x."""
    torch.manual_seed(11)
    b, g, c, s = 512, 16, 768, 4                                 # M = 2^17 tokens, X = 805 MB in bf16
    dtype = torch.bfloat16
    x = torch.randn(b, 2 * g, 2 * g, c, device=DEV, dtype=dtype)
    alpha = (0.25 + 0.02 * torch.randn(1, c, s, device=DEV)).to(dtype)
    gz = torch.randn(b, g * g, c, device=DEV, dtype=dtype)
    z = R.sublayer_read(x, alpha)[0]
    dx, dalpha = R.ops._read_backward_op(x, [gz], alpha, True, True)
    lhs = (z.double() * gz.double()).sum()
    rhs = (x.double() * dx.double()).sum()
    assert abs(lhs - rhs) / abs(lhs) < 5e-3                      # bf16 rounding of z and dx
    # dalpha[c,s] = sum_m x*g  -> checks against a torch reduction on the GPU in fp64 chunks
    cells = x.view(b * g, 2, g, 2, c)
    ref = torch.zeros(c, s, dtype=torch.float64, device=DEV)
    gv = gz.view(b * g, 1, g, 1, c)
    for lo in range(0, b * g, 1024):
        prod = cells[lo:lo + 1024].double() * gv[lo:lo + 1024].double()
        ref += prod.sum((0, 2)).permute(2, 0, 1).reshape(c, s)
    rel = (dalpha[0].double() - ref).norm() / ref.norm()
    assert rel < 5e-3, float(rel)                                # result is rounded to bf16
    zero_beta = torch.zeros(1, c, s, device=DEV, dtype=dtype)
    y = R.sublayer_write(x, [gz], zero_beta)
    assert torch.equal(y, x)
    # linearity of the write in dz with beta = 1: write(x, dz, 1) - x == dz broadcast to every slot
    ones = torch.ones(1, c, s, device=DEV, dtype=dtype)
    y0 = R.ops._write_impl(x, [gz], ones, False)
    assert torch.equal(y0.view(b * g, 2, g, 2, c), gz.view(b * g, 1, g, 1, c).expand(b * g, 2, g, 2, c))


def test_full_size_integer_inputs_are_bit_exact(R):
    """The bench workload's full size (2^20 tokens, 4 slots, width 768, bf16 carrier, fp32 weights) with
    small-integer inputs.  Every product and every partial sum is then an integer below 2^24 (weight
    gradients: |x*g| <= 4 over 2^20 tokens) resp. 2^8 (bf16 outputs), so fp32 accumulation is exact in any
    order and every kernel must reproduce integer arithmetic bit for bit: forward values, both adjoint maps,
    the token-reduced weight gradients, the fused write+read step and the triangular pair."""
    torch.manual_seed(5)
    b, g, c, s = 4096, 16, 768, 4
    dtype = torch.bfloat16

    def ints(*shape, dt=dtype):
        return torch.randint(-2, 3, shape, device=DEV, dtype=torch.int8).to(dt)

    x = ints(b, 2 * g, 2 * g, c)                                 # 6.4 GB
    gz = ints(b, g * g, c)
    alpha, beta = ints(1, c, s, dt=torch.float32), ints(1, c, s, dt=torch.float32)
    rows, step = b * g, 4096
    slot_map = lambda w: w[0].T.reshape(1, 2, 1, 2, c)           # [C,S] -> broadcast over [rows, uy, wx, ux, C]
    cells = lambda t: t.view(rows, 2, g, 2, c)
    tokens = lambda t: t.view(rows, 1, g, 1, c)

    z = R.sublayer_read(x, alpha)[0]
    dx, dalpha = R.ops._read_backward_op(x, [gz], alpha, True, True)
    y = R.sublayer_write(x, [gz], beta)
    ddz, dbeta = R.ops._write_backward_op(x, [gz], beta, True, True)
    y2, z2 = R.sihc_write_read(x, gz, beta[0].contiguous(), alpha[0].contiguous())
    assert dalpha.dtype == torch.float32 and dbeta.dtype == torch.float32
    wsum = torch.zeros(2, 2, c, dtype=torch.float64, device=DEV)
    for lo in range(0, rows, step):
        sl = slice(lo, lo + step)
        xc, gt = cells(x)[sl].float(), tokens(gz)[sl].float()
        assert torch.equal(z.view(rows, g, c)[sl], (xc * slot_map(alpha)).sum((1, 3)).to(dtype)), lo
        assert torch.equal(cells(dx)[sl], (gt * slot_map(alpha)).to(dtype).expand_as(xc)), lo
        yc = xc + gt * slot_map(beta)
        assert torch.equal(cells(y)[sl], yc.to(dtype)), lo
        assert torch.equal(ddz[0].view(rows, g, c)[sl], (xc * slot_map(beta)).sum((1, 3)).to(dtype)), lo
        assert torch.equal(cells(y2)[sl], yc.to(dtype)), lo
        assert torch.equal(z2.view(rows, g, c)[sl], (yc * slot_map(alpha)).sum((1, 3)).to(dtype)), lo
        wsum += (xc * gt).double().sum((0, 2))
    expected = wsum.reshape(s, c).T.float()                       # sum_m x[m,s,c] * g[m,c]
    assert float(expected.abs().max()) < 2 ** 24
    assert torch.equal(dalpha[0], expected)
    assert torch.equal(dbeta[0], expected)                        # same sum: carrier gradient = x, update = gz
    del dx, y, y2, z2, ddz

    ups = [ints(b, g * g, c) for _ in range(3)]
    gamma = ints(3, c, dt=torch.float32)
    out = R.sublayer_triangular(z, ups, gamma)
    dd, dgamma = R.ops._tri_backward_op(gz, ups, gamma, True, True)
    acc = z.float()
    for l, u in enumerate(ups):
        acc += u.float() * gamma[l]
        assert torch.equal(dd[l], (gz.float() * gamma[l]).to(dtype)), l
        assert torch.equal(dgamma[l], (gz.double() * u.double()).sum((0, 1)).float()), l
    assert torch.equal(out, acc.to(dtype))


def test_c_abi_direct_calls_and_status_codes(R):
    """Raw ctypes calls: status codes for bad arguments, no torch op layer in between."""
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    x = torch.randn(1, 4, 4, 8, device=DEV)
    a = torch.full((1, 8, 4), 0.25, device=DEV)
    out = torch.empty(1, 4, 8, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(), a.data_ptr(), _lib.ptr_array([out.data_ptr()]), 1, 1, 2, 2, 2, 8)
    assert lib.sihc_read_fwd(*args, _lib.F32, _lib.F32, s) == 0
    torch.cuda.synchronize()
    assert torch.allclose(out.cpu(), O.read(x.cpu(), a[0].cpu()), atol=1e-6)
    assert lib.sihc_read_fwd(None, a.data_ptr(), _lib.ptr_array([out.data_ptr()]), 1, 1, 2, 2, 2, 8, 0, 0, s) == -1
    assert lib.sihc_read_fwd(*args, 7, 0, s) == -2
    assert lib.sihc_read_fwd(x.data_ptr(), a.data_ptr(), _lib.ptr_array([out.data_ptr()]), 0, 1, 2, 2, 2, 8, 0, 0, s) == -3
    assert lib.sihc_read_fwd(x.data_ptr(), a.data_ptr(), _lib.ptr_array([out.data_ptr()]), 1, 1, 2, 3, 3, 8, 0, 0, s) == -4
    assert lib.sihc_read_fwd(x.data_ptr(), a.data_ptr(), _lib.ptr_array([out.data_ptr()]), 1, 0, 2, 2, 2, 8, 0, 0, s) == -5
    da = torch.empty(1, 8, 4, device=DEV)
    dx = torch.empty_like(x)
    assert lib.sihc_read_bwd(x.data_ptr(), _lib.ptr_array([out.data_ptr()]), a.data_ptr(), dx.data_ptr(), da.data_ptr(),
                             None, 0, 1, 1, 2, 2, 2, 8, 0, 0, s) == -6
    assert b"workspace" in lib.sihc_status_string(-6)
    before = _lib.launch_count()
    assert lib.sihc_read_fwd(*args, _lib.F32, _lib.F32, s) == 0
    assert _lib.launch_count() == before + 1
    torch.cuda.synchronize()


@pytest.mark.parametrize("stages", [0, 3, 4, 8])
@pytest.mark.parametrize("slots,dtype", [(4, torch.bfloat16), (8, torch.bfloat16), (2, torch.float32), (16, torch.bfloat16)])
def test_single_event_adjoints_register_and_ring_variants(R, stages, slots, dtype):
    """The fused single-event adjoints exist in two forms (loads staged in registers, or through a
    shared-memory async-copy ring); both must give the same answer, including ragged token counts."""
    from residual_stream_burden_b200 import _lib
    torch.manual_seed(77 + slots)
    kh, kw = O.cell_shape(slots)
    b, g, c = 5, 7, 128                                   # 245 tokens: not a multiple of any tile
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(1, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype)]
    gz = [torch.randn(b, g * g, c).to(dtype)]
    gy = torch.randn(b, g * kh, g * kw, c).to(dtype)
    _lib.tune("ring_stages", stages)
    try:
        got = run_all(R, x, alpha, alpha, dz, gz, gy)
    finally:
        _lib.tune("ring_default", 0)
    odx, oda = O.read_backward(x, gz, alpha, acc=torch.float64)
    oddz, odb = O.write_backward(gy, dz, alpha, acc=torch.float64)
    close(got["dx_read"], odx, dtype, "dx_read")
    close(got["ddz"], torch.stack(oddz), dtype, "ddz")
    close(got["dalpha"], oda.to(dtype), dtype, "dalpha")
    close(got["dbeta"], odb.to(dtype), dtype, "dbeta")


@pytest.mark.parametrize("tiled", [0, 1])
@pytest.mark.parametrize("slots,b,g,c,events,dtype", [(4, 3, 7, 768, 24, torch.bfloat16), (4, 2, 5, 1152, 16, torch.bfloat16),
                                                      (4, 2, 6, 64, 5, torch.float32), (2, 3, 5, 128, 8, torch.bfloat16),
                                                      (8, 2, 4, 256, 12, torch.bfloat16), (8, 2, 4, 256, 24, torch.bfloat16), (16, 2, 3, 64, 12, torch.bfloat16),
                                                      (4, 1, 3, 40, 3, torch.bfloat16)])
def test_stage_weight_gradient_tiled_and_per_thread_forms(R, tiled, slots, b, g, c, events, dtype):
    """The multi-event weight gradient exists as a block-tiled kernel (carrier tile shared through shared memory)
    and as a per-thread kernel; both must match the fp64 oracle, with unused read outputs left at exactly zero."""
    from residual_stream_burden_b200 import _lib
    torch.manual_seed(812 + slots + events)
    kh, kw = O.cell_shape(slots)
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * kh, g * kw, c).to(dtype)
    _lib.tune("wgrad_tiled", tiled)
    try:
        got = run_all(R, x, alpha, alpha, dz, gz, gy)
        holes = [t.to(DEV) if i % 3 else None for i, t in enumerate(gz)]
        _, da_holes = R.ops._read_backward_op(x.to(DEV), holes, alpha.to(DEV), False, True)
        torch.cuda.synchronize()
    finally:
        _lib.tune("wgrad_tiled", -1)
    _, oda = O.read_backward(x, gz, alpha, acc=torch.float64)
    _, odb = O.write_backward(gy, dz, alpha, acc=torch.float64)
    close(got["dalpha"], oda.to(dtype), dtype, "dalpha")
    close(got["dbeta"], odb.to(dtype), dtype, "dbeta")
    for i in range(events):
        if i % 3 == 0:
            assert not da_holes[i].any()
        else:
            close(da_holes[i], oda[i].to(dtype), dtype, f"dalpha[{i}] with unused outputs")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b,g,c,events", [(3, 7, 768, 24), (2, 5, 1152, 16), (2, 6, 72, 20), (1, 16, 776, 18), (5, 3, 8, 24),
                                          (2, 6, 1152, 12), (3, 5, 768, 8), (2, 4, 64, 5), (2, 4, 72, 3)])
def test_stage_adjoints_in_one_pass_and_as_two_kernels(R, b, g, c, events, dtype):
    """With four slots and enough events (8 for the write, 12 for the read) both adjoints of the stage read (dx, dalpha) and of the stage write (ddz, dbeta)
    come from one pass over the carrier and the event tensors (the `"one_pass_min_events"` knob lowers that event count: the
    kernels themselves take any); `"one_pass_adjoints" = 0` restores the two-kernel forms.  Both
    must match the fp64 oracle; the write side is the same arithmetic in the same order, hence bit-identical; a read
    output nobody used (no gradient) contributes nothing to dx and leaves its dalpha rows exactly zero in both."""
    from residual_stream_burden_b200 import _lib
    torch.manual_seed(4100 + events + c)
    slots = 4
    x = torch.randn(b, g * 2, g * 2, c).to(dtype)
    w = (0.25 + 0.05 * torch.randn(events, c, slots)).to(dtype)
    ev = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    holes = [t if i % 5 != 2 else None for i, t in enumerate(ev)]
    xd, wd = x.to(DEV), w.to(DEV)
    evd = [t.to(DEV) for t in ev]
    holesd = [t.to(DEV) if t is not None else None for t in holes]
    got = {}
    for form, knob in (("one pass", -1), ("two kernels", 0)):
        _lib.tune("one_pass_adjoints", knob)
        _lib.tune("one_pass_min_events", 2)
        try:
            n0 = _lib.lib.sihc_launch_count()
            dx, da = R.ops._read_backward_op(xd, holesd, wd, True, True)
            n1 = _lib.lib.sihc_launch_count()
            ddz, db = R.ops._write_backward_op(xd, evd, wd, True, True)
            n2 = _lib.lib.sihc_launch_count()
            torch.cuda.synchronize()
        finally:
            _lib.tune("one_pass_adjoints", -1)
            _lib.tune("one_pass_min_events", 0)
        got[form] = (dx, da, torch.stack(ddz), db)
        if form == "one pass":
            assert (n1 - n0, n2 - n1) == (2, 2), (n1 - n0, n2 - n1)        # the pass and the finishing kernel
        else:
            assert n1 - n0 >= 3 and n2 - n1 >= 3, (n1 - n0, n2 - n1)
    odx, oda = O.read_backward(x, holes, w, acc=torch.float64)
    oddz, odb = O.write_backward(x, ev, w, acc=torch.float64)
    for form, (dx, da, ddz, db) in got.items():
        close(dx, odx, dtype, f"dx ({form})")
        close(da, oda.to(dtype), dtype, f"dalpha ({form})")
        close(ddz, torch.stack(oddz), dtype, f"ddz ({form})")
        close(db, odb.to(dtype), dtype, f"dbeta ({form})")
        for i, t in enumerate(holes):
            if t is None:
                assert not da[i].any(), (form, i)
    assert torch.equal(got["one pass"][2], got["two kernels"][2])
    if events >= 16:        # below, the two-kernel form takes the per-thread weight gradient: another summation order
        assert torch.equal(got["one pass"][3], got["two kernels"][3])


@pytest.mark.parametrize("active,c,dtype,gamma_fp32", [(3, 64, torch.bfloat16, False), (5, 768, torch.bfloat16, True),
                                                       (8, 128, torch.float32, True), (12, 1152, torch.bfloat16, False),
                                                       (23, 768, torch.bfloat16, False), (23, 64, torch.bfloat16, True)])
def test_triangular_backward_event_slices_and_single_outputs(R, active, c, dtype, gamma_fp32):
    """The triangular backward must match the oracle for every chunking of the events (1, 2 or 3 slices of at
    most 8), both gamma dtypes and a token count that is not a multiple of any tile; asking for only one of
    the two outputs must give the same bits as asking for both."""
    torch.manual_seed(291 + active)
    b, n = 3, 83                                          # 249 tokens
    ups = [torch.randn(b, n, c).to(dtype) for _ in range(active)]
    gamma = (torch.randn(active, c) * 0.05).to(torch.float32 if gamma_fp32 else dtype)
    grad = torch.randn(b, n, c).to(dtype)
    ud, gd, gr = [u.to(DEV) for u in ups], gamma.to(DEV), grad.to(DEV)
    ddz, dgamma = R.ops._tri_backward_op(gr, ud, gd, True, True)
    ddz_only, _ = R.ops._tri_backward_op(gr, ud, gd, True, False)
    _, dgamma_only = R.ops._tri_backward_op(gr, ud, gd, False, True)
    oddz, odg = O.triangular_backward(grad, ups, gamma, acc=torch.float64)
    close(torch.stack(ddz), torch.stack(oddz), dtype, "ddz")
    close(dgamma, odg.to(gamma.dtype), gamma.dtype, "dgamma")
    assert all(torch.equal(a, b_) for a, b_ in zip(ddz, ddz_only))
    assert torch.equal(dgamma, dgamma_only)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("slots,b,g,c", [(4, 3, 7, 67), (4, 4, 16, 768), (2, 2, 5, 64), (8, 2, 6, 128), (16, 2, 4, 64)])
def test_fused_write_then_read_step_is_the_unfused_pair(R, slots, b, g, c, dtype):
    """sihc_write_read == write_torch followed by read_torch, including the rounding of the carrier
    between the two (so bf16 results are bit-identical to the unfused oracle pair)."""
    torch.manual_seed(40 + slots + c)
    kh, kw = O.cell_shape(slots)
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    dz = torch.randn(b, g * g, c).to(dtype)
    beta = (1.0 + 0.05 * torch.randn(c, slots)).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(c, slots)).to(dtype)
    y, z = R.sihc_write_read(x.to(DEV), dz.to(DEV), beta.to(DEV), alpha.to(DEV))
    oy = O.write(x, [dz], [beta])
    oz = O.read(oy, alpha)
    close(y, oy, dtype, "carrier")
    close(z, oz, dtype, "next read")
    # and it agrees with this library's own separate write + read
    y2 = R.sihc_write(x.to(DEV), dz.to(DEV), beta.to(DEV))
    z2 = R.sihc_read(y2, alpha.to(DEV))
    assert torch.equal(y, y2)
    close(z, z2, dtype, "fused vs separate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("slots,b,g,c", [(4, 4, 16, 768), (4, 3, 7, 67), (16, 2, 4, 64)])
def test_fused_write_then_read_in_place_through_the_c_abi(slots, b, g, c, dtype):
    """`y` may be `x` in sihc_write_read_fwd: the carrier is updated where it lies and the result is
    bit-identical to the out-of-place call (vector and scalar paths)."""
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    torch.manual_seed(77 + slots + c)
    kh, kw = O.cell_shape(slots)
    x = torch.randn(b, g * kh, g * kw, c, device=DEV).to(dtype)
    dz = torch.randn(b, g * g, c, device=DEV).to(dtype)
    beta = (1.0 + 0.05 * torch.randn(c, slots, device=DEV)).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(c, slots, device=DEV)).to(dtype)
    stream = torch.cuda.current_stream().cuda_stream

    def call(src, dst, z):
        rc = lib.sihc_write_read_fwd(src.data_ptr(), dz.data_ptr(), beta.data_ptr(), alpha.data_ptr(), dst.data_ptr(),
                                     z.data_ptr(), b, g, kh, kw, c, code, code, stream)
        assert rc == 0, lib.sihc_status_string(rc)

    y_out, z_out = torch.empty_like(x), torch.empty_like(dz)
    call(x, y_out, z_out)
    carrier, z_in = x.clone(), torch.empty_like(dz)
    call(carrier, carrier, z_in)
    torch.cuda.synchronize()
    assert torch.equal(carrier, y_out)
    assert torch.equal(z_in, z_out)
    oy = O.write(x.cpu(), [dz.cpu()], [beta.cpu()])
    close(carrier, oy, dtype, "in-place carrier")
    close(z_in, O.read(oy, alpha.cpu()), dtype, "in-place next read")


@pytest.mark.parametrize("slots,c,events", [(4, 4104, 1), (8, 2056, 1), (4, 4104, 3), (2, 4100, 2)])
def test_channel_counts_wider_than_one_block(R, slots, c, events):
    """More channel vectors than a block has lanes: the channel dimension is tiled over blockIdx.y,
    with a partly filled last tile (and, for 4100 channels in bf16, the scalar path)."""
    dtype = torch.bfloat16
    torch.manual_seed(c + slots)
    kh, kw = O.cell_shape(slots)
    b, g = 2, 5
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots)).to(dtype)
    beta = (1.0 + 0.05 * torch.randn(events, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * kh, g * kw, c).to(dtype)
    got = run_all(R, x, alpha, beta, dz, gz, gy)
    close(got["z"], torch.stack(O.multi_read(x, alpha)), dtype, "z")
    close(got["y"], O.write(x, dz, beta), dtype, "y")
    odx, oda = O.read_backward(x, gz, alpha, acc=torch.float64)
    oddz, odb = O.write_backward(gy, dz, beta, acc=torch.float64)
    close(got["dx_read"], odx, dtype, "dx_read")
    close(got["ddz"], torch.stack(oddz), dtype, "ddz")
    close(got["dalpha"], oda.to(dtype), dtype, "dalpha")
    close(got["dbeta"], odb.to(dtype), dtype, "dbeta")
    base = torch.randn(b, g * g, c).to(dtype)
    gamma = torch.randn(events, c) * 0.05
    out = R.sublayer_triangular(base.to(DEV), [t.to(DEV) for t in dz], gamma.to(DEV))
    close(out, O.triangular(base, dz, gamma), dtype, "triangular")
    y2, z2 = R.sihc_write_read(x.to(DEV), dz[0].to(DEV), beta[0].to(DEV), alpha[0].to(DEV))
    close(y2, O.write(x, [dz[0]], [beta[0]]), dtype, "write_read y")
    close(z2, O.read(O.write(x, [dz[0]], [beta[0]]), alpha[0]), dtype, "write_read z")


@pytest.mark.parametrize("staged", [0, 1])
@pytest.mark.parametrize("slots,events,c,dtype,wf32", [(4, 24, 768, torch.bfloat16, False), (16, 12, 256, torch.bfloat16, True),
                                                       (8, 5, 1152, torch.bfloat16, False), (2, 3, 64, torch.float32, False)])
def test_stage_read_write_coefficient_staging_variants(R, staged, slots, events, c, dtype, wf32):
    """The stage read and write exist with their coefficients re-read from L1 or staged (transposed) in
    shared memory, including channel counts split over several blocks; both against the oracle."""
    from residual_stream_burden_b200 import _lib
    torch.manual_seed(900 + slots + events)
    kh, kw = O.cell_shape(slots)
    wdtype = torch.float32 if wf32 else dtype
    b, g = 2, 7
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots)).to(wdtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    _lib.tune("stage_smem", staged)
    try:
        z = R.sublayer_read(x.to(DEV), alpha.to(DEV))
        y = R.sublayer_write(x.to(DEV), [t.to(DEV) for t in dz], alpha.to(DEV))
    finally:
        _lib.tune("stage_smem_default", 0)
    close(torch.stack(z), torch.stack(O.multi_read(x, alpha)), dtype, "z")
    close(y, O.write(x, dz, alpha), dtype, "y")


def _misaligned(t, dev=DEV):
    """Same values, packed, but starting one element past a 16-byte boundary."""
    flat = torch.empty(t.numel() + 1, dtype=t.dtype, device=dev)
    view = flat[1:].view(t.shape)
    view.copy_(t)
    assert view.is_contiguous() and view.data_ptr() % 16 != 0
    return view


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("events", [1, 3])
def test_pointers_off_the_16_byte_grid_take_the_scalar_path(R, dtype, events):
    """Packed tensors whose storage does not start on a 16-byte boundary are legal inputs; the library
    must fall back to element-wise accesses rather than fault or mis-read."""
    torch.manual_seed(314)
    slots, b, g, c = 4, 2, 5, 64
    x = torch.randn(b, 2 * g, 2 * g, c).to(dtype)
    alpha = (0.25 + 0.05 * torch.randn(events, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, 2 * g, 2 * g, c).to(dtype)
    xd, ad = _misaligned(x).requires_grad_(), _misaligned(alpha).requires_grad_()
    dzd = [_misaligned(t).requires_grad_() for t in dz]
    z = R.sublayer_read(xd, ad)
    dx, dalpha = torch.autograd.grad(z, (xd, ad), [_misaligned(t) for t in gz])
    y = R.sublayer_write(xd, dzd, ad)
    _, dbeta, *ddz = torch.autograd.grad(y, (xd, ad, *dzd), _misaligned(gy))
    close(torch.stack(z), torch.stack(O.multi_read(x, alpha)), dtype, "z")
    close(y, O.write(x, dz, alpha), dtype, "y")
    odx, oda = O.read_backward(x, gz, alpha, acc=torch.float64)
    oddz, odb = O.write_backward(gy, dz, alpha, acc=torch.float64)
    close(dx, odx, dtype, "dx")
    close(dalpha, oda.to(dtype), dtype, "dalpha")
    close(torch.stack(ddz), torch.stack(oddz), dtype, "ddz")
    close(dbeta, odb.to(dtype), dtype, "dbeta")
    base = _misaligned(torch.randn(b, g * g, c).to(dtype))
    gamma = _misaligned((torch.randn(events, c) * 0.05).to(dtype))
    out = R.sublayer_triangular(base, dzd, gamma)
    close(out, O.triangular(base.cpu(), dz, gamma.cpu()), dtype, "triangular")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("events,tokens,c", [(24, 1030, 768), (16, 515, 1152), (12, 300, 72), (8, 257, 64), (5, 99, 40),
                                             (2, 33, 16), (24, 70, 37), (7, 50, 36), (1, 10, 16)])
def test_stage_coefficient_gradient_in_one_pass(events, tokens, c, dtype):
    """sihc_tri_dgamma: dgamma[i,j,c] = sum_m g_i * dz_j for j < i, zero elsewhere, against an fp64 sum; vector
    path, channel tails, the scalar path (37 and, in bf16, 36 channels), an unused read (NULL gradient) and the
    one-event stage.  Deterministic: two calls give identical bits."""
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
    torch.manual_seed(events * 1000 + c)
    g = [torch.randn(1, tokens, c, device=DEV).to(dtype) for _ in range(events)]
    dz = [torch.randn(1, tokens, c, device=DEV).to(dtype) for _ in range(events)]
    unused = 2 if events > 3 else None
    ptr_g = _lib.ptr_array([None if i == unused else t.data_ptr() for i, t in enumerate(g)])
    ptr_dz = _lib.ptr_array([t.data_ptr() for t in dz])
    nbytes = lib.sihc_tri_dgamma_workspace_bytes(events, tokens, c, code)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):
        out = torch.full((events, events, c), float("nan"), device=DEV)
        rc = lib.sihc_tri_dgamma(ptr_g, ptr_dz, out.data_ptr(), ws.data_ptr(), ws.numel(), events, tokens, c, code, stream)
        assert rc == 0, lib.sihc_status_string(rc)
        outs.append(out)
        ws.fill_(0xFF)                                   # the scratch needs no particular contents
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    G = torch.stack([t[0].double() for t in g])          # [E, M, C]
    D = torch.stack([t[0].double() for t in dz])
    want = torch.einsum("imc,jmc->ijc", G, D)
    mask = torch.tril(torch.ones(events, events, device=DEV), diagonal=-1)
    if unused is not None:
        mask[unused] = 0
    want = want * mask[:, :, None]
    got = outs[0].double()
    assert torch.count_nonzero(got * (1 - mask[:, :, None])) == 0          # exactly zero outside the lower triangle
    if events > 1:
        rel = (got - want).norm() / want.norm()
        assert rel <= 1e-5, float(rel)                     # fp32 accumulation of exact products
        torch.testing.assert_close(got, want, atol=2e-4 * tokens ** 0.5, rtol=2e-4)


@pytest.fixture(params=[-1, 0], ids=["ring", "register-staged"])
def adjoint_form(request):
    """Both forms of the fused adjoint: loads staged through the async-copy ring (default) or through registers."""
    from residual_stream_burden_b200 import _lib
    _lib.tune("ring_stages", request.param)
    yield request.param
    _lib.tune("ring_stages", -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("slots,b,g,c,wf32", [(4, 4, 16, 768, False), (4, 3, 7, 67, False), (2, 2, 5, 64, False),
                                              (8, 2, 6, 128, False), (16, 2, 4, 64, False), (4, 2, 6, 1152, True)])
def test_fused_adjoint_of_the_write_then_read_step(R, adjoint_form, slots, b, g, c, wf32, dtype):
    """Every gradient of sihc_write_read (carrier, update, beta, alpha_next) from the fused 3S+3 pass, against fp64
    autograd through the oracle's write followed by read, and against this library's separate operators."""
    if wf32 and dtype == torch.float32:
        pytest.skip("fp32 weights over fp32 tensors is the plain fp32 case")
    torch.manual_seed(61 + slots + c)
    kh, kw = O.cell_shape(slots)
    wdt = torch.float32 if wf32 else dtype
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    dz = torch.randn(b, g * g, c).to(dtype)
    beta = (1.0 + 0.05 * torch.randn(c, slots)).to(wdt)
    alpha = (1.0 / slots + 0.05 * torch.randn(c, slots)).to(wdt)
    gy = torch.randn_like(x)
    gz = torch.randn_like(dz)
    dev = [t.to(DEV).requires_grad_() for t in (x, dz, beta, alpha)]
    y, z = R.sihc_write_read(*dev)
    got = torch.autograd.grad((y, z), dev, (gy.to(DEV), gz.to(DEV)))
    ref = [t.double().requires_grad_() for t in (x, dz, beta, alpha)]

    def stored(t):          # the unfused path stores the carrier in `dtype` before the read sees it; the rounding is
        return t + (t.to(dtype).double() - t).detach()      # applied to the value only (gradients pass unrounded)

    oy = stored(O.write(ref[0], [ref[1]], [ref[2]], acc=torch.float64))
    oz = O.read(oy, ref[3], acc=torch.float64)
    want = torch.autograd.grad((oy, oz), ref, (gy.double(), gz.double()))
    for name, a, w in zip(("dx", "ddz", "dbeta", "dalpha_next"), got, want):
        close(a, w.to(a.dtype), dtype, name)
    # only one incoming gradient: the other side is treated as zero
    only_y = torch.autograd.grad(R.sihc_write_read(*dev)[0], dev[:3], gy.to(DEV))
    want_y = torch.autograd.grad(O.write(ref[0], [ref[1]], [ref[2]], acc=torch.float64), ref[:3], gy.double())
    assert torch.equal(only_y[0], gy.to(DEV))
    close(only_y[1], want_y[1].to(dtype), dtype, "ddz (carrier gradient only)")
    close(only_y[2], want_y[2].to(wdt), dtype, "dbeta (carrier gradient only)")
    only_z = torch.autograd.grad(R.sihc_write_read(*dev)[1], dev, gz.to(DEV))
    oy2 = stored(O.write(ref[0], [ref[1]], [ref[2]], acc=torch.float64))
    want_z = torch.autograd.grad(O.read(oy2, ref[3], acc=torch.float64), ref, gz.double())
    for name, a, w in zip(("dx", "ddz", "dbeta", "dalpha_next"), only_z, want_z):
        close(a, w.to(a.dtype), dtype, name + " (read gradient only)")
