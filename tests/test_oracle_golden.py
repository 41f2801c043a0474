"""Pin the CPU oracle against fixtures produced by the reference itself.

The fixtures under ``tests/golden`` come from ``tests/golden/make_golden.py``,
which runs the reference's unfused PyTorch path.  The oracle restates the same
arithmetic in the same order, so forward values are compared bit-exactly and
gradients (explicit adjoints here, autograd there) to a few ulps.
"""

import pytest
import torch

from conftest import load_golden, regenerate_op_inputs
from oracle import sihc_oracle as O

OP_CASES = ["tails_s4_e24", "tails_s16_e16", "vec_s4_e8"]
TRI_CASES = ["tri_a3", "tri_a23"]


def tol(dtype):
    # explicit adjoints vs autograd: same math, different summation order
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
@pytest.mark.parametrize("case", OP_CASES)
def test_op_cases_forward_bit_exact_and_adjoints(case, tag):
    meta, t = load_golden(f"{case}_{tag}")
    dtype = getattr(torch, meta["dtype"])
    x, alpha, beta = t["x"], t["alpha"], t["beta"]
    assert x.dtype == dtype
    z = O.multi_read(x, alpha)
    assert torch.equal(torch.stack(z), t["z"])
    y = O.write(x, list(t["dz"].unbind(0)), beta)
    assert torch.equal(y, t["y"])
    dx, dalpha = O.read_backward(x, list(t["gz"].unbind(0)), alpha)
    torch.testing.assert_close(dx, t["dx_read"], **tol(dtype))
    torch.testing.assert_close(dalpha.to(dtype), t["dalpha"], **tol(dtype))
    ddz, dbeta = O.write_backward(t["gy"], list(t["dz"].unbind(0)), beta)
    torch.testing.assert_close(torch.stack(ddz), t["ddz"], **tol(dtype))
    torch.testing.assert_close(dbeta.to(dtype), t["dbeta"], **tol(dtype))
    assert torch.equal(t["dx_write"], t["gy"])          # identity carry of the write
    # read's adjoint is the write without the carry (and vice versa)
    dx2 = O.write(None, list(t["gz"].unbind(0)), alpha, like=x)
    torch.testing.assert_close(dx2, t["dx_read"], **tol(dtype))


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_config1_seed0_sampled(tag):
    meta, t = load_golden(f"cfg1_{tag}")
    dtype = getattr(torch, meta["dtype"])
    stride = meta["sample_stride"]
    inp = regenerate_op_inputs(meta)
    assert torch.equal(inp["x"].flatten()[::stride], t["x_sample"])
    assert torch.equal(inp["alpha"], t["alpha"]) and torch.equal(inp["beta"], t["beta"])
    x, alpha, beta = inp["x"], inp["alpha"], inp["beta"]
    z = O.read(x, alpha[0])
    y = O.write(x, [inp["dz"][0]], beta)
    assert torch.equal(z.flatten()[::stride], t["z"])
    assert torch.equal(y.flatten()[::stride], t["y"])
    dx, dalpha = O.read_backward(x, [inp["gz"][0]], alpha)
    ddz, dbeta = O.write_backward(inp["gy"], [inp["dz"][0]], beta)
    torch.testing.assert_close(dx.flatten()[::stride], t["dx_read"], **tol(dtype))
    torch.testing.assert_close(ddz[0].flatten()[::stride], t["ddz"], **tol(dtype))
    # weight gradients reduce over 1024 tokens: compare in relative L2
    for mine, ref in ((dalpha, t["dalpha"]), (dbeta, t["dbeta"])):
        mine = mine.to(dtype).float().flatten()[::stride]
        rel = (mine - ref.float()).norm() / ref.float().norm()
        assert rel < (1e-5 if dtype == torch.float32 else 5e-3), rel


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
@pytest.mark.parametrize("case", TRI_CASES)
def test_triangular_cases(case, tag):
    meta, t = load_golden(f"{case}_{tag}")
    dtype = getattr(torch, meta["dtype"])
    updates = list(t["updates"].unbind(0))
    out = O.triangular(t["base"], updates, t["gamma"])
    assert torch.equal(out, t["out"])
    ddz, dgamma = O.triangular_backward(t["grad"], updates, t["gamma"])
    torch.testing.assert_close(torch.stack(ddz), t["ddz"], **tol(dtype))
    torch.testing.assert_close(dgamma.to(t["gamma"].dtype), t["dgamma"], **tol(t["gamma"].dtype))
    assert torch.equal(t["dbase"], t["grad"])


@pytest.mark.parametrize("case", ["stage_p8", "stage_p4"])
def test_reference_stage_and_cell_layout(case):
    meta, t = load_golden(case)
    slots = meta["slots"]
    x, alpha, beta = t["x"], t["alpha"], t["beta"]
    assert torch.equal(O.cells(x, slots), t["cells_of_x"])
    assert torch.equal(O.high(O.cells(x, slots)), x)
    fns = [lambda z, s=s: torch.tanh(z * s) for s in meta["scales"]]
    carrier, reads, updates = O.factored_stage(x, alpha, beta, fns)
    torch.testing.assert_close(carrier, t["carrier"], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(torch.stack(reads), t["reads"], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(torch.stack(updates), t["updates"], atol=2e-5, rtol=2e-5)
    # the literal dense-carrier recurrence is algebraically the same stage
    torch.testing.assert_close(O.literal_stage(x, alpha, beta, fns), t["carrier"], atol=5e-5, rtol=5e-5)


def test_known_answer_slot_order_p8():
    # research/tests/test_reference_variants.py:85-94: first cell of a 32x32 ramp
    ramp = torch.arange(32 * 32, dtype=torch.float32).reshape(1, 32, 32, 1)
    c = O.cells(ramp, 4)
    assert c.shape == (1, 256, 4, 1)
    assert c[0, 0, :, 0].tolist() == [0.0, 1.0, 32.0, 33.0]
    _, t = load_golden("stage_p8")
    assert t["cell0"].tolist() == [0.0, 1.0, 32.0, 33.0]
    assert torch.equal(O.high(c), ramp)


def test_identity_init_stage_is_plain_residual_recurrence():
    # research/tests/test_reference_variants.py:97-123
    torch.manual_seed(3)
    x = torch.randn(2, 32, 32, 5)
    alpha = torch.full((3, 5, 4), 0.25)
    beta = torch.ones(3, 5, 4)
    fns = [lambda z, s=s: torch.tanh(z * s) for s in (0.1, 0.2, 0.3)]
    actual, _, updates = O.factored_stage(x, alpha, beta, fns)
    cx = O.cells(x, 4)
    z = cx.mean(dim=2)
    expect = []
    for fn in fns:
        u = fn(z)
        expect.append(u)
        z = z + u
    torch.testing.assert_close(actual, O.high(cx + torch.stack(expect).sum(0).unsqueeze(2)))
    for a, b in zip(updates, expect):
        torch.testing.assert_close(a, b)


def test_rectangular_cells_round_trip_and_unused_read_rows():
    for slots, (kh, kw) in ((2, (1, 2)), (8, (2, 4))):
        x = torch.randn(2, 3 * kh, 3 * kw, 5)
        assert torch.equal(O.high(O.cells(x, slots)), x)
        alpha = torch.randn(3, 5, slots)
        g = [torch.randn(2, 9, 5), None, torch.randn(2, 9, 5)]
        dx, dalpha = O.read_backward(x, g, alpha)
        assert torch.count_nonzero(dalpha[1]) == 0
        xr, ar = x.clone().requires_grad_(), alpha.clone().requires_grad_()
        z = O.multi_read(xr, ar)
        gx, ga = torch.autograd.grad([z[0], z[2]], (xr, ar), [g[0], g[2]])
        torch.testing.assert_close(dx, gx, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dalpha, ga, atol=1e-5, rtol=1e-5)
