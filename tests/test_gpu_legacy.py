"""The reference's fixed-arity block-wise operator names on the CUDA kernels, against the oracle
(shapes and tolerances of research/tests/test_p8_kernels.py and research/tests/test_blockwise_kernels.py)."""

import pytest
import torch

from oracle import sihc_oracle as O
from test_gpu_parity import close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,events,slots,high", [("p8_12", 12, 4, 32), ("b4_12", 12, 16, 64), ("b4_8", 8, 16, 64)])
def test_all_base_and_final_accumulate(name, events, slots, high, dtype):
    from residual_stream_burden_b200 import legacy
    torch.manual_seed(810)
    c = 37
    x = torch.randn(2, high, high, c).to(dtype)
    alpha = (torch.randn(events, c, slots) * 0.1).to(dtype)
    betas = [(1.0 + torch.randn(c, slots) * 0.1).to(dtype) for _ in range(events)]
    dz = [torch.randn(2, 256, c).to(dtype) * 0.3 for _ in range(events)]
    xd = x.to(DEV).requires_grad_()
    ad = alpha.to(DEV).requires_grad_()
    bd = [b.to(DEV).requires_grad_() for b in betas]
    dd = [d.to(DEV).requires_grad_() for d in dz]
    base = getattr(legacy, f"all_base_{name}_split_traceable")(xd, ad)
    close(torch.stack(base), torch.stack(O.multi_read(x, alpha)), dtype, "base")
    y = getattr(legacy, f"final_accumulate_{name}_traceable")(xd, *dd, *bd)
    close(y, O.write(x, dz, betas), dtype, "carrier")
    gy = torch.randn(y.shape).to(dtype)
    grads = torch.autograd.grad(y, (xd, *dd, *bd), gy.to(DEV))
    oddz, odb = O.write_backward(gy, dz, torch.stack(betas), acc=torch.float64)
    assert torch.equal(grads[0].cpu(), gy)
    close(torch.stack(grads[1:1 + events]), torch.stack(oddz), dtype, "ddz")
    close(torch.stack(grads[1 + events:]), odb.to(dtype), dtype, "dbeta")
    with pytest.raises(ValueError):
        getattr(legacy, f"all_base_{name}_split_traceable")(xd[:, :16], ad)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stage,active", [(8, 1), (8, 4), (8, 7), (12, 1), (12, 6), (12, 11)])
def test_triangular_active_prefix_ops(stage, active, dtype):
    from residual_stream_burden_b200 import legacy
    torch.manual_seed(1000 + stage * 16 + active)
    c = 97
    base = torch.randn(2, 256, c).to(dtype)
    dz = [torch.randn(2, 256, c).to(dtype) for _ in range(stage)]
    gamma = (torch.randn(stage, c) * 0.2).to(dtype)
    ops = getattr(legacy, f"triangular_accumulate_b4_{stage}_ptr_active_traceable_ops")
    bd = base.to(DEV).requires_grad_()
    dd = [d.to(DEV).requires_grad_() for d in dz]
    gd = gamma.to(DEV).requires_grad_()
    out = ops[active - 1](bd, *dd, gd)
    close(out, O.triangular(base, dz[:active], gamma[:active]), dtype, "out")
    go = torch.randn(out.shape).to(dtype)
    grads = torch.autograd.grad(out, (bd, gd, *dd[:active]), go.to(DEV))
    oddz, odg = O.triangular_backward(go, dz[:active], gamma[:active], acc=torch.float64)
    close(torch.stack(grads[2:]), torch.stack(oddz), dtype, "ddz")
    close(grads[1][:active], odg.to(dtype), dtype, "dgamma")
    assert torch.count_nonzero(grads[1][active:]) == 0


def test_cell_mean_b4_and_gradient():
    from residual_stream_burden_b200 import legacy
    torch.manual_seed(5)
    x = torch.randn(2, 64, 64, 24, device=DEV, requires_grad=True)
    out = legacy.cell_mean_b4_traceable(x)
    expect = O.cells(x.detach().cpu(), 16).mean(2)
    torch.testing.assert_close(out.cpu(), expect, atol=1e-6, rtol=1e-5)
    g = torch.randn_like(out)
    (dx,) = torch.autograd.grad(out, x, g)
    want = O.high((g.cpu() / 16).unsqueeze(2).expand(2, 256, 16, 24))
    torch.testing.assert_close(dx.cpu(), want, atol=1e-6, rtol=1e-5)
