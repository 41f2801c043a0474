"""Model-level parity on the GPU: the fused CUDA routing inside ``SublayerSiHC`` against the
reference model's own output/gradients (fixture) and against the literal dense-carrier oracle."""

import copy

import pytest
import torch

from conftest import load_golden
from test_model_cpu import build_from_golden, golden_inputs

pytestmark = pytest.mark.gpu


def test_fused_model_matches_reference_fixture_fp32():
    meta, t, model = build_from_golden()
    x, tt, y = golden_inputs(meta, t)
    model = model.cuda()
    out = model(x.cuda(), tt.cuda(), y.cuda())
    torch.testing.assert_close(out.flatten()[::meta["stride"]].cpu(), t["out_sample"], atol=3e-5, rtol=3e-4)
    out.float().square().mean().backward()
    checked = 0
    for name, p in model.named_parameters():
        key = "grad::" + name
        if key in t:
            torch.testing.assert_close(p.grad.cpu(), t[key], atol=3e-5, rtol=3e-3, msg=name)
            checked += 1
    assert checked >= 30


@pytest.mark.parametrize("patch,depth,stages", [(8, 8, (8,)), (4, 4, (4,)), (8, 6, (2, 4))])
def test_fused_model_bf16_autocast_vs_literal_oracle(patch, depth, stages):
    """bf16 autocast as in training; tolerances of research/tests/test_sublayer_kernels.py:245-263."""
    from oracle import sihc_model_oracle as MO
    from residual_stream_burden_b200.model import SublayerSiHC
    torch.manual_seed(19)
    model = SublayerSiHC(hidden_size=32, num_heads=4, depth=depth, stage_sizes=stages, patch_size=patch)
    model.open_gates()
    ref = copy.deepcopy(model)
    model = model.cuda()
    x = torch.randn(1, 3, 256, 256)
    tt, y = torch.rand(1), torch.zeros(1, dtype=torch.long)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(x.cuda(), tt.cuda(), y.cuda())
    with torch.autocast("cpu", dtype=torch.bfloat16):
        expect = MO.literal_forward(ref, x, tt, y)
    out.float().square().mean().backward()
    expect.float().square().mean().backward()
    torch.testing.assert_close(out.float().cpu(), expect.float(), atol=0.025, rtol=0.03)
    for (name, a), (_, b) in zip(model.named_parameters(), ref.named_parameters()):
        assert a.grad is not None and torch.isfinite(a.grad).all(), name
        if "connection" in name:
            rel = (a.grad.cpu() - b.grad).norm() / b.grad.norm().clamp_min(1e-8)
            assert rel < 0.15, (name, float(rel))


def test_training_step_and_sampler_run():
    from residual_stream_burden_b200.model import SublayerSiHC, sample_heun, velocity_training_batch
    torch.manual_seed(3)
    model = SublayerSiHC(hidden_size=64, num_heads=4, depth=4, stage_sizes=(4,), patch_size=8).cuda()
    model.open_gates()
    opt = torch.optim.AdamW(model.parameters(), lr=2e-4, betas=(0.9, 0.95), fused=True)
    x = torch.randn(4, 3, 256, 256, device="cuda")
    y = torch.randint(0, 1000, (4,), device="cuda")
    losses = []
    for _ in range(3):
        z, t, v = velocity_training_batch(x)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            pred = model(z, t, y)
        loss = (pred.float() - v).square().mean()
        loss.backward()
        assert all(p.grad is not None for p in model.parameters())
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(loss))
    assert all(torch.isfinite(torch.tensor(losses)))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        img = sample_heun(model, y, steps=3, cfg_scale=2.4, interval=(0.1, 0.9))
    assert img.shape == (4, 3, 256, 256) and torch.isfinite(img).all()


def test_triangular_under_fullgraph_compile():
    """The ops are opaque custom ops with fake kernels: they must trace under fullgraph compile
    (research/tests/test_sublayer_kernels.py:185-213)."""
    import residual_stream_burden_b200 as R
    torch.manual_seed(583)
    base = torch.randn(3, 49, 64, device="cuda", requires_grad=True)
    ups = [torch.randn_like(base).requires_grad_() for _ in range(3)]
    gamma = (torch.randn(3, 64, device="cuda") * 0.05).requires_grad_()

    def fn(base, ups, gamma):
        out = R.sublayer_triangular(base, ups, gamma)
        return out.float().square().mean() + sum(u.float().square().mean() for u in ups)

    eager = torch.autograd.grad(fn(base, ups, gamma), (base, *ups, gamma))
    compiled = torch.compile(fn, fullgraph=True)
    got = torch.autograd.grad(compiled(base, ups, gamma), (base, *ups, gamma))
    for a, b in zip(eager, got):
        torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_literal_inference_schedule_matches_oracle_and_factored(dtype):
    from oracle import sihc_model_oracle as MO
    meta, t, model = build_from_golden()
    x, tt, y = golden_inputs(meta, t)
    ref = copy.deepcopy(model)
    model = model.cuda()
    auto = torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16)
    with torch.no_grad(), auto:
        factored = model(x.cuda(), tt.cuda(), y.cuda())
        model.inference_schedule = "literal"
        literal = model(x.cuda(), tt.cuda(), y.cuda())
    with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
        expect = MO.literal_forward(ref, x, tt, y)
    atol, rtol = (3e-5, 3e-4) if dtype == torch.float32 else (0.025, 0.03)
    torch.testing.assert_close(literal.float().cpu(), expect.float(), atol=atol, rtol=rtol)
    torch.testing.assert_close(literal.float(), factored.float(), atol=atol, rtol=rtol)
    if dtype == torch.float32:
        torch.testing.assert_close(literal.flatten()[::meta["stride"]].cpu(), t["out_sample"], atol=3e-5, rtol=3e-4)


@pytest.mark.parametrize("name", ["model_block_tiny", "model_ctx_sublayer_tiny", "model_ctx_block_tiny"])
def test_blockwise_and_in_context_variants_on_gpu(name):
    """Fused CUDA routing inside the block-wise and in-context models vs the reference models' own results."""
    from test_model_cpu import build_variant
    meta, t, model = build_variant(name)
    x, tt, y = golden_inputs(meta, t)
    model = model.cuda()
    out = model(x.cuda(), tt.cuda(), y.cuda())
    torch.testing.assert_close(out.flatten()[::meta["stride"]].cpu(), t["out_sample"], atol=3e-5, rtol=3e-4)
    out.float().square().mean().backward()
    checked = 0
    for pname, p in model.named_parameters():
        key = "grad::" + pname
        if key in t:
            torch.testing.assert_close(p.grad.cpu(), t[key], atol=3e-5, rtol=3e-3, msg=pname)
            checked += 1
    assert checked >= 15
    with torch.no_grad():
        model.inference_schedule = "literal"
        lit = model(x.cuda(), tt.cuda(), y.cuda())
    torch.testing.assert_close(lit, out.detach(), atol=3e-5, rtol=3e-4)


@pytest.mark.parametrize("name", ["model_tiny", "model_block_tiny", "model_ctx_sublayer_tiny", "model_ctx_block_tiny"])
def test_stage_scoped_backward_matches_reference_fixtures(name):
    """``training_schedule = "stage"`` (lazily transposed triangular backward, one gamma-gradient pass per stage)
    against the reference models' own outputs and parameter gradients, fp32."""
    from test_model_cpu import build_variant
    meta, t, model = build_from_golden() if name == "model_tiny" else build_variant(name)
    x, tt, y = golden_inputs(meta, t)
    model = model.cuda()
    model.training_schedule = "stage"
    out = model(x.cuda(), tt.cuda(), y.cuda())
    torch.testing.assert_close(out.flatten()[::meta["stride"]].cpu(), t["out_sample"], atol=3e-5, rtol=3e-4)
    out.float().square().mean().backward()
    checked = 0
    for pname, p in model.named_parameters():
        key = "grad::" + pname
        if key in t:
            torch.testing.assert_close(p.grad.cpu(), t[key], atol=3e-5, rtol=3e-3, msg=pname)
            checked += 1
    assert checked >= 15


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("events,slots,c", [(24, 4, 64), (16, 16, 40), (5, 2, 37)])
def test_stage_scoped_backward_all_gradients_vs_literal_oracle_and_per_op_path(events, slots, c, dtype):
    """Every gradient of one stage (carrier, alpha, beta, sublayer weights): the stage-scoped schedule on the CUDA
    operators vs autograd through the oracle's literal dense-carrier recurrence (fp32 1e-5 relative, bf16 2e-2)
    and vs this package's per-operator autograd."""
    import residual_stream_burden_b200 as R
    from oracle import sihc_oracle as O
    from residual_stream_burden_b200 import stage
    torch.manual_seed(92 + events)
    kh, kw = O.cell_shape(slots)
    b, g = 2, 4
    x = torch.randn(b, g * kh, g * kw, c).to(dtype)
    alpha = (1.0 / slots + 0.05 * torch.randn(events, c, slots)).to(dtype)
    beta = (1.0 + 0.05 * torch.randn(events, c, slots)).to(dtype)
    mix = [(0.3 * torch.randn(c, c)).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * kh, g * kw, c).to(dtype)

    def leaves(dev):
        return [t.to(dev).clone().requires_grad_() for t in (x, alpha, beta, *mix)]

    def sublayers(ws):
        return [lambda z, w=w: (0.05 * torch.tanh(z.float() @ w.float())).to(z.dtype) for w in ws]

    cpu = leaves("cpu")
    want_out = O.literal_stage(cpu[0], cpu[1], cpu[2], sublayers(cpu[3:]))
    want = torch.autograd.grad(want_out, cpu, gy)

    dev = leaves("cuda")
    out = stage.run_stage(dev[0], dev[1], dev[2], sublayers(dev[3:]))
    got = torch.autograd.grad(out, dev, gy.cuda())

    per = leaves("cuda")
    base = R.sublayer_read(per[0], per[1])
    gamma = (per[1][:, None] * per[2][None, :]).sum(dim=-1)
    ups = []
    for e, fn in enumerate(sublayers(per[3:])):
        z = base[e] if e == 0 else R.sublayer_triangular(base[e], ups, gamma[e, :e].contiguous())
        ups.append(fn(z).contiguous())
    per_out = R.sublayer_write(per[0], ups, per[2])
    per_got = torch.autograd.grad(per_out, per, gy.cuda())

    tol = 1e-5 if dtype == torch.float32 else 2e-2

    def rel(a, b):
        a, b = a.detach().double().cpu(), b.detach().double().cpu()
        return float((a - b).norm() / b.norm().clamp_min(1e-12))

    assert torch.equal(out, per_out)                       # same forward kernels, same order
    # the literal recurrence rounds the carrier after every event, the factored stage once: forward and
    # gradients agree to a few roundings of the storage type
    assert rel(out, want_out) <= (1e-5 if dtype == torch.float32 else 2e-2)
    for i, (a, p, w) in enumerate(zip(got, per_got, want)):
        assert rel(a, w) <= (2e-5 if dtype == torch.float32 else 3e-2), (i, rel(a, w))
        assert rel(a, p) <= tol, (i, rel(a, p))


@pytest.mark.parametrize("name", ["model_tiny", "model_block_tiny", "model_ctx_sublayer_tiny", "model_ctx_block_tiny"])
def test_literal_training_schedule_matches_reference_fixtures(name):
    """``training_schedule = "literal"``: the fused write+read step and its fused adjoint (3S+3 elements per event)
    against the reference models' own outputs and parameter gradients, fp32."""
    from test_model_cpu import build_variant
    meta, t, model = build_from_golden() if name == "model_tiny" else build_variant(name)
    x, tt, y = golden_inputs(meta, t)
    model = model.cuda()
    model.training_schedule = "literal"
    out = model(x.cuda(), tt.cuda(), y.cuda())
    torch.testing.assert_close(out.flatten()[::meta["stride"]].cpu(), t["out_sample"], atol=3e-5, rtol=3e-4)
    out.float().square().mean().backward()
    checked = 0
    for pname, p in model.named_parameters():
        key = "grad::" + pname
        if key in t:
            torch.testing.assert_close(p.grad.cpu(), t[key], atol=3e-5, rtol=3e-3, msg=pname)
            checked += 1
    assert checked >= 15


@pytest.mark.parametrize("patch,depth,stages", [(8, 8, (8,)), (4, 4, (4,)), (8, 6, (2, 4))])
def test_literal_training_bf16_autocast_vs_literal_oracle(patch, depth, stages):
    """bf16 autocast: the literal schedule on the CUDA operators rounds the carrier after every event exactly as the
    unfused oracle does; output and connection-weight gradients against autograd through the oracle."""
    from oracle import sihc_model_oracle as MO
    from residual_stream_burden_b200.model import SublayerSiHC
    torch.manual_seed(23)
    model = SublayerSiHC(hidden_size=32, num_heads=4, depth=depth, stage_sizes=stages, patch_size=patch)
    model.open_gates()
    ref = copy.deepcopy(model)
    model = model.cuda()
    model.training_schedule = "literal"
    x = torch.randn(1, 3, 256, 256)
    tt, y = torch.rand(1), torch.zeros(1, dtype=torch.long)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(x.cuda(), tt.cuda(), y.cuda())
    with torch.autocast("cpu", dtype=torch.bfloat16):
        expect = MO.literal_forward(ref, x, tt, y)
    out.float().square().mean().backward()
    expect.float().square().mean().backward()
    torch.testing.assert_close(out.float().cpu(), expect.float(), atol=0.025, rtol=0.03)
    for (name, a), (_, b) in zip(model.named_parameters(), ref.named_parameters()):
        assert a.grad is not None and torch.isfinite(a.grad).all(), name
        if "connection" in name:
            rel = (a.grad.cpu() - b.grad).norm() / b.grad.norm().clamp_min(1e-8)
            assert rel < 0.15, (name, float(rel))
