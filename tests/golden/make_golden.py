"""Generate the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own unfused PyTorch routing path
(``sihc/bench/fusion_controls.py``: ``read_torch``, ``write_torch``,
``triangular_torch``; ``sihc/models/sihc/reference.py``: ``_reference_stage``,
``_high_to_cells``) and records its outputs and autograd gradients on seeded
inputs.  The fixtures travel with the repository; the reference does not, so
no test reads the reference at run time.

Fixture format: one ``.npz`` per case; fp32 tensors are stored as float32, bf16
tensors as their raw 16-bit patterns (``uint16``), ``meta`` is a JSON string.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:          # stored as raw bf16 bit patterns
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.float().numpy()


def _save(name: str, meta: dict, **tensors) -> None:
    arrays = {k: _np(v) if isinstance(v, torch.Tensor) else np.asarray(v) for k, v in tensors.items()}
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, meta=json.dumps(meta), **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def op_case(name, fc, *, seed, b, g, slots, c, events, dtype, scale_a, mean_a, scale_b, mean_b,
            sample_stride=0):
    """Reference read/write (single- and multi-event) + all gradients on one seeded input set."""
    torch.manual_seed(seed)
    k = int(round(slots ** 0.5))
    x = torch.randn(b, g * k, g * k, c).to(dtype)
    alpha = (mean_a + scale_a * torch.randn(events, c, slots)).to(dtype)
    beta = (mean_b + scale_b * torch.randn(events, c, slots)).to(dtype)
    dz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gz = [torch.randn(b, g * g, c).to(dtype) for _ in range(events)]
    gy = torch.randn(b, g * k, g * k, c).to(dtype)

    xr, ar, br = (t.clone().requires_grad_() for t in (x, alpha, beta))
    dzr = [t.clone().requires_grad_() for t in dz]
    z = [fc.read_torch(xr, a, grid=g) for a in ar.unbind(0)]
    dx_read, dalpha = torch.autograd.grad(z, (xr, ar), gz)
    y = fc.write_torch(xr, dzr, list(br.unbind(0)), grid=g)
    dx_write, dbeta, *ddz = torch.autograd.grad(y, (xr, br, *dzr), gy)

    meta = dict(seed=seed, b=b, g=g, slots=slots, c=c, events=events,
                dtype=str(dtype).replace("torch.", ""), sample_stride=sample_stride,
                source="sihc/bench/fusion_controls.py read_torch/write_torch + torch.autograd")
    out = dict(z=torch.stack(z), y=y, dx_read=dx_read, dalpha=dalpha,
               dx_write=dx_write, dbeta=dbeta, ddz=torch.stack(ddz))
    if sample_stride:
        # Large case: inputs are regenerated from the seed by the test; keep
        # strided samples of every output plus a sample of the inputs to prove
        # the regeneration is identical.
        out = {k_: v.flatten()[::sample_stride] for k_, v in out.items()}
        out.update(x_sample=x.flatten()[::sample_stride], alpha=alpha, beta=beta)
        _save(name, meta, **out)
    else:
        _save(name, meta, x=x, alpha=alpha, beta=beta, dz=torch.stack(dz),
              gz=torch.stack(gz), gy=gy, **out)


def tri_case(name, fc, *, seed, shape, active, dtype, gamma_fp32):
    torch.manual_seed(seed)
    base = torch.randn(*shape).to(dtype)
    updates = [torch.randn(*shape).to(dtype) for _ in range(active)]
    gamma = torch.randn(active, shape[-1]) * 0.05
    if not gamma_fp32:
        gamma = gamma.to(dtype)
    grad = torch.randn(*shape).to(dtype)
    br, gr = base.clone().requires_grad_(), gamma.clone().requires_grad_()
    ur = [u.clone().requires_grad_() for u in updates]
    out = fc.triangular_torch(br, ur, gr)
    dbase, dgamma, *ddz = torch.autograd.grad(out, (br, gr, *ur), grad)
    meta = dict(seed=seed, shape=list(shape), active=active,
                dtype=str(dtype).replace("torch.", ""), gamma_fp32=gamma_fp32,
                source="sihc/bench/fusion_controls.py triangular_torch + torch.autograd")
    _save(name, meta, base=base, updates=torch.stack(updates), gamma=gamma, grad=grad,
          out=out, dbase=dbase, dgamma=dgamma, ddz=torch.stack(ddz))


def stage_case(name, reference_module, *, seed, patch, c, events):
    """``_reference_stage`` (einsum form) with tanh sublayers, fp32."""
    torch.manual_seed(seed)
    model = reference_module.ReferenceSiHCModel(
        patch_size=patch, hidden_size=16, depth=2, num_heads=4, bottleneck_dim=8,
        workspace_grid=16, fused_stage_size=2, attn_backend="math")
    k = model.high_grid // 16
    slots = k * k
    x = torch.randn(2, model.high_grid, model.high_grid, c)
    alpha = 1.0 / slots + 0.05 * torch.randn(events, c, slots)
    beta = 1.0 + 0.05 * torch.randn(events, c, slots)
    scales = [0.1 * (i + 1) for i in range(events)]
    fns = [lambda z, s=s: torch.tanh(z * s) for s in scales]
    carrier, reads, updates = model._reference_stage(x, alpha, beta, fns)
    arange = torch.arange(model.high_grid ** 2, dtype=torch.float32).reshape(1, model.high_grid, model.high_grid, 1)
    meta = dict(seed=seed, patch=patch, slots=slots, c=c, events=events, scales=scales,
                source="sihc/models/sihc/reference.py _reference_stage/_high_to_cells")
    _save(name, meta, x=x, alpha=alpha, beta=beta, carrier=carrier,
          reads=torch.stack(reads), updates=torch.stack(updates),
          cell0=model._high_to_cells(arange)[0, 0, :, 0],
          cells_of_x=model._high_to_cells(x))


def model_case(name, *, seed, depth, hidden, heads, patch):
    """The reference's own sublayer-wise model (tiny), unfused reference schedule, forward + backward on CPU."""
    from sihc.models.sihc.reference import enable_reference_schedule
    from sihc.models.sihc.sublayer import SublayerSiHCModel
    torch.manual_seed(seed)
    model = SublayerSiHCModel(hidden_size=hidden, num_heads=heads, depth=depth, fused_stage_size=depth,
                              patch_size=patch, attn_backend="math")
    with torch.no_grad():   # non-zero gates, as research/tests/test_sublayer_kernels.py:229-242
        for block in model.blocks:
            block.branch.adaLN_modulation[-1].weight.normal_(std=0.01)
            block.branch.adaLN_modulation[-1].bias.normal_(std=0.03)
            for c in (block.attention_connection, block.mlp_connection):
                c.read_weight.add_(torch.randn_like(c.read_weight) * 0.01)
                c.write_weight.add_(torch.randn_like(c.write_weight) * 0.02)
        model.final_layer.linear.weight.normal_(std=0.03)
        model.final_layer.adaLN_modulation[-1].weight.normal_(std=0.01)
    enable_reference_schedule(model)
    gen = torch.Generator().manual_seed(1234)     # inputs come from their own generator so tests can rebuild them
    x = torch.randn(2, 3, 256, 256, generator=gen)
    t = torch.rand(2, generator=gen)
    y = torch.tensor([3, 977])
    out = model(x, t, y)
    out.float().square().mean().backward()
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    grads = {"grad::" + k: p.grad.detach().clone() for k, p in model.named_parameters()
             if ("connection" in k or k.startswith("final_layer.linear") or "blocks.0.branch.attn.qkv" in k
                 or k.startswith("x_embedder"))}
    meta = dict(seed=seed, depth=depth, hidden=hidden, heads=heads, patch=patch, stride=7,
                source="sihc SublayerSiHCModel + enable_reference_schedule, CPU fp32")
    _save(name, meta, t=t, y=y.float(), x_sample=x.flatten()[::7], out_sample=out.detach().flatten()[::7], **state, **grads)


def _open_gates(model, connections):
    with torch.no_grad():   # non-zero gates, as research/tests/test_sublayer_kernels.py:229-242
        for block in model.blocks:
            block.branch.adaLN_modulation[-1].weight.normal_(std=0.01)
            block.branch.adaLN_modulation[-1].bias.normal_(std=0.03)
            for c in connections(block):
                c.read_weight.add_(torch.randn_like(c.read_weight) * 0.01)
                c.write_weight.add_(torch.randn_like(c.write_weight) * 0.02)
        model.final_layer.linear.weight.normal_(std=0.03)
        model.final_layer.adaLN_modulation[-1].weight.normal_(std=0.01)


def _model_fixture(name, model, meta, grad_filter):
    gen = torch.Generator().manual_seed(1234)
    x = torch.randn(2, 3, 256, 256, generator=gen)
    t = torch.rand(2, generator=gen)
    y = torch.tensor([3, 977])
    out = model(x, t, y)
    out.float().square().mean().backward()
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    grads = {"grad::" + k: p.grad.detach().clone() for k, p in model.named_parameters() if grad_filter(k)}
    meta = dict(meta, stride=29)
    _save(name, meta, t=t, y=y.float(), x_sample=x.flatten()[::29], out_sample=out.detach().flatten()[::29], **state, **grads)


def variant_model_cases():
    """Block-wise model under the reference schedule, and the two in-context (class-prefix) models under the
    reference's pure-torch factored control (``attach``, sihc/bench/fusion_controls.py:88-96), CPU fp32."""
    from sihc.bench.fusion_controls import attach
    from sihc.models.sihc.model import SiHCInContextModel
    from sihc.models.sihc.reference import ReferenceSiHCModel
    from sihc.models.sihc.sublayer import SublayerSiHCInContextModel
    keep = lambda k: ("connection" in k or k.startswith("final_layer.linear") or "blocks.0.branch.attn.qkv" in k
                      or k.startswith("x_embedder") or k == "in_context_posemb")
    torch.manual_seed(23)
    m = ReferenceSiHCModel(patch_size=8, hidden_size=32, depth=6, num_heads=4, workspace_grid=16,
                           stage_sizes=(2, 4), attn_backend="math")
    _open_gates(m, lambda b: [b.connection])
    _model_fixture("model_block_tiny", m, dict(kind="block", depth=6, hidden=32, heads=4, patch=8, stages=[2, 4],
                   ctx_len=0, ctx_start=0, source="sihc ReferenceSiHCModel (reference schedule), CPU fp32"), keep)
    common = dict(patch_size=4, hidden_size=32, depth=8, num_heads=4, stage_sizes=(8,), in_context_len=8,
                  in_context_start=2, attn_backend="math", repa_z_dims=(), repa_depth=None)
    torch.manual_seed(29)
    m = SublayerSiHCInContextModel(**common)
    _open_gates(m, lambda b: [b.attention_connection, b.mlp_connection])
    attach(m, "factored", "sublayer")
    _model_fixture("model_ctx_sublayer_tiny", m, dict(kind="sublayer", depth=8, hidden=32, heads=4, patch=4, stages=[8],
                   ctx_len=8, ctx_start=2, source="sihc SublayerSiHCInContextModel + factored torch control, CPU fp32"), keep)
    torch.manual_seed(31)
    m = SiHCInContextModel(kernel_backend="tuple", **common)
    _open_gates(m, lambda b: [b.connection])
    attach(m, "factored", "block")
    _model_fixture("model_ctx_block_tiny", m, dict(kind="block", depth=8, hidden=32, heads=4, patch=4, stages=[8],
                   ctx_len=8, ctx_start=2, source="sihc SiHCInContextModel + factored torch control, CPU fp32"), keep)


def main(reference_root: str) -> None:
    sys.path[:0] = [reference_root, os.path.join(reference_root, "sihc")]
    from sihc.bench import fusion_controls as fc
    from sihc.models.sihc import reference as reference_module

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    f32, bf16 = torch.float32, torch.bfloat16
    # The standalone-op configuration: batch 4, 256 tokens, n=4, width 768, fp32, seed 0.
    op_case("cfg1_fp32", fc, seed=0, b=4, g=16, slots=4, c=768, events=1, dtype=f32,
            scale_a=0.02, mean_a=0.25, scale_b=0.02, mean_b=1.0, sample_stride=251)
    op_case("cfg1_bf16", fc, seed=0, b=4, g=16, slots=4, c=768, events=1, dtype=bf16,
            scale_a=0.02, mean_a=0.25, scale_b=0.02, mean_b=1.0, sample_stride=251)
    # The reference tests' tail shapes (C=37/67, g=4/7, E up to 24; seeds from research/tests).
    for dt, tag in ((f32, "fp32"), (bf16, "bf16")):
        op_case(f"tails_s4_e24_{tag}", fc, seed=317, b=1, g=7, slots=4, c=67, events=24, dtype=dt,
                scale_a=0.05, mean_a=0.0, scale_b=0.05, mean_b=0.0)
        op_case(f"tails_s16_e16_{tag}", fc, seed=92, b=2, g=4, slots=16, c=37, events=16, dtype=dt,
                scale_a=0.07, mean_a=0.0, scale_b=0.07, mean_b=0.0)
        op_case(f"vec_s4_e8_{tag}", fc, seed=153, b=2, g=5, slots=4, c=64, events=8, dtype=dt,
                scale_a=0.05, mean_a=0.25, scale_b=0.05, mean_b=1.0)
        tri_case(f"tri_a3_{tag}", fc, seed=583, shape=(2, 49, 67), active=3, dtype=dt, gamma_fp32=True)
        tri_case(f"tri_a23_{tag}", fc, seed=583, shape=(1, 49, 67), active=23, dtype=dt, gamma_fp32=(dt == bf16))
    stage_case("stage_p8", reference_module, seed=7, patch=8, c=5, events=3)
    stage_case("stage_p4", reference_module, seed=8, patch=4, c=3, events=4)
    model_case("model_tiny", seed=19, depth=8, hidden=32, heads=4, patch=8)
    variant_model_cases()


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
