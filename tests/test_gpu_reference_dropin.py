"""The UNMODIFIED reference model classes with their routing operators rebound to this library.

``oracle/_ref`` holds an unmodified copy of the reference's ``sihc`` package (made by ``oracle/make_ref.py``).
Its models import the three routing operators by name (sihc/models/sihc/sublayer.py:11,
sihc/models/sihc/model.py:29); the tests rebind exactly those names to this package's operators - the seam the
reference's own tests use (research/tests/test_blockwise_tuple_kernels.py:166-168) - and compare

  * the sublayer-wise ``SublayerSiHCModel`` and the block-wise ``SiHCModel(kernel_backend="tuple")`` against the
    reference's explicit PyTorch recurrence (``enable_reference_schedule``, sihc/models/sihc/reference.py:234-260)
    run on the same GPU with the same weights: output and every parameter gradient;
  * the class-prefix context model against the literal dense-carrier recurrence written in the test;
  * ``torch.compile(fullgraph=True)`` of the rebound model against its eager run
    (research/tests/test_sublayer_kernels.py:266-286).

Tolerances are the reference's own: fp32 output 3e-5 / 3e-4, parameter gradients atol 2e-5..3e-5, rtol 0.003;
bf16 autocast output 0.025 / 0.03, gradients atol 5e-4, rtol 0.15 (research/tests/test_sublayer_kernels.py:259-263).
"""

import copy
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    """The reference package with its operator names rebound to the CUDA library (restored afterwards)."""
    from oracle.make_ref import ref_path
    path = ref_path()
    if path is None:
        pytest.skip("oracle/_ref is missing: run `python oracle/make_ref.py` where the reference checkout exists")
    if path not in sys.path:
        sys.path.insert(0, path)
    import residual_stream_burden_b200 as b200
    import sihc.models.sihc.model as mod
    import sihc.models.sihc.sublayer as sub
    from sihc.models.sihc import reference as refmod
    saved = {(m, n): getattr(m, n) for m, names in ((sub, ("sublayer_read", "sublayer_triangular", "sublayer_write")),
                                                     (mod, ("blockwise_read", "blockwise_triangular", "blockwise_write")))
             for n in names}
    sub.sublayer_read, sub.sublayer_triangular, sub.sublayer_write = \
        b200.sublayer_read, b200.sublayer_triangular, b200.sublayer_write
    mod.blockwise_read, mod.blockwise_triangular, mod.blockwise_write = \
        b200.blockwise_read, b200.blockwise_triangular, b200.blockwise_write

    class Namespace:
        pass

    ns = Namespace()
    ns.sub, ns.mod, ns.reference, ns.b200 = sub, mod, refmod, b200
    yield ns
    for (m, n), fn in saved.items():
        setattr(m, n, fn)


def open_gates(model, connections):
    """The zero-initialised heads get small random values, as in the reference's tests
    (research/tests/test_sublayer_kernels.py:229-242): with zero heads every update is zero."""
    with torch.no_grad():
        for block in model.blocks:
            block.branch.adaLN_modulation[-1].weight.normal_(std=0.01)
            block.branch.adaLN_modulation[-1].bias.normal_(std=0.03)
            for conn in connections(block):
                conn.read_weight.add_(torch.randn_like(conn.read_weight) * 0.01)
                conn.write_weight.add_(torch.randn_like(conn.write_weight) * 0.02)
        model.final_layer.linear.weight.normal_(std=0.03)
    return model


def sublayer_connections(block):
    return (block.attention_connection, block.mlp_connection)


def block_connections(block):
    return (block.connection,)


def inputs(batch=2, seed=5):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(batch, 3, 256, 256, device=DEV, generator=g)
    t = torch.rand(batch, device=DEV, generator=g)
    y = torch.randint(0, 1000, (batch,), device=DEV, generator=g)
    return x, t, y


def compare(actual_model, expected_model, run_expected, dtype, launches):
    x, t, y = inputs()
    before = launches()
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
        actual = actual_model(x, t, y)
        expected = run_expected(expected_model, x, t, y)
    actual.float().square().mean().backward()
    expected.float().square().mean().backward()
    assert launches() > before, "the rebound model did not reach the CUDA library"
    torch.testing.assert_close(actual, expected, atol=3e-5 if dtype == torch.float32 else 0.025,
                               rtol=3e-4 if dtype == torch.float32 else 0.03)
    for (name, a), (_, b) in zip(actual_model.named_parameters(), expected_model.named_parameters()):
        assert a.grad is not None and b.grad is not None, name
        assert torch.isfinite(a.grad).all(), name
        torch.testing.assert_close(a.grad, b.grad, atol=3e-5 if dtype == torch.float32 else 5e-4,
                                   rtol=0.003 if dtype == torch.float32 else 0.15, msg=lambda m: f"{name}: {m}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("depth,patch", [(8, 8), (12, 4)])
def test_reference_sublayer_model_on_cuda_ops_matches_its_reference_schedule(ref, depth, patch, dtype):
    torch.manual_seed(19)
    model = open_gates(ref.sub.SublayerSiHCModel(hidden_size=32, num_heads=4, depth=depth, fused_stage_size=depth,
                                                 patch_size=patch, attn_backend="math").to(DEV), sublayer_connections)
    expected = ref.reference.enable_reference_schedule(copy.deepcopy(model))
    compare(model, expected, lambda m, x, t, y: m(x, t, y), dtype, ref.b200._lib.launch_count)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("depth,patch", [(8, 4), (12, 8)])
def test_reference_blockwise_tuple_model_on_cuda_ops_matches_its_reference_schedule(ref, depth, patch, dtype):
    torch.manual_seed(23)
    cls = ref.mod.SiHCModel if patch == 4 else ref.mod.FusedP8SiHCModel     # the reference's class per patch size
    model = open_gates(cls(hidden_size=32, num_heads=4, depth=depth, fused_stage_size=depth,
                           patch_size=patch, attn_backend="math", kernel_backend="tuple").to(DEV),
                       block_connections)
    expected = ref.reference.enable_reference_schedule(copy.deepcopy(model))
    compare(model, expected, lambda m, x, t, y: m(x, t, y), dtype, ref.b200._lib.launch_count)


def literal_context_forward(model, x, t, y):
    """Dense-carrier recurrence of the sublayer-wise class-prefix model: every event reads the carrier, runs its
    sublayer on [prefix tokens, spatial tokens] and writes the spatial part back (the definition used by
    research/tests/test_sublayer_context.py:40-65, on the reference's own cell view of the carrier)."""
    from sihc.models.sihc.reference import _ReferenceScheduleMixin as Cells
    y_emb = model.y_embedder(y)
    cond = model.t_embedder(t) + y_emb
    carrier = Cells._high_to_cells(model, model.x_embedder(x))
    n = model.in_context_len
    context = (y_emb.unsqueeze(1).expand(-1, n, -1) + model.in_context_posemb).to(carrier.dtype)
    for i, block in enumerate(model.blocks):
        modulation = block.branch.conditioning(cond)
        use_context = i >= model.in_context_start
        for part, conn in enumerate((block.attention_connection, block.mlp_connection)):
            z = (carrier.float() * conn.alpha(carrier.dtype).T.float()).sum(2).to(carrier.dtype)
            seq = torch.cat((context, z), dim=1) if use_context else z
            if part == 0:
                rope = model.workspace_rope_incontext if use_context else model.workspace_rope
                dseq = block.branch.attention_update(seq, modulation, rope)
            else:
                dseq = block.branch.mlp_update(seq, modulation)
            if use_context:
                context = context + dseq[:, :n]
                dz = dseq[:, n:]
            else:
                dz = dseq
            carrier = (carrier.float() + dz.float().unsqueeze(2) * conn.beta(carrier.dtype).T.float()).to(carrier.dtype)
    return model._dense_output(Cells._cells_to_high(model, carrier), cond)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_context_model_on_cuda_ops_matches_the_literal_recurrence(ref, dtype):
    torch.manual_seed(31)
    model = open_gates(ref.sub.SublayerSiHCInContextModel(hidden_size=32, num_heads=4, depth=8, fused_stage_size=8,
                                                          patch_size=8, attn_backend="math", in_context_len=4,
                                                          in_context_start=2).to(DEV), sublayer_connections)
    expected = copy.deepcopy(model)
    compare(model, expected, literal_context_forward, dtype, ref.b200._lib.launch_count)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reference_model_on_cuda_ops_compiles_fullgraph(ref, dtype):
    torch.manual_seed(42)
    model = open_gates(ref.sub.SublayerSiHCModel(hidden_size=32, num_heads=4, depth=8, fused_stage_size=8,
                                                 patch_size=8 if dtype == torch.float32 else 4,
                                                 attn_backend="math").to(DEV), sublayer_connections)
    x, t, y = inputs(batch=1)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
        eager = model(x, t, y)
    eager.float().square().mean().backward()
    grads = {name: p.grad.clone() for name, p in model.named_parameters()}
    model.zero_grad(set_to_none=True)
    compiled = torch.compile(model, mode="default", fullgraph=True)
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
        result = compiled(x, t, y)
    result.float().square().mean().backward()
    torch.testing.assert_close(result, eager, atol=3e-5 if dtype == torch.float32 else 0.025,
                               rtol=3e-4 if dtype == torch.float32 else 0.03)
    for name, p in model.named_parameters():
        torch.testing.assert_close(p.grad, grads[name], atol=3e-5 if dtype == torch.float32 else 5e-4,
                                   rtol=0.003 if dtype == torch.float32 else 0.15, msg=lambda m: f"{name}: {m}")
