"""The model-level caller: this package's ``SublayerSiHC`` carries the reference's parameters and, with the
routing done by the CPU oracle, reproduces the reference model's output (fixture made by the reference itself)."""

import pytest
import torch

from conftest import load_golden


def build_from_golden():
    from residual_stream_burden_b200.model import SublayerSiHC
    meta, t = load_golden("model_tiny")
    model = SublayerSiHC(hidden_size=meta["hidden"], num_heads=meta["heads"], depth=meta["depth"],
                         stage_sizes=(meta["depth"],), patch_size=meta["patch"])
    state = {k: v for k, v in t.items() if k in model.state_dict()}
    model.load_state_dict(state, strict=True)
    return meta, t, model


def golden_inputs(meta, t):
    """Rebuild the fixture's inputs (same dedicated generator as ``model_case`` in make_golden.py)."""
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(2, 3, 256, 256, generator=g)
    tt = torch.rand(2, generator=g)
    assert torch.equal(x.flatten()[::meta["stride"]], t["x_sample"]) and torch.equal(tt, t["t"])
    return x, tt, t["y"].long()


def test_oracle_schedule_reproduces_reference_model_output_and_gradients():
    from oracle import sihc_model_oracle as MO
    meta, t, model = build_from_golden()
    x, tt, y = golden_inputs(meta, t)
    out = MO.factored_forward(model, x, tt, y)
    torch.testing.assert_close(out.flatten()[::meta["stride"]], t["out_sample"], atol=2e-5, rtol=2e-4)
    out.float().square().mean().backward()
    checked = 0
    for name, p in model.named_parameters():
        key = "grad::" + name
        if key in t:
            torch.testing.assert_close(p.grad, t[key], atol=2e-6, rtol=2e-3, msg=name)
            checked += 1
    assert checked >= 30


def test_state_dict_of_reference_model_loads_strictly():
    from residual_stream_burden_b200.model import SublayerSiHC
    meta, t, model = build_from_golden()
    names = set(model.state_dict())
    assert {"blocks.0.attention_connection.read_weight", "blocks.7.mlp_connection.write_weight",
            "x_embedder.proj.weight", "final_layer.linear.weight", "t_embedder.mlp.0.weight"} <= names
    assert model.blocks[0].attention_connection.read_weight.shape == (32, 4)
    assert SublayerSiHC(patch_size=4, hidden_size=32, num_heads=4, depth=2, stage_sizes=(2,)).slots == 16


def test_preset_parameter_counts_match_reference():
    from residual_stream_burden_b200.model import sihc_b, sihc_xl
    with torch.device("meta"):
        b, xl = sihc_b(), sihc_xl()
    assert sum(p.numel() for p in b.parameters()) == 130_754_496        # sihc_sublayer_1x12_d768_b8
    assert sum(p.numel() for p in xl.parameters()) == 675_850_752       # 28 x 1152, stages 8+12+8
    routing = sum(p.numel() for n, p in xl.named_parameters() if "connection" in n)
    assert routing == 516_096


def test_literal_and_factored_oracle_schedules_agree():
    from oracle import sihc_model_oracle as MO
    meta, t, model = build_from_golden()
    x, tt, y = golden_inputs(meta, t)
    with torch.no_grad():
        a = MO.literal_forward(model, x, tt, y)
        b = MO.factored_forward(model, x, tt, y)
    torch.testing.assert_close(a, b, atol=2e-5, rtol=2e-4)
    assert a.abs().mean() > 1e-3                       # gates are open: the output is not vacuous


VARIANTS = ["model_block_tiny", "model_ctx_sublayer_tiny", "model_ctx_block_tiny"]


def build_variant(name):
    from residual_stream_burden_b200.model import SiHC
    meta, t = load_golden(name)
    model = SiHC(hidden_size=meta["hidden"], num_heads=meta["heads"], depth=meta["depth"],
                 stage_sizes=tuple(meta["stages"]), patch_size=meta["patch"], frequency=meta["kind"],
                 in_context_len=meta["ctx_len"], in_context_start=meta["ctx_start"])
    model.load_state_dict({k: v for k, v in t.items() if k in model.state_dict()}, strict=True)
    return meta, t, model


@pytest.mark.parametrize("name", VARIANTS)
def test_blockwise_and_in_context_variants_reproduce_reference_models(name):
    """Block-wise events, and class-prefix context tokens in both frequencies: fixtures come from the
    reference's ``ReferenceSiHCModel`` / ``SiHCInContextModel`` / ``SublayerSiHCInContextModel`` on CPU."""
    from oracle import sihc_model_oracle as MO
    meta, t, model = build_variant(name)
    x, tt, y = golden_inputs(meta, t)
    out = MO.factored_forward(model, x, tt, y)
    torch.testing.assert_close(out.flatten()[::meta["stride"]], t["out_sample"], atol=2e-5, rtol=2e-4)
    out.float().square().mean().backward()
    checked = 0
    for pname, p in model.named_parameters():
        key = "grad::" + pname
        if key in t:
            torch.testing.assert_close(p.grad, t[key], atol=2e-6, rtol=2e-3, msg=pname)
            checked += 1
    assert checked >= 15
    with torch.no_grad():
        torch.testing.assert_close(MO.literal_forward(model, x, tt, y), out.detach(), atol=3e-5, rtol=3e-4)
