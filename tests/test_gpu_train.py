"""The captured training step (``TrainStep``) against a plain eager training loop, one GPU.

The same model, inputs, noise and optimizer settings must give the same parameters after several steps whether
the step runs as this package's single CUDA graph (stage-scoped backward, compiled sublayers, bucketed gradient
hooks, optional per-bucket optimizer on the side stream) or as the ordinary loop
``model(...) -> loss.backward() -> AdamW.step()`` with per-operator autograd.
"""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def fixed_noise_batch(x):
    """Deterministic stand-in for the random timestep / noise draw, so both runs see the same numbers."""
    b = x.shape[0]
    t = torch.linspace(0.2, 0.8, b, device=x.device)
    e = torch.sin(torch.arange(x.numel(), device=x.device, dtype=torch.float32)).reshape(x.shape)
    tt = t.view(b, 1, 1, 1)
    z = tt * x + (1 - tt) * e
    return z, t, (x - z) / (1 - tt).clamp_min(0.05)


def assert_same_training(model, ref, init):
    """Adam divides by the gradient's running magnitude, so an element whose gradient is rounding noise can move by
    a whole step in either direction; the comparison is therefore on the mean: the two runs' parameters must differ
    by a small fraction of the distance either of them travelled from the common start."""
    for (name, a), (_, b) in zip(model.named_parameters(), ref.named_parameters()):
        travelled = (b.detach() - init[name]).abs().mean()
        apart = (a.detach() - b.detach()).abs().mean()
        assert float(travelled) > 0, name
        assert float(apart) <= 0.05 * float(travelled), (name, float(apart), float(travelled))


def eager_reference(model, images, labels, steps, schedule="stage"):
    model.training_schedule = schedule         # same routing arithmetic as the captured step
    opt = torch.optim.AdamW(model.parameters(), lr=2e-4, betas=(0.9, 0.95), weight_decay=0.0, fused=True)
    losses = []
    for k in range(steps):
        z, t, v = fixed_noise_batch(images[k])
        with torch.autocast("cuda", dtype=torch.bfloat16):
            pred = model(z, t, labels)
        loss = (pred.float() - v).square().mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(loss))
    return losses


@pytest.mark.parametrize("schedule,overlap_optimizer,compile_model,shard", [
    ("stage", False, False, False), ("stage", True, False, False), ("stage", False, True, False), ("stage", True, True, True),
    ("literal", True, False, True), ("literal", True, True, True)])
def test_captured_step_matches_eager_training_loop(monkeypatch, schedule, compile_model, overlap_optimizer, shard):
    import residual_stream_burden_b200.train as T
    from residual_stream_burden_b200.model import SublayerSiHC
    monkeypatch.setattr(T, "velocity_training_batch", fixed_noise_batch)
    torch.manual_seed(7)
    model = SublayerSiHC(hidden_size=64, num_heads=4, depth=4, stage_sizes=(2, 2), patch_size=8).cuda()
    model.open_gates(std=0.05)
    ref = copy.deepcopy(model)
    init = {name: p.detach().clone() for name, p in model.named_parameters()}
    steps, batch = 6, 2
    images = [torch.randn(batch, 3, 256, 256, device="cuda") for _ in range(steps)]
    labels = torch.tensor([3, 977], device="cuda")
    want = eager_reference(ref, images, labels, steps, schedule)

    with T.TrainStep(model, batch, compile_model=compile_model, overlap_optimizer=overlap_optimizer,
                     bucket_mb=0.05, warmup=2, schedule=schedule, shard_optimizer=shard) as trainer:
        got = [float(trainer.step(images[k], labels)) for k in range(steps)]
        assert trainer.graph is not None                          # steps 3.. ran as graph replays
        if overlap_optimizer:
            assert len(trainer.exchange.buckets) > 1
    torch.testing.assert_close(torch.tensor(got), torch.tensor(want), atol=2e-3, rtol=2e-2)
    assert_same_training(model, ref, init)


def test_captured_step_exchange_hooks_with_a_single_rank_group(monkeypatch, tmp_path):
    """With a one-rank NCCL group and ``force_exchange`` the bucketed all-reduces are issued from the backward hooks
    and captured in the graph; averaging over one rank changes nothing, so the result equals the plain step."""
    import torch.distributed as dist
    import residual_stream_burden_b200.train as T
    from residual_stream_burden_b200.model import SublayerSiHC
    monkeypatch.setattr(T, "velocity_training_batch", fixed_noise_batch)
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("nccl", init_method=f"file://{tmp_path}/rendezvous", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        torch.manual_seed(11)
        model = SublayerSiHC(hidden_size=64, num_heads=4, depth=2, stage_sizes=(2,), patch_size=8).cuda()
        model.open_gates(std=0.05)
        ref = copy.deepcopy(model)
        init = {name: p.detach().clone() for name, p in model.named_parameters()}
        steps, batch = 5, 2
        images = [torch.randn(batch, 3, 256, 256, device="cuda") for _ in range(steps)]
        labels = torch.tensor([1, 2], device="cuda")
        want = eager_reference(ref, images, labels, steps)
        for in_place, sharded in ((True, False), (False, False), (True, True)):
            m = copy.deepcopy(model)
            # the graph captures collectives: it is closed before the group is destroyed, whatever happens
            with T.TrainStep(m, batch, compile_model=False, force_exchange=True, bucket_mb=0.05,
                             in_place_exchange=in_place, warmup=2, overlap_optimizer=sharded,
                             shard_optimizer=sharded) as trainer:
                got = [float(trainer.step(images[k], labels)) for k in range(steps)]
                assert trainer.graph is not None
                assert trainer.exchange.active and len(trainer.exchange.buckets) > 1
            torch.testing.assert_close(torch.tensor(got), torch.tensor(want), atol=2e-3, rtol=2e-2)
            assert_same_training(m, ref, init)
    finally:
        if own_group:
            dist.destroy_process_group()
