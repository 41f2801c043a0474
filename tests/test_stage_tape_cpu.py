"""The stage-scoped backward (lazily transposed triangular accumulation) on CPU.

The routing operators exist on CUDA only, so - like the reference's own schedule tests, which monkey-patch the
three operators with einsum lambdas (research/tests/test_blockwise_tuple_kernels.py:141-179) - the operator names
used by ``residual_stream_burden_b200.stage`` are replaced by the CPU oracle here.  What is tested is the autograd
structure of the tape: every gradient of a stage (carrier, alpha, beta, the sublayers' own parameters) must equal
plain autograd through the oracle's factored stage and through the literal dense-carrier recurrence.
The oracle accumulates in fp32 and rounds at operator boundaries, so agreement is to fp32 rounding (2e-6 / 2e-5);
a structural error (a missing or doubled term) would be of order one.
"""

import types

import pytest
import torch

from oracle import sihc_oracle as O


def oracle_ops():
    """Differentiable CPU stand-ins with the signatures :mod:`stage` calls."""
    def stage_gamma_backward_op(grads, updates, gamma):
        dgamma = torch.zeros_like(gamma)
        for i in range(1, gamma.shape[0]):
            if grads[i] is not None:
                dgamma[i, :i] = O.triangular_backward(grads[i], updates[:i], gamma[i, :i])[1].to(gamma.dtype)
        return dgamma

    return types.SimpleNamespace(
        sublayer_read=lambda x, alpha: O.multi_read(x, alpha),
        sublayer_write=lambda x, updates, beta: O.write(x, updates, beta),
        sublayer_triangular=lambda base, updates, gamma: O.triangular(base, updates, gamma),
        _stage_gamma_backward_op=stage_gamma_backward_op,
    )


@pytest.fixture()
def stage(monkeypatch):
    import residual_stream_burden_b200.stage as stage_mod
    monkeypatch.setattr(stage_mod, "ops", oracle_ops())
    return stage_mod


def make_case(events, slots, b=2, g=3, c=10, seed=0, dtype=torch.float64):
    torch.manual_seed(seed)
    kh, kw = O.cell_shape(slots)
    x = torch.randn(b, g * kh, g * kw, c, dtype=dtype, requires_grad=True)
    alpha = (1.0 / slots + 0.1 * torch.randn(events, c, slots, dtype=dtype)).requires_grad_()
    beta = (1.0 + 0.1 * torch.randn(events, c, slots, dtype=dtype)).requires_grad_()
    mix = [(0.3 * torch.randn(c, c, dtype=dtype)).requires_grad_() for _ in range(events)]
    fns = [lambda z, w=w: 0.05 * torch.tanh(z @ w) for w in mix]
    gy = torch.randn(b, g * kh, g * kw, c, dtype=dtype)
    return x, alpha, beta, mix, fns, gy


@pytest.mark.parametrize("events,slots", [(1, 4), (2, 4), (5, 2), (8, 16), (24, 4)])
def test_stage_tape_gradients_equal_plain_autograd(stage, events, slots):
    x, alpha, beta, mix, fns, gy = make_case(events, slots, seed=events)
    leaves = [x, alpha, beta, *mix]
    out = stage.run_stage(x, alpha, beta, fns)
    got = torch.autograd.grad(out, leaves, gy)
    want_out = O.factored_stage(x, alpha, beta, fns)[0]
    want = torch.autograd.grad(want_out, leaves, gy)
    torch.testing.assert_close(out, want_out, atol=1e-6, rtol=1e-6)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=2e-6, rtol=2e-5)
    lit = torch.autograd.grad(O.literal_stage(x, alpha, beta, fns), leaves, gy)
    for a, b in zip(got, lit):
        torch.testing.assert_close(a, b, atol=2e-6, rtol=2e-5)


def test_stage_tape_with_unused_reads_and_frozen_weights(stage):
    """Events whose read feeds nothing (a sublayer that ignores its input) record no gradient; frozen
    read/write weights ask for no gamma gradient."""
    events, slots = 6, 4
    x, alpha, beta, mix, fns, gy = make_case(events, slots, seed=11)
    const = torch.randn(2, 9, 10, dtype=torch.float64)
    fns[3] = lambda z: const                      # event 3 ignores z_3: g_3 is never produced
    leaves = [x, alpha, beta] + [m for i, m in enumerate(mix) if i != 3]
    got = torch.autograd.grad(stage.run_stage(x, alpha, beta, fns), leaves, gy)
    want = torch.autograd.grad(O.factored_stage(x, alpha, beta, fns)[0], leaves, gy)
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=2e-6, rtol=2e-5)
    a0, b0 = alpha.detach(), beta.detach()        # frozen connection weights
    got = torch.autograd.grad(stage.run_stage(x, a0, b0, fns), [x], gy)
    want = torch.autograd.grad(O.factored_stage(x, a0, b0, fns)[0], [x], gy)
    torch.testing.assert_close(got[0], want[0], atol=2e-6, rtol=2e-5)


def test_stage_tape_rejects_mismatched_arguments(stage):
    x, alpha, beta, _, fns, _ = make_case(3, 4)
    with pytest.raises(ValueError):
        stage.run_stage(x, alpha, beta, fns[:2])
    with pytest.raises(ValueError):
        stage.run_stage(x, alpha, beta[:2], fns)
