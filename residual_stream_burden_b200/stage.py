"""Stage-scoped schedule: one fused stage with a lazily transposed triangular backward.

Forward is the reference's factored stage (``_run_fused_schedule_stage``, sihc/models/sihc/sublayer.py:52-72):

    base_i = read(X0, alpha_i)                         one multi-output read
    z_i    = base_i + sum_{j<i} gamma[i,j] * dz_j      triangular accumulation (gamma = sum_s alpha*beta, torch)
    dz_i   = F_i(z_i)                                  the sublayer, ordinary torch
    X_out  = X0 + sum_i beta_i * dz_i                  one multi-input write

With per-operator autograd (the reference's ``_tri_autograd``, sihc/models/sihc/sublayer_kernels.py:369-379, and
this package's ``sublayer_triangular``) event i's backward emits one ``ddz`` tensor per earlier event - about
E*E/2 tensors per stage - which autograd then adds up pair by pair.  The adjoint of the triangular accumulation
is the same accumulation with gamma transposed, so here nothing is emitted per edge.  The nodes of a stage
share a :class:`StageTape`:

  * the backward of event i's accumulation only records ``g_i = dL/dz_i`` (and passes it on to ``base_i``);
  * when autograd reaches the update ``dz_j`` - after every later event, because those consume it - its total
    gradient is formed in ONE triangular call,
        G_j = (write term) + sum_{i>j} gamma[i,j] * g_i ,
    reading E-j tensors and writing one;
  * the gradient of gamma is produced once per stage, after the last accumulation node, from the recorded
    ``g_i`` and the saved updates: ``dgamma[i,j] = sum_m g_i * dz_j``.

Traffic per stage, in workspace tensors: about E*E/2 + 2E for the update gradients instead of E*E (emit) plus
the additions.  The tape is a Python object, so this schedule runs eagerly (it can be captured in a CUDA graph);
``torch.compile`` cannot trace it - under compile use the per-operator path of :mod:`.ops`.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
from torch import Tensor

from . import ops


class StageTape:
    """What the autograd nodes of one stage share: the updates, the recorded ``g_i`` and gamma."""

    def __init__(self, events: int):
        self.events = events
        self.updates: List[Optional[Tensor]] = [None] * events     # dz_j (values only)
        self.grads: List[Optional[Tensor]] = [None] * events       # g_i = dL/dz_i, recorded in backward
        self.gamma: Optional[Tensor] = None                        # [E, E, C], values only
        self._gamma_t: Optional[Tensor] = None

    def gamma_transposed(self) -> Tensor:
        """``gamma_t[j, i] = gamma[i, j]``: row j then holds event j's coefficients in every later event."""
        if self._gamma_t is None:
            self._gamma_t = self.gamma.transpose(0, 1).contiguous()
        return self._gamma_t

    def release(self) -> None:
        self.updates = [None] * self.events
        self.grads = [None] * self.events
        self.gamma = self._gamma_t = None


class _GammaGate(torch.autograd.Function):
    """Identity on gamma in forward.  Its backward runs after every accumulation node of the stage (they all consume
    its output) and returns the whole ``dgamma`` from the tape."""

    @staticmethod
    def forward(ctx, gamma: Tensor, tape: StageTape) -> Tensor:
        ctx.set_materialize_grads(False)
        ctx.tape = tape
        tape.gamma = gamma.detach()
        return gamma.view_as(gamma)

    @staticmethod
    def backward(ctx, _unused):
        tape: StageTape = ctx.tape
        if not ctx.needs_input_grad[0]:
            return None, None
        if tape.events < 2 or all(g is None for g in tape.grads[1:]):
            return torch.zeros_like(tape.gamma), None
        # every recorded gradient and every update is read once; rows of unused reads come out zero
        return ops._stage_gamma_backward_op(tape.grads, tape.updates, tape.gamma), None


class _Accumulate(torch.autograd.Function):
    """``z_i = base_i + sum_{j<i} gamma[i,j] * dz_j``; the backward records ``g_i`` instead of emitting products."""

    @staticmethod
    def forward(ctx, tape: StageTape, event: int, base: Tensor, gamma: Tensor, *updates: Tensor) -> Tensor:
        ctx.tape, ctx.event, ctx.count = tape, event, len(updates)
        return ops.sublayer_triangular(base, list(updates), gamma[event, :event].contiguous())

    @staticmethod
    def backward(ctx, grad: Tensor):
        grad = grad.contiguous()
        ctx.tape.grads[ctx.event] = grad
        # base_i gets g_i; gamma and the updates get theirs from the gate and the injection nodes
        return (None, None, grad, None) + (None,) * ctx.count


class _Inject(torch.autograd.Function):
    """Identity on ``dz_j`` in forward; the backward adds the transposed triangular term to the incoming gradient
    (which is the write's term): ``G_j = grad + sum_{i>j} gamma[i,j] * g_i``."""

    @staticmethod
    def forward(ctx, tape: StageTape, event: int, dz: Tensor) -> Tensor:
        ctx.set_materialize_grads(False)
        ctx.tape, ctx.event = tape, event
        tape.updates[event] = dz.detach()
        return dz.view_as(dz)

    @staticmethod
    def backward(ctx, grad: Optional[Tensor]):
        tape: StageTape = ctx.tape
        j = ctx.event
        later = [(i, tape.grads[i]) for i in range(j + 1, tape.events) if tape.grads[i] is not None]
        if not later:
            return None, None, grad
        g_list = [g for _, g in later]
        coeff = tape.gamma_transposed()[j]
        if len(later) == tape.events - j - 1:
            coeff = coeff[j + 1:].contiguous()
        else:                                         # some later reads were unused: pick the live rows
            coeff = coeff[[i for i, _ in later]].contiguous()
        base = grad.contiguous() if grad is not None else torch.zeros_like(g_list[0])
        return None, None, ops.sublayer_triangular(base, g_list, coeff)


def run_stage(x0: Tensor, alpha: Tensor, beta: Tensor, sublayers: Sequence[Callable[[Tensor], Tensor]],
              gamma: Optional[Tensor] = None) -> Tensor:
    """One fused stage with the stage-scoped backward.

    ``alpha`` / ``beta`` are ``[E, C, S]`` in the carrier dtype (or fp32); ``sublayers[i](z_i)`` returns event i's
    update ``dz_i`` (any torch code; the result is made contiguous).  Same values as the per-operator stage of
    :meth:`residual_stream_burden_b200.model.SiHC.run_stage`; gradients agree to rounding (sums are formed in
    fp32 inside one kernel here, pair by pair in the storage dtype there).  ``gamma`` may be passed when the caller
    has already formed ``sum_s alpha_i * beta_j`` (``[E, E, C]``, differentiable).
    """
    events = alpha.shape[0]
    if len(sublayers) != events or beta.shape != alpha.shape:
        raise ValueError("one sublayer per connection event and matching read/write weights are required")
    base = ops.sublayer_read(x0, alpha)
    if gamma is None:
        gamma = (alpha[:, None] * beta[None, :]).sum(dim=-1)
    tape = StageTape(events)
    gamma = _GammaGate.apply(gamma, tape)
    updates: List[Tensor] = []
    for e, sublayer in enumerate(sublayers):
        z = base[e] if e == 0 else _Accumulate.apply(tape, e, base[e], gamma, *updates)
        updates.append(_Inject.apply(tape, e, sublayer(z).contiguous()))
    return ops.sublayer_write(x0, updates, beta)
