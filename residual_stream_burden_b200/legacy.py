"""Fixed-arity block-wise operator names of the reference, as thin wrappers over the same CUDA kernels.

The reference's "legacy" backend (sihc/models/sihc/kernels.py) exposes one Triton op per stage size and
geometry, with every update and every beta as a separate positional tensor:

    all_base_{b4_12,b4_8,p8_12}_split_traceable(x0, alpha_stack)            -> list of base reads
    final_accumulate_{b4_12,b4_8,p8_12}_traceable(x0, *dz, *betas)          -> carrier
    triangular_accumulate_b4_{12,8}_ptr_active_traceable_ops[active - 1](base, *dz, gamma_row)
    cell_mean_b4_traceable(x)                                                -> mean over each 4x4 cell

(b4 = patch 4 = 16 slots on a 64x64 carrier; p8 = patch 8 = 4 slots on a 32x32 carrier; 8 or 12 events.)
They compute exactly what ``sublayer_read`` / ``sublayer_write`` / ``sublayer_triangular`` compute, so here
they only check the fixed shapes and forward to those operators; gradients come from the same autograd
registrations.  With these names rebound (sihc/models/sihc/model.py:30-40) every registered block-wise SiHC
model runs without Triton.
"""

from __future__ import annotations

from typing import Callable, List

import torch
from torch import Tensor

from . import ops


def _check_carrier(x0: Tensor, high: int, name: str) -> None:
    if x0.ndim != 4 or x0.shape[1] != high or x0.shape[2] != high:
        raise ValueError(f"{name} expects a carrier [B,{high},{high},C], got {tuple(x0.shape)}")


def _make_all_base(events: int, slots: int, high: int, name: str) -> Callable[[Tensor, Tensor], List[Tensor]]:
    def all_base(x0: Tensor, alpha_stack: Tensor) -> List[Tensor]:
        _check_carrier(x0, high, name)
        if alpha_stack.ndim != 3 or alpha_stack.shape[0] != events or alpha_stack.shape[2] != slots:
            raise ValueError(f"{name} expects alpha [{events},C,{slots}], got {tuple(alpha_stack.shape)}")
        return ops.sublayer_read(x0, alpha_stack)
    all_base.__name__ = name
    all_base.__doc__ = f"Multi-output base read, {events} events x {slots} slots (reference op ``sihc::{name}``)."
    return all_base


def _make_final_accumulate(events: int, slots: int, high: int, name: str):
    def final_accumulate(x0: Tensor, *args: Tensor) -> Tensor:
        _check_carrier(x0, high, name)
        if len(args) != 2 * events:
            raise ValueError(f"{name} expects {events} updates followed by {events} beta maps, got {len(args)} tensors")
        updates, betas = list(args[:events]), list(args[events:])
        for beta in betas:
            if beta.ndim != 2 or beta.shape[1] != slots:
                raise ValueError(f"{name} expects beta maps [C,{slots}], got {tuple(beta.shape)}")
        return ops.sublayer_write(x0, updates, torch.stack(betas).contiguous())
    final_accumulate.__name__ = name
    final_accumulate.__doc__ = f"Stage write x0 + sum_l beta_l dz_l, {events} events x {slots} slots (``sihc::{name}``)."
    return final_accumulate


def _make_triangular_active(stage: int, active: int):
    def triangular_active(base: Tensor, *args: Tensor) -> Tensor:
        if len(args) != stage + 1:
            raise ValueError(f"expected {stage} update slots and one gamma row, got {len(args)} tensors")
        updates, gamma = list(args[:active]), args[stage]        # slots beyond the active prefix are placeholders
        if gamma.ndim != 2 or gamma.shape[0] < active:
            raise ValueError(f"gamma must be [{stage},C] (at least {active} rows), got {tuple(gamma.shape)}")
        return ops.sublayer_triangular(base, updates, gamma[:active].contiguous())
    triangular_active.__name__ = f"triangular_accumulate_b4_{stage}_ptr_active{active}"
    triangular_active.__doc__ = (f"base + sum over the first {active} of {stage} updates of gamma[l]*dz_l "
                                 f"(``sihc::triangular_accumulate_b4_{stage}_ptr_active{active}``).")
    return triangular_active


all_base_b4_12_split_traceable = _make_all_base(12, 16, 64, "all_base_b4_12_split_traceable")
all_base_b4_8_split_traceable = _make_all_base(8, 16, 64, "all_base_b4_8_split_traceable")
all_base_p8_12_split_traceable = _make_all_base(12, 4, 32, "all_base_p8_12_split_traceable")
final_accumulate_b4_12_traceable = _make_final_accumulate(12, 16, 64, "final_accumulate_b4_12_traceable")
final_accumulate_b4_8_traceable = _make_final_accumulate(8, 16, 64, "final_accumulate_b4_8_traceable")
final_accumulate_p8_12_traceable = _make_final_accumulate(12, 4, 32, "final_accumulate_p8_12_traceable")
triangular_accumulate_b4_12_ptr_active_traceable_ops = tuple(_make_triangular_active(12, a) for a in range(1, 12))
triangular_accumulate_b4_8_ptr_active_traceable_ops = tuple(_make_triangular_active(8, a) for a in range(1, 8))


def cell_mean_b4_traceable(x: Tensor) -> Tensor:
    """Parameter-free stage seed of the write-only model: the mean of each 4x4 cell of a ``[B,64,64,C]``
    carrier (reference ``sihc::cell_mean_b4_traceable``, sihc/models/sihc/kernels.py:2532-2587).  It is the
    read with every coefficient 1/16, so it runs on the read kernel; its gradient is the matching write."""
    _check_carrier(x, 64, "cell_mean_b4")
    alpha = torch.full((1, x.shape[3], 16), 1.0 / 16.0, device=x.device, dtype=x.dtype)
    return ops.sublayer_read(x, alpha)[0]


__all__ = [
    "all_base_b4_12_split_traceable", "all_base_b4_8_split_traceable", "all_base_p8_12_split_traceable",
    "final_accumulate_b4_12_traceable", "final_accumulate_b4_8_traceable", "final_accumulate_p8_12_traceable",
    "triangular_accumulate_b4_12_ptr_active_traceable_ops", "triangular_accumulate_b4_8_ptr_active_traceable_ops",
    "cell_mean_b4_traceable",
]
