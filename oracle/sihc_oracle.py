"""CPU oracle for the SiHC hyper-connection read / write / triangular path.

THIS FILE IS TEST INFRASTRUCTURE.  It is a plain PyTorch (CPU, eager)
restatement of the reference's *unfused* routing path and exists only so that
the CUDA kernels can be checked against it and so that the benchmark can time a
CPU baseline next to the GPU number.  Nothing in the shipped package imports
it; the product path is the CUDA library and fails loudly without it.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
itself (``sihc/bench/fusion_controls.py`` and ``sihc/models/sihc/reference.py``)
and stores its outputs on seeded inputs as fixtures under ``tests/golden``;
``tests/test_oracle_golden.py`` checks every function here against them, and
against the reference's one known-answer vector (slot order ``[0, 1, 32, 33]``,
``research/tests/test_reference_variants.py:85-94``).

Geometry (restates ``_high_offsets``, ``sihc/models/sihc/sublayer_kernels.py:21-25``
and ``_high_to_cells`` / ``_cells_to_high``, ``sihc/models/sihc/reference.py:22-51``):
the carrier ``X`` is NHWC ``[B, g*KH, g*KW, C]``; workspace token ``m = (b, wy, wx)``
owns the ``KH x KW`` cell of carrier pixels ``(wy*KH+uy, wx*KW+ux)``; slot
``s = uy*KW + ux``.  The reference only has square cells (``KH == KW``, S in {4,16});
rectangular cells (S=2 -> 1x2, S=8 -> 2x4) are this build's extension and keep
the same row-major slot numbering.

All functions accumulate in fp32 (or fp64 when asked) and cast once at the
boundary, which is the reference's kernel contract
(``sihc/bench/fusion_controls.py:6-8``).
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch
from torch import Tensor

CELL_SHAPES = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4), 16: (4, 4)}


def cell_shape(slots: int) -> tuple[int, int]:
    """Slots per token -> (KH, KW); square for the reference's S in {4, 16}."""
    if slots not in CELL_SHAPES:
        raise ValueError(f"unsupported slot count {slots}")
    return CELL_SHAPES[slots]


def cells(x: Tensor, slots: int) -> Tensor:
    """Carrier ``[B, g*KH, g*KW, C]`` -> cells ``[B, g*g, S, C]``.

    Follows ``_high_to_cells`` (``sihc/models/sihc/reference.py:22-35``) and the
    test helper ``cells`` (``research/tests/test_sublayer_kernels.py:20-24``).
    """
    kh, kw = cell_shape(slots)
    b, h, w, c = x.shape
    g = h // kh
    if g * kh != h or g * kw != w:
        raise ValueError("carrier grid does not match the slot grid")
    return (x.reshape(b, g, kh, g, kw, c).permute(0, 1, 3, 2, 4, 5)
            .reshape(b, g * g, slots, c))


def high(cell: Tensor) -> Tensor:
    """Cells ``[B, g*g, S, C]`` -> carrier; inverse of :func:`cells`.

    Follows ``_cells_to_high`` (``sihc/models/sihc/reference.py:37-51``).
    """
    b, n, s, c = cell.shape
    kh, kw = cell_shape(s)
    g = int(round(n ** 0.5))
    if g * g != n:
        raise ValueError("token count is not a square grid")
    return (cell.reshape(b, g, g, kh, kw, c).permute(0, 1, 3, 2, 4, 5)
            .reshape(b, g * kh, g * kw, c))


def read(x: Tensor, alpha: Tensor, acc: torch.dtype = torch.float32) -> Tensor:
    """Single-event read ``z[m,c] = sum_s alpha[c,s] * X[m,s,c]``.

    ``alpha`` is ``[C, S]``.  Follows ``read_torch``
    (``sihc/bench/fusion_controls.py:14-20``): accumulate wide, cast once.
    """
    s = alpha.shape[1]
    kh, kw = cell_shape(s)
    b, h, w, c = x.shape
    g = h // kh
    view = x.reshape(b, g, kh, g, kw, c).to(acc)
    weights = alpha.T.reshape(1, 1, kh, 1, kw, c).to(acc)
    return (view * weights).sum((2, 4)).reshape(b, g * g, c).to(x.dtype)


def write(x: Tensor | None, updates: Sequence[Tensor], betas: Sequence[Tensor] | Tensor,
          acc: torch.dtype = torch.float32, like: Tensor | None = None) -> Tensor:
    """Write ``Y[m,s,c] = X[m,s,c] + sum_l beta_l[c,s] * dz_l[m,c]``.

    ``betas`` is a sequence (or stacked ``[E, C, S]`` tensor) of ``[C, S]`` maps.
    Follows ``write_torch`` (``sihc/bench/fusion_controls.py:23-31``).  With
    ``x=None`` the identity carry is dropped, which is the read's adjoint
    (``_write_impl(..., add_x=False)``, ``sihc/models/sihc/sublayer_kernels.py:284``);
    ``like`` then gives the carrier shape/dtype.
    """
    ref = x if x is not None else like
    s = betas[0].shape[1]
    kh, kw = cell_shape(s)
    b, h, w, c = ref.shape
    g = h // kh
    value = (x.reshape(b, g, kh, g, kw, c).to(acc) if x is not None
             else torch.zeros(b, g, kh, g, kw, c, dtype=acc))
    for dz, beta in zip(updates, betas):
        delta = dz.reshape(b, g, 1, g, 1, c).to(acc)
        weight = beta.T.reshape(1, 1, kh, 1, kw, c).to(acc)
        value = value + delta * weight
    return value.reshape(ref.shape).to(ref.dtype)


def triangular(base: Tensor, updates: Sequence[Tensor], gamma: Tensor,
               acc: torch.dtype = torch.float32) -> Tensor:
    """``out = base + sum_{l<j} gamma[l,c] * dz_l``; ``gamma`` is ``[j, C]``.

    Follows ``triangular_torch`` (``sihc/bench/fusion_controls.py:34-38``).
    """
    value = base.to(acc)
    for j, dz in enumerate(updates):
        value = value + dz.to(acc) * gamma[j].to(acc)
    return value.to(base.dtype)


def multi_read(x: Tensor, alpha: Tensor, acc: torch.dtype = torch.float32) -> list[Tensor]:
    """Stage read: one workspace tensor per event, ``alpha`` is ``[E, C, S]``.

    Same contraction as ``torch.einsum("bnsc,lcs->lbnc", cells, alpha)``
    (``sihc/models/sihc/reference.py:72``).
    """
    return [read(x, a, acc) for a in alpha.unbind(0)]


# --- explicit adjoints (written out, not autograd) ---------------------------
# The adjoint structure is the one the reference's autograd glue uses:
# ``_read_backward`` (sihc/models/sihc/sublayer_kernels.py:280-284) and
# ``_write_backward`` (:300-303), ``_tri_autograd`` (:369-379).  Weight and
# gamma gradients are returned in fp32 ([E, C, S] / [J, C]); callers cast.

def read_backward(x: Tensor, grads: Sequence[Tensor | None], alpha: Tensor,
                  acc: torch.dtype = torch.float32) -> tuple[Tensor, Tensor]:
    """Adjoint of the stage read.  Returns ``(dX like x, dalpha [E,C,S] in acc)``.

    ``dX[m,s,c] = sum_l alpha_l[c,s] g_l[m,c]``;
    ``dalpha_l[c,s] = sum_m X[m,s,c] g_l[m,c]``.  A missing (``None``) output
    gradient contributes nothing and leaves its ``dalpha`` row exactly zero
    (``research/tests/test_sublayer_kernels.py:122-123``).
    """
    e, c, s = alpha.shape
    cx = cells(x, s).to(acc)                                   # [B, N, S, C]
    dcell = torch.zeros_like(cx)
    dalpha = torch.zeros(e, c, s, dtype=acc)
    for l, g in enumerate(grads):
        if g is None:
            continue
        gl = g.to(acc)                                          # [B, N, C]
        dcell += gl.unsqueeze(2) * alpha[l].T.to(acc)           # [S, C] broadcast
        dalpha[l] = (cx * gl.unsqueeze(2)).sum((0, 1)).T
    return high(dcell).to(x.dtype), dalpha


def write_backward(grad: Tensor, updates: Sequence[Tensor], beta: Tensor,
                   acc: torch.dtype = torch.float32) -> tuple[list[Tensor], Tensor]:
    """Adjoint of the stage write w.r.t. updates and beta (``dX`` is ``grad`` itself).

    ``ddz_l[m,c] = sum_s beta_l[c,s] h[m,s,c]``;
    ``dbeta_l[c,s] = sum_m dz_l[m,c] h[m,s,c]``.
    """
    e, c, s = beta.shape
    ch = cells(grad, s).to(acc)
    ddz = []
    dbeta = torch.zeros(e, c, s, dtype=acc)
    for l, dz in enumerate(updates):
        ddz.append((ch * beta[l].T.to(acc)).sum(2).to(dz.dtype))
        dbeta[l] = (ch * dz.to(acc).unsqueeze(2)).sum((0, 1)).T
    return ddz, dbeta


def triangular_backward(grad: Tensor, updates: Sequence[Tensor], gamma: Tensor,
                        acc: torch.dtype = torch.float32) -> tuple[list[Tensor], Tensor]:
    """``ddz_l = grad * gamma_l`` (fp32 product, one cast); ``dgamma[l,c] = sum_m grad*dz_l``."""
    g = grad.to(acc)
    ddz = [(g * gamma[l].to(acc)).to(grad.dtype) for l in range(len(updates))]
    dgamma = torch.stack([(g * dz.to(acc)).sum((0, 1)) for dz in updates])
    return ddz, dgamma


# --- stage recurrences -------------------------------------------------------

def gamma_matrix(alpha: Tensor, beta: Tensor) -> Tensor:
    """``gamma[i,j,c] = sum_s alpha_i[c,s] beta_j[c,s]`` (``sihc/models/sihc/sublayer.py:60``)."""
    return (alpha[:, None] * beta[None, :]).sum(dim=-1)


def factored_stage(x: Tensor, alpha: Tensor, beta: Tensor,
                   update_functions: Sequence[Callable[[Tensor], Tensor]]):
    """Factored stage: one read of X0, triangular accumulation, one write.

    Restates ``_reference_stage`` (``sihc/models/sihc/reference.py:64-84``) with
    the boundary-cast operators above; returns ``(carrier, reads, updates)``.
    """
    base = multi_read(x, alpha)
    gamma = gamma_matrix(alpha, beta)
    reads, updates = [], []
    for i, fn in enumerate(update_functions):
        z = base[i] if i == 0 else triangular(base[i], updates, gamma[i, :i])
        reads.append(z)
        updates.append(fn(z))
    return write(x, updates, beta), reads, updates


def literal_stage(x: Tensor, alpha: Tensor, beta: Tensor,
                  update_functions: Sequence[Callable[[Tensor], Tensor]]) -> Tensor:
    """Literal dense-carrier recurrence: read, sublayer, write, for every event.

    This is the unfused path the fused ops must agree with
    (``research/tests/test_sublayer_kernels.py:91-99``, ``sihc/bench/fusion_controls.py:64,80``).
    """
    carrier = x
    for i, fn in enumerate(update_functions):
        z = read(carrier, alpha[i])
        carrier = write(carrier, [fn(z)], [beta[i]])
    return carrier
