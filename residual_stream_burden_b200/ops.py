"""SiHC routing operators on the B200 CUDA library, behind the reference's API.

Drop-in for ``sihc/models/sihc/sublayer_kernels.py``: the same three callables
(``sublayer_read``, ``sublayer_write``, ``sublayer_triangular``), the same
argument meaning, the same ``ValueError`` contract for non-packed or mismatched
inputs, registered as ``torch.library`` custom ops with fake (shape-only)
implementations and autograd formulas so they work in eager mode, under
``torch.compile(fullgraph=True)`` and under DDP.  The op namespace is
``sihc_b200`` so that both libraries can be loaded in one process.

Differences from the reference, all supersets:
  * events E in 1..24 (reference: 8/12/16/24); slots S in {2,4,8,16} with cells
    1x2, 2x2, 2x4, 4x4 (reference: 4 and 16);
  * weights may be fp32 while activations are bf16 (reference: same dtype);
  * backward passes are fused where one pass can produce both adjoints, and all
    weight-gradient reductions are deterministic (no atomics).

There is no CPU implementation and no fallback: every op requires CUDA tensors
and the in-tree shared library.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch
from torch import Tensor
from torch.library import custom_op, register_autograd

from . import _lib
from ._lib import check, lib, ptr_array

CELLS = {2: (1, 2), 4: (2, 2), 8: (2, 4), 16: (4, 4)}
_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _require_packed(op_name: str, **tensors: Tensor) -> None:
    """Reject views whose memory is not the packed row-major array (reference:
    ``_require_packed``, sihc/models/sihc/kernels.py:26-32)."""
    for name, tensor in tensors.items():
        if not tensor.is_contiguous():
            raise ValueError(f"{op_name} requires contiguous {name}, got stride {tensor.stride()}")


def _geometry(x: Tensor, weights: Tensor, fake: bool = False):
    """Validate carrier/weights and return ``(batch, channels, grid, kh, kw)``.

    Mirrors ``_geometry`` (sihc/models/sihc/sublayer_kernels.py:180-193) with the
    widened event/slot ranges.
    """
    _require_packed("sublayer read/write", x=x, weights=weights)
    if x.ndim != 4 or weights.ndim != 3:
        raise ValueError("expected NHWC carrier and [events, channels, slots] weights")
    b, h, w, c = x.shape
    events, wc, slots = weights.shape
    if not 1 <= events <= _lib.MAX_EVENTS or wc != c or slots not in CELLS:
        raise ValueError("fused stages require 1..24 events, matching channels and 2/4/8/16 spatial slots")
    kh, kw = CELLS[slots]
    if h % kh or w % kw or h // kh != w // kw:
        raise ValueError("carrier grid must be square in cells and divisible by the slot grid")
    if x.dtype not in _DTYPES or weights.dtype not in (x.dtype, torch.float32):
        raise ValueError("carrier must be fp32 or bf16 and weights must use the carrier dtype or fp32")
    if x.device != weights.device or (not fake and not x.is_cuda):
        raise ValueError("carrier and weights must share one CUDA device")
    return b, c, h // kh, kh, kw


def _validate_updates(x: Tensor, weights: Tensor, updates: Sequence[Optional[Tensor]], fake: bool = False,
                      allow_missing: bool = False):
    """Reference: ``_validate_updates`` (sihc/models/sihc/sublayer_kernels.py:235-243)."""
    b, c, g, kh, kw = _geometry(x, weights, fake)
    if len(updates) != weights.shape[0]:
        raise ValueError("one workspace update is required per connection event")
    for dz in updates:
        if dz is None:
            if allow_missing:
                continue
            raise ValueError("one workspace update is required per connection event")
        _require_packed("sublayer write", update=dz)
        if dz.shape != (b, g * g, c) or dz.dtype != x.dtype or dz.device != x.device:
            raise ValueError("update geometry, dtype, or device does not match carrier")
    return b, c, g, kh, kw


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptrs(tensors: Sequence[Optional[Tensor]]):
    return ptr_array([None if t is None else t.data_ptr() for t in tensors])


def _workspace(nbytes: int, device) -> Tensor:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


# --------------------------------------------------------------------------- read
@custom_op("sihc_b200::sublayer_read", mutates_args=())
def sublayer_read(x: Tensor, alpha: Tensor) -> List[Tensor]:
    """``out[l][b,n,c] = sum_s alpha[l,c,s] * X[b, cell(n), s, c]`` for every event ``l``.

    ``x`` is the packed NHWC carrier ``[B, g*kh, g*kw, C]``; ``alpha`` is
    ``[E, C, S]``.  Returns ``E`` workspace tensors ``[B, g*g, C]`` in ``x.dtype``
    (fp32 accumulation, one rounding).  Reference: ``sublayer_read``,
    sihc/models/sihc/sublayer_kernels.py:219-232.
    """
    b, c, g, kh, kw = _geometry(x, alpha)
    out = [torch.empty((b, g * g, c), device=x.device, dtype=x.dtype) for _ in range(alpha.shape[0])]
    with torch.cuda.device(x.device):
        check(lib.sihc_read_fwd(x.data_ptr(), alpha.data_ptr(), _ptrs(out), alpha.shape[0], b, g, kh, kw, c,
                                _DTYPES[x.dtype], _DTYPES[alpha.dtype], _stream(x)), "sihc_read_fwd")
    return out


@sublayer_read.register_fake
def _read_fake(x, alpha):
    b, c, g, _, _ = _geometry(x, alpha, fake=True)
    return [x.new_empty((b, g * g, c)) for _ in range(alpha.shape[0])]


@custom_op("sihc_b200::sublayer_read_backward", mutates_args=())
def _read_backward_op(x: Tensor, grads: List[Optional[Tensor]], alpha: Tensor, need_dx: bool,
                      need_dalpha: bool) -> tuple[Tensor, Tensor]:
    """Both adjoints of the read in one call: ``(dX, dalpha)``.

    ``grads[l] is None`` marks an unused read output.  ``dalpha`` is accumulated in
    fp32 and returned in ``alpha.dtype`` (reference: ``_weights_backward`` returns
    ``weights.dtype``, sihc/models/sihc/sublayer_kernels.py:273).  An output that is
    not needed is returned as an empty tensor.
    """
    b, c, g, kh, kw = _validate_updates(x, alpha, grads, allow_missing=True)
    e = alpha.shape[0]
    dx = torch.empty_like(x) if need_dx else x.new_empty(0)
    dalpha = torch.empty(alpha.shape, device=x.device, dtype=torch.float32) if need_dalpha else alpha.new_empty(0)
    with torch.cuda.device(x.device):
        nbytes = lib.sihc_wgrad_workspace_bytes(e, b, g, kh, kw, c, _DTYPES[x.dtype]) if need_dalpha else 0
        ws = _workspace(nbytes, x.device)
        check(lib.sihc_read_bwd(x.data_ptr(), _ptrs(grads), alpha.data_ptr(),
                                dx.data_ptr() if need_dx else None, dalpha.data_ptr() if need_dalpha else None,
                                ws.data_ptr(), ws.numel(), e, b, g, kh, kw, c,
                                _DTYPES[x.dtype], _DTYPES[alpha.dtype], _stream(x)), "sihc_read_bwd")
    return dx, (dalpha.to(alpha.dtype) if need_dalpha else dalpha)


@_read_backward_op.register_fake
def _read_backward_fake(x, grads, alpha, need_dx, need_dalpha):
    return (torch.empty_like(x) if need_dx else x.new_empty(0),
            torch.empty_like(alpha) if need_dalpha else alpha.new_empty(0))


def _read_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _read_backward(ctx, grads):
    x, alpha = ctx.saved_tensors
    need_dx, need_dalpha = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    if not (need_dx or need_dalpha):
        return None, None
    grads = [g.contiguous() if g is not None else None for g in grads]
    dx, dalpha = _read_backward_op(x, grads, alpha, need_dx, need_dalpha)
    return (dx if need_dx else None), (dalpha if need_dalpha else None)


register_autograd(sublayer_read, _read_backward, setup_context=_read_setup)


# --------------------------------------------------------------------------- write
@custom_op("sihc_b200::sublayer_write_impl", mutates_args=())
def _write_impl(x: Tensor, updates: List[Tensor], beta: Tensor, add_x: bool) -> Tensor:
    """``x (if add_x) + sum_l beta[l,c,s] * updates[l]`` scattered to the carrier
    (reference: ``_write_impl``, sihc/models/sihc/sublayer_kernels.py:246-258)."""
    b, c, g, kh, kw = _validate_updates(x, beta, updates)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.sihc_write_fwd(x.data_ptr() if add_x else None, _ptrs(updates), beta.data_ptr(), out.data_ptr(),
                                 beta.shape[0], b, g, kh, kw, c, _DTYPES[x.dtype], _DTYPES[beta.dtype], _stream(x)),
              "sihc_write_fwd")
    return out


@_write_impl.register_fake
def _write_impl_fake(x, updates, beta, add_x):
    _validate_updates(x, beta, updates, fake=True)
    return torch.empty_like(x)


@custom_op("sihc_b200::sublayer_write", mutates_args=())
def sublayer_write(x: Tensor, updates: List[Tensor], beta: Tensor) -> Tensor:
    """``Y[b, cell(n), s, c] = X + sum_l beta[l,c,s] * updates[l][b,n,c]``; a new tensor like ``x``.

    Reference: ``sublayer_write``, sihc/models/sihc/sublayer_kernels.py:290-292.
    """
    return _write_impl(x, updates, beta, True)


@sublayer_write.register_fake
def _write_fake(x, updates, beta):
    return _write_impl_fake(x, updates, beta, True)


@custom_op("sihc_b200::sublayer_write_backward", mutates_args=())
def _write_backward_op(grad: Tensor, updates: List[Tensor], beta: Tensor, need_ddz: bool,
                       need_dbeta: bool) -> tuple[List[Tensor], Tensor]:
    """``(ddz list, dbeta)`` of the write; the carrier gradient is ``grad`` itself."""
    b, c, g, kh, kw = _validate_updates(grad, beta, updates)
    e = beta.shape[0]
    ddz = [torch.empty_like(u) for u in updates] if need_ddz else []
    dbeta = torch.empty(beta.shape, device=grad.device, dtype=torch.float32) if need_dbeta else beta.new_empty(0)
    with torch.cuda.device(grad.device):
        nbytes = lib.sihc_wgrad_workspace_bytes(e, b, g, kh, kw, c, _DTYPES[grad.dtype]) if need_dbeta else 0
        ws = _workspace(nbytes, grad.device)
        check(lib.sihc_write_bwd(grad.data_ptr(), _ptrs(updates), beta.data_ptr(),
                                 _ptrs(ddz) if need_ddz else None, dbeta.data_ptr() if need_dbeta else None,
                                 ws.data_ptr(), ws.numel(), e, b, g, kh, kw, c,
                                 _DTYPES[grad.dtype], _DTYPES[beta.dtype], _stream(grad)), "sihc_write_bwd")
    return ddz, (dbeta.to(beta.dtype) if need_dbeta else dbeta)


@_write_backward_op.register_fake
def _write_backward_fake(grad, updates, beta, need_ddz, need_dbeta):
    return ([torch.empty_like(u) for u in updates] if need_ddz else [],
            torch.empty_like(beta) if need_dbeta else beta.new_empty(0))


def _write_setup(ctx, inputs, output):
    _, updates, beta = inputs
    ctx.save_for_backward(beta, *updates)


def _write_backward(ctx, grad):
    beta, *updates = ctx.saved_tensors
    need_x, need_u, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
    grad = grad.contiguous()
    ddz, dbeta = None, None
    if need_u or need_b:
        ddz_list, dbeta_t = _write_backward_op(grad, updates, beta, bool(need_u), bool(need_b))
        ddz = ddz_list if need_u else None
        dbeta = dbeta_t if need_b else None
    return (grad if need_x else None), ddz, dbeta


register_autograd(sublayer_write, _write_backward, setup_context=_write_setup)


# --------------------------------------------------------------------------- triangular
def _validate_triangular(base: Tensor, updates: Sequence[Tensor], gamma: Tensor, fake: bool = False):
    """Reference: ``sublayer_triangular`` checks, sihc/models/sihc/sublayer_kernels.py:339-347
    (active prefix 1..23 there; 1..24 here)."""
    _require_packed("sublayer triangular", base=base, gamma=gamma)
    if base.ndim != 3:
        raise ValueError("workspace tensor must be [batch, tokens, channels]")
    if not 1 <= len(updates) <= _lib.MAX_EVENTS or gamma.shape != (len(updates), base.shape[-1]):
        raise ValueError("gamma must match the active prefix (1..24) and channel count")
    for dz in updates:
        _require_packed("sublayer triangular", update=dz)
        if dz.shape != base.shape or dz.dtype != base.dtype or dz.device != base.device:
            raise ValueError("active updates must match the workspace tensor")
    if base.dtype not in _DTYPES:
        raise ValueError("workspace tensor must be fp32 or bf16")
    if gamma.device != base.device or gamma.dtype not in (base.dtype, torch.float32):
        raise ValueError("gamma must share workspace device and use workspace dtype or fp32")
    if not fake and not base.is_cuda:
        raise ValueError("workspace tensor must be a CUDA tensor")


@custom_op("sihc_b200::sublayer_triangular", mutates_args=())
def sublayer_triangular(base: Tensor, updates: List[Tensor], gamma: Tensor) -> Tensor:
    """``out = base + sum_{l<len(updates)} gamma[l] * updates[l]`` (fp32 accumulate).

    Reference: ``sublayer_triangular``, sihc/models/sihc/sublayer_kernels.py:337-352.
    """
    _validate_triangular(base, updates, gamma)
    b, n, c = base.shape
    out = torch.empty_like(base)
    with torch.cuda.device(base.device):
        check(lib.sihc_tri_fwd(base.data_ptr(), _ptrs(updates), gamma.data_ptr(), out.data_ptr(), len(updates),
                               b * n, c, _DTYPES[base.dtype], _DTYPES[gamma.dtype], _stream(base)), "sihc_tri_fwd")
    return out


@sublayer_triangular.register_fake
def _tri_fake(base, updates, gamma):
    _validate_triangular(base, updates, gamma, fake=True)
    return torch.empty_like(base)


@custom_op("sihc_b200::sublayer_triangular_backward", mutates_args=())
def _tri_backward_op(grad: Tensor, updates: List[Tensor], gamma: Tensor, need_ddz: bool,
                     need_dgamma: bool) -> tuple[List[Tensor], Tensor]:
    """``ddz[l] = grad * gamma[l]`` and ``dgamma[l,c] = sum_m grad * updates[l]`` in one pass over ``grad``."""
    _validate_triangular(grad, updates, gamma)
    b, n, c = grad.shape
    j = len(updates)
    ddz = [torch.empty_like(grad) for _ in range(j)] if need_ddz else []
    dgamma = torch.empty(gamma.shape, device=grad.device, dtype=torch.float32) if need_dgamma else gamma.new_empty(0)
    with torch.cuda.device(grad.device):
        nbytes = lib.sihc_tri_workspace_bytes(j, b * n, c, _DTYPES[grad.dtype]) if need_dgamma else 0
        ws = _workspace(nbytes, grad.device)
        check(lib.sihc_tri_bwd(grad.data_ptr(), _ptrs(updates), gamma.data_ptr(), _ptrs(ddz) if need_ddz else None,
                               dgamma.data_ptr() if need_dgamma else None, ws.data_ptr(), ws.numel(), j, b * n, c,
                               _DTYPES[grad.dtype], _DTYPES[gamma.dtype], _stream(grad)), "sihc_tri_bwd")
    return ddz, (dgamma.to(gamma.dtype) if need_dgamma else dgamma)


@_tri_backward_op.register_fake
def _tri_backward_fake(grad, updates, gamma, need_ddz, need_dgamma):
    return ([torch.empty_like(grad) for _ in updates] if need_ddz else [],
            torch.empty_like(gamma) if need_dgamma else gamma.new_empty(0))


def _tri_setup(ctx, inputs, output):
    _, updates, gamma = inputs
    ctx.save_for_backward(gamma, *updates)


def _tri_backward(ctx, grad):
    gamma, *updates = ctx.saved_tensors
    need_base, need_u, need_g = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
    grad = grad.contiguous()
    ddz, dgamma = None, None
    # The per-edge products ddz_l = grad * gamma_l are produced by the kernel (one pass over grad for all
    # edges).  Leaving them to the compiler as torch ops, as the reference does
    # (sihc/models/sihc/sublayer_kernels.py:373-379), was measured slower here: 94.6 vs 60.5 ms per
    # SiHC-XL training step on B200.
    if need_u or need_g:
        ddz_list, dgamma_t = _tri_backward_op(grad, updates, gamma, bool(need_u), bool(need_g))
        ddz = ddz_list if need_u else None
        dgamma = dgamma_t if need_g else None
    return (grad if need_base else None), ddz, dgamma


register_autograd(sublayer_triangular, _tri_backward, setup_context=_tri_setup)


@custom_op("sihc_b200::stage_gamma_backward", mutates_args=())
def _stage_gamma_backward_op(grads: List[Optional[Tensor]], updates: List[Tensor], gamma: Tensor) -> Tensor:
    """``dgamma[i,j,c] = sum_m grads[i] * updates[j]`` for ``j < i`` (zero elsewhere), the gradient of a whole
    stage's coefficient matrix ``gamma [E,E,C]`` in one pass over the recorded gradients and the updates.

    ``grads[i]`` is the gradient that reached event i's accumulated read (``grads[0]`` is ignored; ``None`` = the
    read was never used: zero row).  Replaces one ``_tri_gamma_backward`` call per event
    (sihc/models/sihc/sublayer_kernels.py:355-361).  Returned in ``gamma.dtype`` (fp32 accumulation).
    """
    e = gamma.shape[0]
    if gamma.ndim != 3 or gamma.shape[1] != e or len(grads) != e or len(updates) != e:
        raise ValueError("expected gamma [events, events, channels] and one gradient slot and one update per event")
    ref = updates[0]
    _require_packed("stage gamma backward", gamma=gamma)
    for t in list(updates) + [g for g in grads if g is not None]:
        _require_packed("stage gamma backward", tensor=t)
        if t.shape != ref.shape or t.dtype != ref.dtype or t.device != ref.device:
            raise ValueError("gradients and updates must share shape, dtype and device")
    if ref.ndim != 3 or ref.shape[-1] != gamma.shape[-1] or ref.dtype not in _DTYPES or not ref.is_cuda:
        raise ValueError("expected CUDA workspace tensors [batch, tokens, channels] matching gamma's channels")
    b, n, c = ref.shape
    dgamma = torch.empty((e, e, c), device=ref.device, dtype=torch.float32)
    with torch.cuda.device(ref.device):
        nbytes = lib.sihc_tri_dgamma_workspace_bytes(e, b * n, c, _DTYPES[ref.dtype])
        ws = _workspace(nbytes, ref.device)
        check(lib.sihc_tri_dgamma(_ptrs(grads), _ptrs(updates), dgamma.data_ptr(), ws.data_ptr(), ws.numel(), e, b * n, c,
                                  _DTYPES[ref.dtype], _stream(ref)), "sihc_tri_dgamma")
    return dgamma.to(gamma.dtype)


@_stage_gamma_backward_op.register_fake
def _stage_gamma_backward_fake(grads, updates, gamma):
    return torch.empty_like(gamma)


# --------------------------------------------------------------------------- single-event API
class _SihcRead(torch.autograd.Function):
    """Single-event read as a plain autograd Function (eager path)."""

    @staticmethod
    def forward(ctx, x: Tensor, alpha: Tensor) -> Tensor:
        ctx.save_for_backward(x, alpha)
        return sublayer_read(x, alpha.unsqueeze(0).contiguous())[0]

    @staticmethod
    def backward(ctx, grad: Tensor):
        x, alpha = ctx.saved_tensors
        dx, dalpha = _read_backward_op(x, [grad.contiguous()], alpha.unsqueeze(0).contiguous(),
                                       ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return (dx if ctx.needs_input_grad[0] else None), (dalpha[0] if ctx.needs_input_grad[1] else None)


class _SihcWrite(torch.autograd.Function):
    """Single-event write as a plain autograd Function (eager path)."""

    @staticmethod
    def forward(ctx, x: Tensor, dz: Tensor, beta: Tensor) -> Tensor:
        ctx.save_for_backward(dz, beta)
        return _write_impl(x, [dz], beta.unsqueeze(0).contiguous(), True)

    @staticmethod
    def backward(ctx, grad: Tensor):
        dz, beta = ctx.saved_tensors
        grad = grad.contiguous()
        need_u, need_b = ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        ddz, dbeta = None, None
        if need_u or need_b:
            ddz_list, dbeta_t = _write_backward_op(grad, [dz], beta.unsqueeze(0).contiguous(), need_u, need_b)
            ddz = ddz_list[0] if need_u else None
            dbeta = dbeta_t[0] if need_b else None
        return (grad if ctx.needs_input_grad[0] else None), ddz, dbeta


def sihc_read(x: Tensor, alpha: Tensor) -> Tensor:
    """One connection event's read: ``z[b,n,c] = sum_s alpha[c,s] * X[b, cell(n), s, c]``.

    ``alpha`` is ``[C, S]``.  The unfused definition is ``read_torch``
    (sihc/bench/fusion_controls.py:14-20).
    """
    if alpha.ndim != 2:
        raise ValueError("expected [channels, slots] read weights")
    return _SihcRead.apply(x, alpha)


def sihc_write(x: Tensor, dz: Tensor, beta: Tensor) -> Tensor:
    """One connection event's write: ``Y[b, cell(n), s, c] = X + beta[c,s] * dz[b,n,c]``.

    ``beta`` is ``[C, S]``.  The unfused definition is ``write_torch``
    (sihc/bench/fusion_controls.py:23-31).
    """
    if beta.ndim != 2:
        raise ValueError("expected [channels, slots] write weights")
    return _SihcWrite.apply(x, dz, beta)


@custom_op("sihc_b200::write_read", mutates_args=())
def sihc_write_read(x: Tensor, dz: Tensor, beta: Tensor, alpha_next: Tensor) -> tuple[Tensor, Tensor]:
    """One step of the literal schedule: ``Y = X + beta * dz`` and the NEXT event's read
    ``z = sum_s alpha_next * Y`` in a single pass over the carrier.  Returns ``(Y, z)``.

    ``beta`` and ``alpha_next`` are ``[C, S]``.  Same values as ``write_torch`` followed by ``read_torch``
    (sihc/bench/fusion_controls.py:14-31): the carrier is rounded to its storage dtype before it is read.
    Differentiable in every argument: the backward is one fused pass (``sihc_write_read_bwd``).
    """
    if beta.ndim != 2 or alpha_next.ndim != 2 or beta.shape != alpha_next.shape or beta.dtype != alpha_next.dtype:
        raise ValueError("expected matching [channels, slots] write and read weights")
    _require_packed("sublayer write/read", alpha_next=alpha_next)
    b, c, g, kh, kw = _validate_updates(x, beta.unsqueeze(0), [dz])
    y = torch.empty_like(x)
    z = torch.empty((b, g * g, c), device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        check(lib.sihc_write_read_fwd(x.data_ptr(), dz.data_ptr(), beta.data_ptr(), alpha_next.data_ptr(),
                                      y.data_ptr(), z.data_ptr(), b, g, kh, kw, c,
                                      _DTYPES[x.dtype], _DTYPES[beta.dtype], _stream(x)), "sihc_write_read_fwd")
    return y, z


@sihc_write_read.register_fake
def _write_read_fake(x, dz, beta, alpha_next):
    b, c, g, _, _ = _validate_updates(x, beta.unsqueeze(0), [dz], fake=True)
    return torch.empty_like(x), x.new_empty((b, g * g, c))


@custom_op("sihc_b200::write_read_backward", mutates_args=())
def _write_read_backward_op(grad_y: Optional[Tensor], grad_z: Optional[Tensor], y: Tensor, dz: Tensor, beta: Tensor,
                            alpha_next: Tensor, need_dx: bool, need_ddz: bool,
                            need_dw: bool) -> tuple[Tensor, Tensor, Tensor]:
    """All adjoints of :func:`sihc_write_read` in one pass: ``(dX, ddz, dweights)`` with
    ``dX = grad_y + alpha_next * grad_z``, ``ddz = sum_s beta * dX``, ``dweights[0] = dalpha_next = sum_m Y * grad_z``
    and ``dweights[1] = dbeta = sum_m dz * dX`` (fp32 accumulation, returned in the weights' dtype).  A missing
    incoming gradient is ``None``; an output that is not needed comes back empty."""
    b, c, g, kh, kw = _validate_updates(y, beta.unsqueeze(0), [dz])
    for name, t, like in (("grad_y", grad_y, y), ("grad_z", grad_z, dz)):
        if t is not None:
            _require_packed("sublayer write/read backward", **{name: t})
            if t.shape != like.shape or t.dtype != like.dtype or t.device != like.device:
                raise ValueError(f"{name} does not match the forward output")
    dx = torch.empty_like(y) if need_dx else y.new_empty(0)
    ddz = torch.empty_like(dz) if need_ddz else dz.new_empty(0)
    dw = torch.empty((2,) + tuple(beta.shape), device=y.device, dtype=torch.float32) if need_dw else beta.new_empty(0)
    with torch.cuda.device(y.device):
        nbytes = lib.sihc_write_read_bwd_workspace_bytes(b, g, kh, kw, c, _DTYPES[y.dtype]) if need_dw else 0
        ws = _workspace(nbytes, y.device)
        check(lib.sihc_write_read_bwd(None if grad_y is None else grad_y.data_ptr(),
                                      None if grad_z is None else grad_z.data_ptr(), y.data_ptr(), dz.data_ptr(),
                                      beta.data_ptr(), alpha_next.data_ptr(), dx.data_ptr() if need_dx else None,
                                      ddz.data_ptr() if need_ddz else None, dw.data_ptr() if need_dw else None,
                                      ws.data_ptr(), ws.numel(), b, g, kh, kw, c, _DTYPES[y.dtype], _DTYPES[beta.dtype],
                                      _stream(y)), "sihc_write_read_bwd")
    return dx, ddz, (dw.to(beta.dtype) if need_dw else dw)


@_write_read_backward_op.register_fake
def _write_read_backward_fake(grad_y, grad_z, y, dz, beta, alpha_next, need_dx, need_ddz, need_dw):
    return (torch.empty_like(y) if need_dx else y.new_empty(0), torch.empty_like(dz) if need_ddz else dz.new_empty(0),
            beta.new_empty((2,) + tuple(beta.shape)) if need_dw else beta.new_empty(0))


def _write_read_setup(ctx, inputs, output):
    _, dz, beta, alpha_next = inputs
    ctx.save_for_backward(output[0], dz, beta, alpha_next)
    ctx.set_materialize_grads(False)


def _write_read_backward(ctx, grad_y, grad_z):
    y, dz, beta, alpha_next = ctx.saved_tensors
    need_x, need_u, need_b, need_a = ctx.needs_input_grad
    if grad_y is None and grad_z is None:
        return None, None, None, None
    grad_y = None if grad_y is None else grad_y.contiguous()
    grad_z = None if grad_z is None else grad_z.contiguous()
    dx, ddz, dw = _write_read_backward_op(grad_y, grad_z, y, dz, beta, alpha_next, bool(need_x), bool(need_u),
                                          bool(need_b or need_a))
    return (dx if need_x else None), (ddz if need_u else None), (dw[1] if need_b else None), (dw[0] if need_a else None)


register_autograd(sihc_write_read, _write_read_backward, setup_context=_write_read_setup)


# --------------------------------------------------------------------------- block-wise adapters
def _require_block_events(weights: Tensor) -> None:
    if weights.ndim != 3 or weights.shape[0] not in (8, 12):
        raise ValueError("block-wise weights must have shape [8 or 12, channels, slots]")


def blockwise_read(x: Tensor, alpha: Tensor) -> List[Tensor]:
    """Reference: ``blockwise_read``, sihc/models/sihc/blockwise_kernels.py:20-23."""
    _require_block_events(alpha)
    return sublayer_read(x, alpha)


def blockwise_write(x: Tensor, updates: List[Tensor], beta: Tensor) -> Tensor:
    """Reference: ``blockwise_write``, sihc/models/sihc/blockwise_kernels.py:26-29."""
    _require_block_events(beta)
    return sublayer_write(x, updates, beta)


def blockwise_triangular(base: Tensor, updates: List[Tensor], gamma: Tensor) -> Tensor:
    """Reference: ``blockwise_triangular``, sihc/models/sihc/blockwise_kernels.py:32-38."""
    if not 1 <= len(updates) <= 11:
        raise ValueError("block-wise triangular accumulation requires 1..11 active updates")
    return sublayer_triangular(base, updates, gamma)


__all__ = [
    "sublayer_read", "sublayer_write", "sublayer_triangular",
    "blockwise_read", "blockwise_write", "blockwise_triangular",
    "sihc_read", "sihc_write", "sihc_write_read",
]
