"""CPU oracle for the model-level callers of the SiHC routing path.

THIS FILE IS TEST INFRASTRUCTURE (see ``oracle/sihc_oracle.py``).  It runs the modules of
``residual_stream_burden_b200.model.SiHC`` (sublayer-wise or block-wise, with or without class-prefix
context tokens) through the *literal dense-carrier recurrence* - read, sublayer, write for every event - or
through the factored stage, with the CPU operators of ``sihc_oracle`` doing all the routing.  The literal
recurrence is the unfused definition the fused stage must agree with (``literal_forward``,
research/tests/test_sublayer_kernels.py:216-226; ``torch_stage``, sihc/bench/fusion_controls.py:41-85).
Pinned by fixtures produced by the reference models themselves (``tests/golden/model_*.npz``).
"""

from __future__ import annotations

import torch

from . import sihc_oracle as O


def _all_events(model, cond):
    events, start = [], 0
    for size in model.stage_sizes:
        events.append(model.stage_events(model.blocks[start:start + size], cond, start))
        start += size
    return events


def _finish(model, carrier, cond):
    b, hh, ww, c = carrier.shape
    return model.unpatchify(model.final_layer(carrier.reshape(b, hh * ww, c), cond))


def literal_forward(model, x, t, y):
    """Forward with every routing step done by the CPU oracle, one read and one write per event."""
    y_emb = model.y_embedder(y)
    cond = model.t_embedder(t) + y_emb
    carrier = model.x_embedder(x)
    context = model.initial_context(y_emb, carrier.dtype)
    for stage in _all_events(model, cond):
        for conn, update, uses_context in stage:
            z = O.read(carrier, conn.alpha(carrier.dtype))
            dz, context = model.apply_update(update, z, context, uses_context)
            carrier = O.write(carrier, [dz], [conn.beta(carrier.dtype)])
    return _finish(model, carrier, cond)


def factored_forward(model, x, t, y):
    """Same model with the factored stage (one read, triangular accumulation, one write) on the CPU oracle."""
    y_emb = model.y_embedder(y)
    cond = model.t_embedder(t) + y_emb
    carrier = model.x_embedder(x)
    context = model.initial_context(y_emb, carrier.dtype)
    for stage in _all_events(model, cond):
        alpha = torch.stack([c.alpha(carrier.dtype) for c, _, _ in stage])
        beta = torch.stack([c.beta(carrier.dtype) for c, _, _ in stage])
        base = O.multi_read(carrier, alpha)
        gamma = O.gamma_matrix(alpha, beta)
        updates = []
        for e, (_, update, uses_context) in enumerate(stage):
            z = base[e] if e == 0 else O.triangular(base[e], updates, gamma[e, :e])
            dz, context = model.apply_update(update, z, context, uses_context)
            updates.append(dz)
        carrier = O.write(carrier, updates, beta)
    return _finish(model, carrier, cond)
