"""CPU oracle for the model-level caller of the SiHC routing path.

THIS FILE IS TEST INFRASTRUCTURE (see ``oracle/sihc_oracle.py``).  It runs the
modules of ``residual_stream_burden_b200.model.SublayerSiHC`` through the
*literal dense-carrier recurrence* - read, sublayer, write for every event,
with the CPU operators of ``sihc_oracle`` - which is the unfused definition the
fused stage must agree with (``literal_forward``,
research/tests/test_sublayer_kernels.py:216-226).  Pinned by
``tests/golden/model_tiny.npz``, produced by the reference model itself under
``enable_reference_schedule`` (sihc/models/sihc/reference.py:234-260).
"""

from __future__ import annotations

import torch

from . import sihc_oracle as O


def literal_forward(model, x, t, y):
    """Forward of a ``SublayerSiHC`` with every routing step done by the CPU oracle."""
    cond = model.t_embedder(t) + model.y_embedder(y)
    carrier = model.x_embedder(x)
    for block in model.blocks:
        mod = block.branch.conditioning(cond)
        for conn, kind in ((block.attention_connection, "attn"), (block.mlp_connection, "mlp")):
            z = O.read(carrier, conn.alpha(carrier.dtype))
            dz = (block.branch.attention_update(z, mod, model.workspace_rope) if kind == "attn"
                  else block.branch.mlp_update(z, mod))
            carrier = O.write(carrier, [dz], [conn.beta(carrier.dtype)])
    b, hh, ww, c = carrier.shape
    return model.unpatchify(model.final_layer(carrier.reshape(b, hh * ww, c), cond))


def factored_forward(model, x, t, y):
    """Same model with the factored stage (one read, triangular accumulation, one write) on the CPU oracle."""
    cond = model.t_embedder(t) + model.y_embedder(y)
    carrier = model.x_embedder(x)
    start = 0
    for size in model.stage_sizes:
        blocks = model.blocks[start:start + size]
        start += size
        conns = [c for blk in blocks for c in (blk.attention_connection, blk.mlp_connection)]
        alpha = torch.stack([c.alpha(carrier.dtype) for c in conns])
        beta = torch.stack([c.beta(carrier.dtype) for c in conns])
        fns = []
        for blk in blocks:
            mod = blk.branch.conditioning(cond)
            fns.append(lambda z, blk=blk, mod=mod: blk.branch.attention_update(z, mod, model.workspace_rope))
            fns.append(lambda z, blk=blk, mod=mod: blk.branch.mlp_update(z, mod))
        carrier, _, _ = O.factored_stage(carrier, alpha, beta, fns)
    b, hh, ww, c = carrier.shape
    return model.unpatchify(model.final_layer(carrier.reshape(b, hh * ww, c), cond))
