"""SiHC denoisers: the callers of the routing operators.

A self-contained mirror of the reference's sublayer-wise and block-wise models, with or without class-prefix
context tokens
(``SublayerSiHCModel``, sihc/models/sihc/sublayer.py:30-72, on top of
``_SiHCBase``, sihc/models/sihc/model.py:186-513, and the blocks of
sihc/models/sihc/components.py).  Parameter names, shapes and initialisation
follow the reference so that its state dicts load unchanged; the code is this
package's own.  The residual carrier is routed exclusively by the CUDA
operators of :mod:`residual_stream_burden_b200.ops` - there is no torch
fallback for the routing in this module - while the attention and MLP sublayers
stay ordinary torch (cuBLAS GEMMs + SDPA), as in the reference.

Stage recurrence for E = 2 * blocks events (attention and MLP of each block):

    base_i = read(X0, alpha_i)                       one multi-output read of X0
    z_i    = base_i + sum_{j<i} gamma[i,j] * dz_j    triangular accumulation
    dz_i   = F_i(z_i)                                gated attention / MLP update
    X_out  = X0 + sum_i beta_i * dz_i                one multi-input write
"""

from __future__ import annotations

import math
from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import ops, stage


def _modulate(x: Tensor, shift: Tensor, scale: Tensor) -> Tensor:
    return x * (1 + scale.unsqueeze(1)) + shift.unsqueeze(1)


class RMSNorm(nn.Module):
    """fp32 root-mean-square norm with a learned scale, cast back to the input dtype."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return (xf * self.weight).to(x.dtype)


class AxialRope(nn.Module):
    """2-D rotary embedding over a ``grid x grid`` token lattice (adjacent-pair rotation).

    Half of each head's channels rotate with the row index, half with the column index
    (reference: ``VisionRotaryEmbeddingFast``, sihc/models/sihc/components.py:39-76).
    """

    def __init__(self, half_head_dim: int, grid: int, theta: float = 10000.0, prefix_tokens: int = 0):
        super().__init__()
        inv = 1.0 / (theta ** (torch.arange(0, half_head_dim, 2).float()[: half_head_dim // 2] / half_head_dim))
        ang = torch.arange(grid).float()[:, None] * inv[None, :]
        ang = ang.repeat_interleave(2, dim=-1)                                   # [grid, half_head_dim]
        rows = ang[:, None, :].expand(grid, grid, -1)
        cols = ang[None, :, :].expand(grid, grid, -1)
        full = torch.cat([rows, cols], dim=-1).reshape(grid * grid, -1)          # [tokens, head_dim]
        cos, sin = full.cos(), full.sin()
        if prefix_tokens:            # class-prefix tokens carry no position: identity rotation
            cos = torch.cat([torch.ones(prefix_tokens, cos.shape[-1]), cos], dim=0)
            sin = torch.cat([torch.zeros(prefix_tokens, sin.shape[-1]), sin], dim=0)
        self.register_buffer("freqs_cos", cos, persistent=False)
        self.register_buffer("freqs_sin", sin, persistent=False)

    def forward(self, x: Tensor) -> Tensor:
        cos = self.freqs_cos.to(x.device, x.dtype)
        sin = self.freqs_sin.to(x.device, x.dtype)
        pairs = x.reshape(*x.shape[:-1], -1, 2)
        rotated = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).flatten(-2)
        return x * cos + rotated * sin


class PatchStem(nn.Module):
    """Non-overlapping patch projection straight into the NHWC carrier, as one GEMM.

    Keeps the ``proj.weight`` / ``proj.bias`` keys and conv-shaped weight of the
    reference stem (``_DirectPatchEmbedGEMM``, sihc/models/sihc/sublayer.py:14-27).
    """

    def __init__(self, img_size: int, patch: int, in_chans: int, embed_dim: int):
        super().__init__()
        self.img_size, self.patch = img_size, patch
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch, stride=patch, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        b, c, h, w = x.shape
        if h != self.img_size or w != self.img_size:
            raise ValueError(f"expected image size {self.img_size}, got {(h, w)}")
        p = self.patch
        tiles = x.reshape(b, c, h // p, p, w // p, p).permute(0, 2, 4, 1, 3, 5).reshape(b, h // p, w // p, c * p * p)
        return F.linear(tiles, self.proj.weight.flatten(1), self.proj.bias)


class TimestepEmbedder(nn.Module):
    def __init__(self, hidden: int, freq_dim: int = 256):
        super().__init__()
        self.freq_dim = freq_dim
        self.mlp = nn.Sequential(nn.Linear(freq_dim, hidden), nn.SiLU(), nn.Linear(hidden, hidden))

    def forward(self, t: Tensor) -> Tensor:
        half = self.freq_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
        args = t[:, None].float() * freqs[None]
        return self.mlp(torch.cat([torch.cos(args), torch.sin(args)], dim=-1))


class LabelEmbedder(nn.Module):
    def __init__(self, num_classes: int, hidden: int):
        super().__init__()
        self.embedding_table = nn.Embedding(num_classes + 1, hidden)     # last row = null label for CFG

    def forward(self, labels: Tensor) -> Tensor:
        return self.embedding_table(labels)


class WorkspaceAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        if dim % heads:
            raise ValueError(f"dim={dim} must be divisible by num_heads={heads}")
        self.heads, self.head_dim = heads, dim // heads
        self.qkv = nn.Linear(dim, 3 * dim)
        self.q_norm = RMSNorm(self.head_dim)
        self.k_norm = RMSNorm(self.head_dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x: Tensor, rope: AxialRope) -> Tensor:
        b, n, c = x.shape
        q, k, v = self.qkv(x).reshape(b, n, 3, self.heads, self.head_dim).permute(2, 0, 3, 1, 4).unbind(0)
        q, k = rope(self.q_norm(q)), rope(self.k_norm(k))
        out = F.scaled_dot_product_attention(q, k, v)
        return self.proj(out.transpose(1, 2).reshape(b, n, c))


class SwiGLU(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        hidden = int(hidden * 2 / 3)
        self.w12 = nn.Linear(dim, 2 * hidden)
        self.w3 = nn.Linear(hidden, dim)

    def forward(self, x: Tensor) -> Tensor:
        a, b = self.w12(x).chunk(2, dim=-1)
        return self.w3(F.silu(a) * b)


class Branch(nn.Module):
    """AdaLN-modulated attention and MLP over workspace tokens (six-way modulation, gated updates)."""

    def __init__(self, hidden: int, heads: int, mlp_ratio: float):
        super().__init__()
        self.norm1 = RMSNorm(hidden)
        self.attn = WorkspaceAttention(hidden, heads)
        self.norm2 = RMSNorm(hidden)
        self.mlp = SwiGLU(hidden, int(hidden * mlp_ratio))
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden, 6 * hidden))

    def conditioning(self, cond: Tensor):
        return self.adaLN_modulation(cond).chunk(6, dim=-1)

    def attention_update(self, z: Tensor, mod, rope: AxialRope) -> Tensor:
        shift, scale, gate = mod[0], mod[1], mod[2]
        return gate.unsqueeze(1) * self.attn(_modulate(self.norm1(z), shift, scale), rope)

    def mlp_update(self, z: Tensor, mod) -> Tensor:
        shift, scale, gate = mod[3], mod[4], mod[5]
        return gate.unsqueeze(1) * self.mlp(_modulate(self.norm2(z), shift, scale))

    def forward(self, z: Tensor, cond: Tensor, rope: AxialRope) -> Tensor:
        """Whole-block update (one block-wise connection event): attention, then MLP on ``z + dz_attn``."""
        mod = self.conditioning(cond)
        dz_attn = self.attention_update(z, mod, rope)
        return dz_attn + self.mlp_update(z + dz_attn, mod)


class Connection(nn.Module):
    """Feature-wise read/write maps of one connection event: ``read_weight``, ``write_weight`` ``[C, S]``
    (reference: ``SpatiallyIndexedHyperConnection``, sihc/models/sihc/model.py:60-96)."""

    def __init__(self, hidden: int, slots: int):
        super().__init__()
        self.read_weight = nn.Parameter(torch.full((hidden, slots), 1.0 / slots))
        self.write_weight = nn.Parameter(torch.full((hidden, slots), 1.0))

    def alpha(self, dtype=None) -> Tensor:
        return self.read_weight if dtype is None else self.read_weight.to(dtype=dtype)

    def beta(self, dtype=None) -> Tensor:
        return self.write_weight if dtype is None else self.write_weight.to(dtype=dtype)


class SublayerBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, slots: int, mlp_ratio: float):
        super().__init__()
        self.attention_connection = Connection(hidden, slots)
        self.mlp_connection = Connection(hidden, slots)
        self.branch = Branch(hidden, heads, mlp_ratio)


class BlockwiseBlock(nn.Module):
    """One connection event per block (reference: ``SiHCBlock``, sihc/models/sihc/model.py:156-183)."""

    def __init__(self, hidden: int, heads: int, slots: int, mlp_ratio: float):
        super().__init__()
        self.connection = Connection(hidden, slots)
        self.branch = Branch(hidden, heads, mlp_ratio)


class FinalLayer(nn.Module):
    def __init__(self, hidden: int, patch: int, out_channels: int):
        super().__init__()
        self.norm_final = RMSNorm(hidden)
        self.linear = nn.Linear(hidden, patch * patch * out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden, 2 * hidden))

    def forward(self, x: Tensor, cond: Tensor) -> Tensor:
        shift, scale = self.adaLN_modulation(cond).chunk(2, dim=1)
        return self.linear(_modulate(self.norm_final(x), shift, scale))


class SiHC(nn.Module):
    """SiHC denoiser with the residual carrier routed by the fused CUDA operators, one fused stage at a time.

    ``frequency="sublayer"``: separate connection events around attention and MLP (2 per block; reference
    ``SublayerSiHCModel``); ``"block"``: one event per block (reference ``SiHCModel`` with the tuple
    backend, sihc/models/sihc/model.py:430-473).  ``stage_sizes`` counts blocks per stage (at most 24
    events per stage).  ``patch_size`` 8 gives n = 4 residual streams per workspace token, 4 gives n = 16.
    ``in_context_len > 0`` adds persistent class-prefix tokens that join the workspace sequence from block
    ``in_context_start`` on, have ordinary residual updates and never enter the spatial routing (reference
    ``SiHCInContextModel`` / ``SublayerSiHCInContextModel``, sihc/models/sihc/model.py:562-639,
    sihc/models/sihc/sublayer.py:75-122).
    """

    def __init__(self, input_size: int = 256, patch_size: int = 8, in_channels: int = 3, hidden_size: int = 768,
                 depth: int = 12, num_heads: int = 12, mlp_ratio: float = 4.0, num_classes: int = 1000,
                 workspace_grid: int = 16, stage_sizes: Sequence[int] | None = None, fused_stage_size: int = 12,
                 frequency: str = "sublayer", in_context_len: int = 0, in_context_start: int = 0):
        super().__init__()
        if frequency not in ("sublayer", "block"):
            raise ValueError("frequency must be 'sublayer' or 'block'")
        high = input_size // patch_size
        if input_size % patch_size or high % workspace_grid:
            raise ValueError("patch size must give a high-resolution grid divisible by the workspace grid")
        k = high // workspace_grid
        if k * k not in ops.CELLS or ops.CELLS[k * k] != (k, k):
            raise ValueError(f"unsupported cell {k}x{k}")
        stages = tuple(int(s) for s in stage_sizes) if stage_sizes is not None else (fused_stage_size,) * (depth // fused_stage_size)
        per_block = 2 if frequency == "sublayer" else 1
        if sum(stages) != depth or any(not 1 <= s * per_block <= 24 for s in stages):
            raise ValueError(f"stage sizes {stages} must give 1..24 events each and sum to depth {depth}")
        if in_context_len < 0 or (in_context_len and not 0 <= in_context_start < depth):
            raise ValueError("in_context_len must be >= 0 and in_context_start inside the depth")
        self.input_size, self.patch_size, self.in_channels, self.out_channels = input_size, patch_size, in_channels, in_channels
        self.hidden_size, self.depth, self.num_heads, self.num_classes = hidden_size, depth, num_heads, num_classes
        self.workspace_grid, self.high_grid, self.slots, self.stage_sizes = workspace_grid, high, k * k, stages
        self.frequency, self.in_context_len, self.in_context_start = frequency, int(in_context_len), int(in_context_start)
        self.t_embedder = TimestepEmbedder(hidden_size)
        self.y_embedder = LabelEmbedder(num_classes, hidden_size)
        self.x_embedder = PatchStem(input_size, patch_size, in_channels, hidden_size)
        half_head = hidden_size // num_heads // 2
        self.workspace_rope = AxialRope(half_head, workspace_grid)
        block_cls = SublayerBlock if frequency == "sublayer" else BlockwiseBlock
        self.blocks = nn.ModuleList(block_cls(hidden_size, num_heads, k * k, mlp_ratio) for _ in range(depth))
        self.final_layer = FinalLayer(hidden_size, patch_size, in_channels)
        if self.in_context_len:
            self.in_context_posemb = nn.Parameter(torch.empty(1, self.in_context_len, hidden_size))
            self.workspace_rope_incontext = AxialRope(half_head, workspace_grid, prefix_tokens=self.in_context_len)
        # "factored": one read, triangular accumulation, one write per stage (training and default).
        # "literal": write event i and read event i+1 in one pass over the carrier, no triangular step;
        # fewer bytes than the factored stage when n <= 4 (10 vs ~16 elements per event at E=24).
        self.inference_schedule = "factored"
        # "per_op": every routing operator carries its own autograd formula (traceable by torch.compile).
        # "stage": the stage-scoped backward of :mod:`.stage` - lazily transposed triangular accumulation, one
        # gamma-gradient pass per stage; eager only (a Python tape), can be captured in a CUDA graph.
        # "literal": the literal recurrence with the fused write+read step and its fused adjoint (traceable).
        self.training_schedule = "per_op"
        self.coefficients = SiHC.stage_coefficients
        self.cast_coefficients = SiHC.cast_weights
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Reference initialisation (``initialize_weights``, sihc/models/sihc/model.py:349-380):
        Xavier linears, N(0, 0.02) embedders, zero AdaLN heads and zero output projection."""
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                nn.init.zeros_(m.bias)
        nn.init.xavier_uniform_(self.x_embedder.proj.weight.data.view(self.hidden_size, -1))
        nn.init.zeros_(self.x_embedder.proj.bias)
        nn.init.normal_(self.y_embedder.embedding_table.weight, std=0.02)
        nn.init.normal_(self.t_embedder.mlp[0].weight, std=0.02)
        nn.init.normal_(self.t_embedder.mlp[2].weight, std=0.02)
        for block in self.blocks:
            nn.init.zeros_(block.branch.adaLN_modulation[-1].weight)
            nn.init.zeros_(block.branch.adaLN_modulation[-1].bias)
        nn.init.zeros_(self.final_layer.adaLN_modulation[-1].weight)
        nn.init.zeros_(self.final_layer.adaLN_modulation[-1].bias)
        nn.init.zeros_(self.final_layer.linear.weight)
        nn.init.zeros_(self.final_layer.linear.bias)
        if self.in_context_len:
            nn.init.normal_(self.in_context_posemb, std=0.02)

    def connections(self, block) -> list:
        return [block.attention_connection, block.mlp_connection] if self.frequency == "sublayer" else [block.connection]

    @torch.no_grad()
    def open_gates(self, std: float = 0.01) -> None:
        """Give the zero-initialised heads small random values so every update ``dz`` is non-zero
        (the reference's tests and benchmark do the same; zero heads make timing and parity vacuous:
        research/tests/test_sublayer_kernels.py:229-242, sihc/bench/fusion_controls.py:114-117)."""
        for block in self.blocks:
            block.branch.adaLN_modulation[-1].weight.normal_(std=std)
            block.branch.adaLN_modulation[-1].bias.normal_(std=3 * std)
            for conn in self.connections(block):
                conn.read_weight.add_(torch.randn_like(conn.read_weight) * std)
                conn.write_weight.add_(torch.randn_like(conn.write_weight) * 2 * std)
        self.final_layer.linear.weight.normal_(std=3 * std)

    def unpatchify(self, x: Tensor) -> Tensor:
        b, n, _ = x.shape
        h, p, c = self.high_grid, self.patch_size, self.out_channels
        return x.reshape(b, h, h, p, p, c).permute(0, 5, 1, 3, 2, 4).reshape(b, c, h * p, h * p)

    # ---- the hot path's caller -----------------------------------------------------------------
    @staticmethod
    def stage_coefficients(read_weights: Sequence[Tensor], write_weights: Sequence[Tensor], dtype: torch.dtype):
        """``alpha, beta [E,C,S]`` in the carrier dtype and ``gamma[i,j,c] = sum_s alpha_i[c,s] beta_j[c,s]`` from the
        stage's fp32 parameters (reference: sihc/models/sihc/sublayer.py:57-60).  A few dozen tiny torch kernels
        with their autograd; a training step may swap in a compiled version through ``self.coefficients``."""
        alpha = torch.stack([w.to(dtype=dtype) for w in read_weights]).contiguous()
        beta = torch.stack([w.to(dtype=dtype) for w in write_weights]).contiguous()
        gamma = (alpha[:, None] * beta[None, :]).sum(dim=-1)
        return alpha, beta, gamma

    def stage_events(self, blocks: Sequence[nn.Module], cond: Tensor, stage_start: int) -> list:
        """The connection events of a stage, in order: ``(connection, update, uses_context)`` where
        ``update(seq, rope)`` is the gated sublayer (or whole-block) update of a token sequence."""
        events = []
        mods: dict = {}

        def modulation(block):
            # Computed when the block's first event runs (as the reference's loop does, sihc/models/sihc/sublayer.py:63),
            # not when the event list is built: autograd runs backward nodes in reverse creation order, so a modulation
            # created up front would get its gradient - and its 6C x C weight gradient - only at the very end of the
            # stage's (or, in the literal schedule, the model's) backward, where nothing is left to overlap its
            # all-reduce with.
            if id(block) not in mods:
                mods[id(block)] = block.branch.conditioning(cond)
            return mods[id(block)]

        for i, block in enumerate(blocks):
            ctx = bool(self.in_context_len) and stage_start + i >= self.in_context_start
            if self.frequency == "sublayer":
                events.append((block.attention_connection,
                               lambda seq, rope, b=block: b.branch.attention_update(seq, modulation(b), rope), ctx))
                events.append((block.mlp_connection,
                               lambda seq, rope, b=block: b.branch.mlp_update(seq, modulation(b)), ctx))
            else:
                events.append((block.connection, lambda seq, rope, b=block: b.branch(seq, cond, rope), ctx))
        return events

    def apply_update(self, update, z: Tensor, context: Tensor | None, uses_context: bool):
        """Run one event's sublayer on ``z`` (with the class-prefix tokens in front when they are active);
        returns the packed spatial update and the new prefix tokens."""
        if uses_context:
            dseq = update(torch.cat((context, z), dim=1), self.workspace_rope_incontext)
            n = self.in_context_len
            # dropping the prefix gives a batch-strided view: the routing operators need it packed
            return dseq[:, n:].contiguous(), context + dseq[:, :n]
        return update(z, self.workspace_rope).contiguous(), context

    def run_stage(self, x0: Tensor, cond: Tensor, blocks: Sequence[nn.Module], stage_start: int = 0,
                  context: Tensor | None = None):
        """One fused stage (reference: ``_run_fused_schedule_stage``, sihc/models/sihc/sublayer.py:52-72, :84-122;
        block-wise sihc/models/sihc/model.py:430-473, :588-639).  Returns ``(carrier, context)``."""
        events = self.stage_events(blocks, cond, stage_start)
        alpha, beta, gamma = self.coefficients(tuple(c.read_weight for c, _, _ in events),
                                               tuple(c.write_weight for c, _, _ in events), x0.dtype)
        if self.training_schedule == "stage":
            state = [context]

            def sublayer(update, uses_context):
                def run(z):
                    dz, state[0] = self.apply_update(update, z, state[0], uses_context)
                    return dz
                return run

            out = stage.run_stage(x0, alpha, beta, [sublayer(u, c) for _, u, c in events], gamma=gamma)
            return out, state[0]
        base = ops.sublayer_read(x0, alpha)
        updates: list[Tensor] = []
        for e, (_, update, uses_context) in enumerate(events):
            z = base[e] if e == 0 else ops.sublayer_triangular(base[e], updates, gamma[e, :e].contiguous())
            dz, context = self.apply_update(update, z, context, uses_context)
            updates.append(dz)
        return ops.sublayer_write(x0, updates, beta), context

    @staticmethod
    def cast_weights(read_weights: Sequence[Tensor], write_weights: Sequence[Tensor], dtype: torch.dtype):
        """``alpha, beta [N,C,S]``: every event's read / write weights in the carrier dtype, stacked (two tiny
        kernels instead of two casts per event; a training step may swap in a compiled version)."""
        return (torch.stack([w.to(dtype=dtype) for w in read_weights]).contiguous(),
                torch.stack([w.to(dtype=dtype) for w in write_weights]).contiguous())

    def run_literal(self, carrier: Tensor, cond: Tensor, context: Tensor | None = None) -> Tensor:
        """All events with the literal recurrence (reference definition: ``literal_forward``,
        research/tests/test_sublayer_kernels.py:216-226), each write fused with the next event's read:
        2S+2 elements per event forward and, through the fused adjoint of that step, 3S+3 backward - fewer bytes than
        the factored stage when S <= 4 and a stage has many events.  The carrier is rounded to its storage dtype after
        every event, exactly as the unfused path rounds it."""
        events, start = [], 0
        for size in self.stage_sizes:
            events += self.stage_events(self.blocks[start:start + size], cond, start)
            start += size
        alpha, beta = self.cast_coefficients(tuple(c.read_weight for c, _, _ in events),
                                             tuple(c.write_weight for c, _, _ in events), carrier.dtype)
        z = ops.sihc_read(carrier, alpha[0])
        for i, (_, update, uses_context) in enumerate(events):
            dz, context = self.apply_update(update, z, context, uses_context)
            if i + 1 < len(events):
                carrier, z = ops.sihc_write_read(carrier, dz, beta[i], alpha[i + 1])
            else:
                carrier = ops.sihc_write(carrier, dz, beta[i])
        return carrier

    def initial_context(self, y_emb: Tensor, dtype) -> Tensor | None:
        if not self.in_context_len:
            return None
        return (y_emb.unsqueeze(1).expand(-1, self.in_context_len, -1) + self.in_context_posemb).to(dtype=dtype)

    def forward(self, x: Tensor, t: Tensor, y: Tensor) -> Tensor:
        y_emb = self.y_embedder(y)
        cond = self.t_embedder(t) + y_emb
        carrier = self.x_embedder(x)
        context = self.initial_context(y_emb, carrier.dtype)
        literal = self.training_schedule == "literal" if torch.is_grad_enabled() else self.inference_schedule == "literal"
        if literal:
            carrier = self.run_literal(carrier, cond, context)
        else:
            start = 0
            for size in self.stage_sizes:
                carrier, context = self.run_stage(carrier, cond, self.blocks[start:start + size], start, context)
                start += size
        b, hh, ww, c = carrier.shape
        return self.unpatchify(self.final_layer(carrier.reshape(b, hh * ww, c), cond))


class SublayerSiHC(SiHC):
    """Sublayer-wise SiHC (two connection events per block)."""

    def __init__(self, **kw):
        kw.setdefault("frequency", "sublayer")
        super().__init__(**kw)


class BlockwiseSiHC(SiHC):
    """Block-wise SiHC (one connection event per block)."""

    def __init__(self, **kw):
        kw.setdefault("frequency", "block")
        super().__init__(**kw)


def sihc_b(**kw) -> SublayerSiHC:
    """SiHC-B: 12 blocks, width 768, 12 heads, patch 8 (n = 4), one stage of 24 events
    (reference preset ``sihc_sublayer_1x12_d768_b8``, sihc/models/sihc/sublayer.py:148-150)."""
    cfg = dict(patch_size=8, hidden_size=768, depth=12, num_heads=12, stage_sizes=(12,))
    cfg.update(kw)
    return SublayerSiHC(**cfg)


def sihc_xl(**kw) -> SublayerSiHC:
    """SiHC-XL as configured by the benchmark: 28 blocks, width 1152, 16 heads, patch 8 (n = 4),
    stages of 8 + 12 + 8 blocks (16, 24, 16 events)."""
    cfg = dict(patch_size=8, hidden_size=1152, depth=28, num_heads=16, stage_sizes=(8, 12, 8))
    cfg.update(kw)
    return SublayerSiHC(**cfg)


# ---- flow-matching objective and sampler used by the model-level benchmarks ------------------------
def velocity_training_batch(x: Tensor, generator: torch.Generator | None = None):
    """Noisy input, timestep and velocity target as in the reference trainer
    (sihc/training/train.py:623-628): ``t ~ sigmoid(N(-0.8, 0.8))``, ``z = t x + (1-t) e``,
    ``v = (x - z) / max(1 - t, 0.05)``."""
    b = x.shape[0]
    t = torch.sigmoid(torch.randn(b, device=x.device, generator=generator) * 0.8 - 0.8)
    e = torch.randn(x.shape, device=x.device, dtype=x.dtype, generator=generator)
    tt = t.view(b, 1, 1, 1)
    z = tt * x + (1 - tt) * e
    v = (x - z) / (1 - tt).clamp_min(0.05)
    return z, t, v


@torch.no_grad()
def cfg_velocity(model, z, t, labels, *, num_classes, cfg_scale, interval):
    """Classifier-free guidance on a guidance interval (reference: ``cfg_velocity``, sihc/sampling.py:20-29):
    two separate forwards (conditional, null label) whenever ``cfg_scale != 1``."""
    # clone(): a model compiled with CUDA graphs may reuse its output buffer on the next call, and both
    # evaluations must be alive at once (same precaution as the reference, sihc/sampling.py:8-11)
    v_cond = model(z, t.flatten(), labels).clone()
    if cfg_scale == 1.0:
        return v_cond
    v_null = model(z, t.flatten(), torch.full_like(labels, num_classes)).clone()
    low, high = interval
    mask = (t < high) & ((low == 0) | (t > low))
    scale = torch.where(mask, torch.full_like(t, cfg_scale), torch.ones_like(t))
    return v_null + scale * (v_cond - v_null)


@torch.no_grad()
def sample_heun(model, labels, *, image_size=256, steps=50, cfg_scale=1.0, interval=(0.0, 1.0), num_classes=1000,
                generator: torch.Generator | None = None):
    """Heun sampler for a velocity-predicting model (reference: ``sample_heun``, sihc/sampling.py:32-62):
    ``steps - 1`` Heun steps and a final Euler step, i.e. ``2*steps - 1`` guided evaluations."""
    b, dev = labels.numel(), labels.device
    z = torch.randn(b, 3, image_size, image_size, device=dev, generator=generator)
    ts = torch.linspace(0.0, 1.0, steps + 1, device=dev)
    kw = dict(num_classes=num_classes, cfg_scale=cfg_scale, interval=interval)
    for i in range(steps - 1):
        t = torch.full((b, 1, 1, 1), float(ts[i]), device=dev)
        tn = torch.full((b, 1, 1, 1), float(ts[i + 1]), device=dev)
        v = cfg_velocity(model, z, t, labels, **kw)
        v_next = cfg_velocity(model, z + (tn - t) * v, tn, labels, **kw)
        z = z + (tn - t) * 0.5 * (v + v_next)
    t = torch.full((b, 1, 1, 1), float(ts[-2]), device=dev)
    tn = torch.full((b, 1, 1, 1), float(ts[-1]), device=dev)
    return z + (tn - t) * cfg_velocity(model, z, t, labels, **kw)
