"""One data-parallel training step of a SiHC model as a single CUDA graph.

The reference trainer compiles the whole model with ``torch.compile(mode="reduce-overhead")`` and wraps it in
``DistributedDataParallel`` (sihc/training/train.py:507-523, step loop :589-697).  The compiled backward is then ONE
autograd node: every gradient becomes ready at its very end, so the gradient all-reduce of the whole model
(2.7 GB of fp32 for the 28 x 1152 model) runs after backward with nothing to hide behind, and the routing
operators must carry per-operator autograd formulas that a tracing compiler can see through.

Here the step is built from streams and one hand-captured graph instead:

  * the model's stages run eagerly from Python with the stage-scoped backward of :mod:`.stage` (lazily
    transposed triangular accumulation, one gamma-gradient pass per stage); only the torch sublayers between the
    routing operators are compiled, ONE compilation per kind of sublayer shared by all blocks;
  * backward is therefore a chain of fine-grained autograd nodes, and :class:`.dist.BucketedGradExchange` issues
    each bucket's all-reduce on a side stream the moment its last gradient lands, under the backward kernels of
    the layers below; optionally the fused AdamW update of a bucket follows its all-reduce on that side stream;
  * forward, loss, backward, the collectives and the optimizer are captured once into a single CUDA graph
    (the cross-stream dependencies become graph edges) and replayed every step: no per-step launch overhead,
    no tracing compiler around the routing path.

Arithmetic is the reference's: bf16 autocast over fp32 master parameters, mean-squared velocity error with
``t ~ sigmoid(N(-0.8, 0.8))`` (:623-628), gradients averaged over ranks in fp32, fused AdamW with betas (0.9, 0.95).
"""

from __future__ import annotations

import functools
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .dist import BucketedGradExchange, ShardedGradExchange, observe_ready_order
from .model import Branch, SiHC, velocity_training_batch


@functools.lru_cache(maxsize=None)
def _compiled_sublayers():
    """The torch sublayers as functions of (module, inputs), compiled once and shared by every block: the
    compiler treats the module's parameters as graph inputs, so blocks of the same shape reuse the same code."""
    import torch._dynamo
    torch._dynamo.config.recompile_limit = max(getattr(torch._dynamo.config, "recompile_limit", 8), 64)
    opts = dict(fullgraph=True, dynamic=False)
    return (torch.compile(Branch.attention_update, **opts), torch.compile(Branch.mlp_update, **opts),
            torch.compile(Branch.forward, **opts))


def compile_sublayers(model: SiHC) -> SiHC:
    """Route every block's attention / MLP update (and the whole-block update of block-wise models) through the
    shared compiled functions.  The routing operators stay outside: they are this package's CUDA kernels."""
    attn, mlp, whole = _compiled_sublayers()
    for block in model.blocks:
        branch = block.branch
        branch.attention_update = functools.partial(attn, branch)
        branch.mlp_update = functools.partial(mlp, branch)
        branch.forward = functools.partial(whole, branch)
    model.final_layer.forward = torch.compile(model.final_layer.forward, fullgraph=True, dynamic=False)
    # casts, stacking and the gamma products of a stage's connection weights: one small compiled graph per stage
    # size instead of a few dozen tiny kernels (and as many again in backward)
    model.coefficients = torch.compile(SiHC.stage_coefficients, fullgraph=True, dynamic=False)
    model.cast_coefficients = torch.compile(SiHC.cast_weights, fullgraph=True, dynamic=False)
    return model


class TrainStep:
    """``step(images_host, labels) -> loss`` for a :class:`SiHC` model on the current CUDA device.

    ``group`` is the data-parallel process group (``None``: single GPU, unless a default group exists and
    ``force_exchange`` asks for its collectives anyway).  ``bucket_mb`` sizes the gradient buckets;
    ``overlap_optimizer`` runs each bucket's AdamW update on the side stream right after its all-reduce instead of
    one update after backward.  ``use_graph=False`` runs the same step eagerly (for tests and debugging).
    ``schedule``: ``"stage"`` = the reference's factored stages with the stage-scoped backward; ``"literal"`` = the
    literal recurrence with the fused write+read step and its fused adjoint (fewer bytes when n <= 4).
    ``shard_optimizer`` (with ``overlap_optimizer``): each rank updates 1/N of every large parameter between a
    reduce-scatter of its gradient and an all-gather of the result (:class:`.dist.ShardedGradExchange`).
    """

    def __init__(self, model: SiHC, batch: int, *, lr: float = 2e-4, betas=(0.9, 0.95), weight_decay: float = 0.0,
                 group=None, bucket_mb: float = 256, in_place_exchange: bool = True, overlap_optimizer: bool = False,
                 compile_model: bool = True, use_graph: bool = True, force_exchange: bool = False, warmup: int = 3,
                 schedule: str = "stage", shard_optimizer: bool = True):
        device = next(model.parameters()).device
        if device.type != "cuda":
            raise ValueError("TrainStep needs the model on a CUDA device")
        self.model, self.device, self.use_graph = model, device, use_graph
        if schedule not in ("stage", "literal"):
            raise ValueError("schedule must be 'stage' (factored stages, stage-scoped backward) or 'literal'")
        model.train()
        model.training_schedule = schedule
        if compile_model:
            compile_sublayers(model)
        self.stream = torch.cuda.Stream(device)
        self.images = torch.zeros(batch, model.in_channels, model.input_size, model.input_size, device=device)
        self.labels = torch.zeros(batch, dtype=torch.long, device=device)
        self.loss = torch.zeros((), device=device)
        # The gradient buckets and the optimizer(s) are built at the first step, after one probe backward pass has
        # shown the order in which the gradients become ready (see _setup).
        self._exchange_kw = dict(group=group, bucket_bytes=int(bucket_mb * (1 << 20)), in_place=in_place_exchange,
                                 force=force_exchange)
        self._opt_kw = dict(lr=lr, betas=betas, weight_decay=weight_decay, fused=True, capturable=use_graph)
        self._overlap_optimizer = overlap_optimizer
        self._shard_optimizer = shard_optimizer
        self.exchange: Optional[BucketedGradExchange] = None
        self.bucket_optimizers = None
        self.optimizer = None
        self._ready = False
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._warmup_left = max(int(warmup), 1 if use_graph else 0)

    # ---- the step body (runs eagerly during warm-up, once more under capture, never again after) -------------
    def _setup(self) -> None:
        """One probe forward + backward on the staged inputs (no update) to observe the order in which the gradients
        become ready; then the buckets follow that order and the optimizers are created."""
        params = [p for p in self.model.parameters() if p.requires_grad]

        def probe():
            z, t, v = velocity_training_batch(self.images)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                pred = self.model(z, t, self.labels)
            (pred.float() - v).square().mean().backward()

        order = observe_ready_order(params, probe)
        self._zero_grad()
        distributed = dist.is_available() and dist.is_initialized()
        if self._overlap_optimizer and self._shard_optimizer:
            # reduce-scatter -> update of this rank's slices -> all-gather, bucket by bucket on the side stream
            self.exchange = ShardedGradExchange(order, ready_order=True, on_bucket_reduced=self._bucket_ready,
                                                **self._exchange_kw)
            self.bucket_optimizers = [torch.optim.AdamW(self.exchange.update_tensors(k), **self._opt_kw)
                                      for k in range(len(self.exchange.buckets))]
        elif distributed or self._overlap_optimizer:
            self.exchange = BucketedGradExchange(order, ready_order=True,
                                                 on_bucket_reduced=self._bucket_ready if self._overlap_optimizer else None,
                                                 **self._exchange_kw)
            if self._overlap_optimizer:
                self.bucket_optimizers = [torch.optim.AdamW(bucket, **self._opt_kw) for bucket in self.exchange.buckets]
        if not self._overlap_optimizer:
            self.optimizer = torch.optim.AdamW(params, **self._opt_kw)
        self._ready = True

    def _bucket_ready(self, k: int) -> None:
        self.bucket_optimizers[k].step()           # on the side stream, right behind the bucket's all-reduce

    def _body(self) -> None:
        z, t, v = velocity_training_batch(self.images)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            pred = self.model(z, t, self.labels)
        loss = (pred.float() - v).square().mean()
        if self.exchange is not None:
            self.exchange.begin()
        loss.backward()
        if self.exchange is not None:
            self.exchange.finish()
        if self.optimizer is not None:
            self.optimizer.step()
        self.loss.copy_(loss.detach())

    def _zero_grad(self) -> None:
        for p in self.model.parameters():
            p.grad = None
        if isinstance(self.exchange, ShardedGradExchange):
            for k in range(len(self.exchange.buckets)):
                for piece in self.exchange._slices[k]:
                    piece.grad = None

    def _capture(self) -> None:
        self._zero_grad()                          # backward allocates the gradients inside the graph's pool
        self.graph = torch.cuda.CUDAGraph()
        # thread_local: the autograd worker thread and the collective library's own threads keep working while
        # this thread captures; only this thread's unsafe calls would abort the capture
        with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
            self._body()

    # ---- public -------------------------------------------------------------------------------------------
    def load(self, images_host: Tensor, labels: Tensor) -> None:
        """Stage this step's inputs (pinned host images are copied asynchronously)."""
        self.images.copy_(images_host, non_blocking=True)
        self.labels.copy_(labels, non_blocking=True)

    def run(self) -> Tensor:
        """Run one step on the staged inputs; returns the loss as a 0-d device tensor (no host sync)."""
        if self._warmup_left > 0 or not self.use_graph:
            self._warmup_left -= 1
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                if not self._ready:
                    self._setup()
                self._body()
                self._zero_grad()
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            return self.loss
        if self.graph is None:
            self._capture()
        self.graph.replay()
        return self.loss

    def step(self, images_host: Tensor, labels: Tensor) -> Tensor:
        self.load(images_host, labels)
        return self.run()

    def close(self) -> None:
        """Destroy the captured graph and detach the gradient hooks.

        Call this before the process group is destroyed: a communicator whose collectives were captured waits, when
        it is torn down, until every graph that holds them is gone, so a graph kept alive past
        ``destroy_process_group()`` (for instance by a reference cycle) blocks the exit of the process.
        """
        torch.cuda.synchronize(self.device)
        if self.graph is not None:
            self.graph.reset()
            self.graph = None
        if self.exchange is not None:
            self.exchange.remove()
            self.exchange.on_bucket_reduced = None       # breaks the trainer <-> exchange reference cycle
        self._warmup_left = 1 << 30                      # any later step runs eagerly

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
