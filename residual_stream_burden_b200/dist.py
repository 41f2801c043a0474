"""Data-parallel plumbing for the routing path.

The path shards by batch with no forward exchange; the only cross-rank quantity is the
gradient of the connection weights (``read_weight`` / ``write_weight``: 2*C*S floats per
connection event, 2 MB for the largest model here).  Under ``DistributedDataParallel`` those
gradients ride in the ordinary buckets (reference: sihc/training/train.py:515-523).  For
callers that drive the operators directly, :func:`allreduce_weight_grads` packs any number of
small gradient tensors into one flat fp32 buffer and issues a single all-reduce, so the exchange
costs one collective launch regardless of the number of events.  :class:`BucketedGradExchange` averages the
gradients of a whole model bucket by bucket while the backward pass is still running.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
from torch import Tensor


def shard_batch(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous ``[start, stop)`` range of images owned by ``rank`` (remainder to the low ranks)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allreduce_weight_grads(grads: Sequence[Tensor], group=None, average: bool = True) -> None:
    """Sum (or average) the given gradient tensors over the process group, in place, with ONE collective."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    if not grads:
        return
    world = dist.get_world_size(group)
    if len(grads) == 1 and grads[0].is_contiguous() and grads[0].dtype == torch.float32:
        # already one flat fp32 buffer (the kernels can write both gradients into it): reduce it where it lies
        flat = grads[0].detach()
        dist.all_reduce(flat, group=group)
        if average:
            flat /= world
        return
    flat = torch.cat([g.detach().reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for g in grads:
        n = g.numel()
        g.detach().copy_(flat[offset:offset + n].view_as(g))
        offset += n


def observe_ready_order(params: Sequence[torch.nn.Parameter], run_backward) -> list:
    """The parameters in the order their gradients are accumulated when ``run_backward()`` runs one backward pass
    (parameters that received no gradient come last, in reverse registration order).  Deterministic for a fixed
    model and schedule, so every rank derives the same order.  The caller clears the gradients afterwards."""
    params = [p for p in params if p.requires_grad]
    order: list = []
    handles = [p.register_post_accumulate_grad_hook(order.append) for p in params]
    try:
        run_backward()
    finally:
        for h in handles:
            h.remove()
    seen = {id(p) for p in order}
    return order + [p for p in reversed(params) if id(p) not in seen]


class BucketedGradExchange:
    """Data-parallel gradient averaging that runs UNDER the backward pass instead of after it.

    The parameters are grouped into buckets in the order their gradients become final during backward: the order
    observed in a real backward pass (:func:`observe_ready_order`, ``ready_order=True``) or, failing that, the reverse
    of the order in which the model registered them.  The observed order matters: the small connection weights of a
    SiHC stage, for instance, are registered with their blocks but receive their gradients only when the backward of
    the whole stage (or, in the literal schedule, of the whole model) has finished, and a bucket cannot be reduced
    before its last gradient - with registration order every bucket would wait for the very end of backward.
    A hook on every parameter counts its bucket down;
    when a bucket's last gradient has been accumulated its all-reduce is issued at once on a side stream, so it
    overlaps the backward kernels of the layers below.  :meth:`finish` makes the calling stream wait for all of
    them.  This is the role ``DistributedDataParallel`` plays in the reference trainer
    (sihc/training/train.py:515-523) - same arithmetic (mean over ranks, fp32) - built here so that it also works
    when the backward pass is a sequence of eager autograd nodes captured into one CUDA graph.

    Two ways of presenting a bucket to the collective:
      * ``in_place=True``: the large gradient tensors are reduced where they lie, all in ONE coalesced call
        (one collective launch per bucket, no packing copy); only the many small tensors (norm scales, biases,
        the connection weights) are packed into one flat buffer and copied back;
      * ``in_place=False``: every gradient of the bucket is packed into one flat buffer (two extra passes over
        the gradients).
    With a single rank the hooks still fire (so the bookkeeping is exercised) and the collectives are skipped
    unless ``force`` is set.
    """

    def __init__(self, params: Sequence[torch.nn.Parameter], group=None, bucket_bytes: int = 256 << 20,
                 in_place: bool = True, small_numel: int = 1 << 16, comm_stream=None, force: bool = False,
                 on_bucket_reduced=None, ready_order: bool = False, tail_buckets: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.active = self.world > 1 or (force and dist.is_available() and dist.is_initialized())
        self.in_place, self.small_numel = in_place, small_numel
        self.on_bucket_reduced = on_bucket_reduced
        params = [p for p in params if p.requires_grad]
        ordered = list(params if ready_order else reversed(params))      # the order the gradients become ready
        # Buckets are cut from the END of that order: the last bucket's all-reduce (and update) cannot hide behind
        # any backward work, so the last two buckets are kept small (1/16 and 1/4 of the regular size).
        caps = [max(bucket_bytes // 16, 1), max(bucket_bytes // 4, 1)]
        self.buckets: list[list[torch.nn.Parameter]] = []
        current, size = [], 0
        for p in reversed(ordered):
            current.append(p)
            size += p.numel() * p.element_size()
            cap = caps[len(self.buckets)] if len(self.buckets) < len(caps) and tail_buckets else bucket_bytes
            if size >= cap:
                self.buckets.append(current[::-1])
                current, size = [], 0
        if current:
            self.buckets.append(current[::-1])
        self.buckets.reverse()
        self._bucket_of = {id(p): k for k, bucket in enumerate(self.buckets) for p in bucket}
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._handles = []
        self.cuda = bool(params) and params[0].is_cuda
        self.comm_stream = comm_stream if comm_stream is not None else (torch.cuda.Stream() if self.cuda else None)
        backend = dist.get_backend(group) if self.active else None
        self._avg_op = dist.ReduceOp.AVG if backend == "nccl" else dist.ReduceOp.SUM
        self._divide = self.active and backend != "nccl"
        for p in params:
            self._handles.append(p.register_post_accumulate_grad_hook(self._hook))
        self.begin()

    # ---- per step ---------------------------------------------------------------------------------------
    def begin(self) -> None:
        """Call before every backward pass."""
        self._pending = [len(b) for b in self.buckets]
        self._launched = [False] * len(self.buckets)

    def finish(self) -> None:
        """Call after backward: reduces buckets whose hooks did not all fire (parameters without a gradient this
        step) and makes the current stream wait for every all-reduce."""
        for k, done in enumerate(self._launched):
            if not done:
                self._reduce(k)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    # ---- internals --------------------------------------------------------------------------------------
    def _hook(self, param) -> None:
        k = self._bucket_of[id(param)]
        self._pending[k] -= 1
        if self._pending[k] == 0 and not self._launched[k]:
            self._reduce(k)

    def _reduce(self, k: int) -> None:
        self._launched[k] = True
        grads = [p.grad for p in self.buckets[k] if p.grad is not None]
        if self.cuda:
            # the gradients were produced on the stream this hook runs on: order the side stream after it
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self._reduce_on_current_stream(k, grads)
        else:
            self._reduce_on_current_stream(k, grads)

    def _reduce_on_current_stream(self, k: int, grads) -> None:
        if self.active and grads:
            if self.in_place:
                large = [g for g in grads if g.numel() >= self.small_numel and g.is_contiguous()]
                small = [g for g in grads if not (g.numel() >= self.small_numel and g.is_contiguous())]
            else:
                large, small = [], list(grads)
            flat = torch.cat([g.reshape(-1) for g in small]) if small else None
            tensors = large + ([flat] if flat is not None else [])
            if len(tensors) == 1:
                dist.all_reduce(tensors[0], op=self._avg_op, group=self.group)
            else:
                with dist._coalescing_manager(group=self.group):        # one collective launch for the bucket
                    for t in tensors:
                        dist.all_reduce(t, op=self._avg_op, group=self.group)
            if self._divide:
                torch._foreach_div_(tensors, float(self.world))
            if flat is not None:
                torch._foreach_copy_(small, [v.view_as(g) for v, g in zip(flat.split([g.numel() for g in small]), small)])
        if self.on_bucket_reduced is not None:
            self.on_bucket_reduced(k)


class ShardedGradExchange(BucketedGradExchange):
    """:class:`BucketedGradExchange` with the update sharded over the ranks (optimizer-state sharding).

    For every large gradient tensor of a bucket the all-reduce is replaced by its two halves with the update in
    between: reduce-scatter (in place: rank r ends up with the mean of slice r), the optimizer step on that slice only
    (``on_bucket_reduced``), all-gather of the updated parameter slices (in place).  The bytes crossing NVLink are those
    of the all-reduce, but each rank runs the optimizer - a pass over four fp32 arrays per parameter, bound by device
    memory bandwidth and competing with the backward pass for it - on 1/N of the elements, and keeps 1/N of the
    optimizer state.  No flat copies: gradients and parameters are reduced and gathered where they lie.  Tensors that
    are small, not contiguous or not divisible by the number of ranks keep the all-reduce and are updated in full on
    every rank.  With a single rank the slices are the whole tensors and no collective runs.

    ``update_tensors(k)`` gives, for bucket k, the tensors the caller's optimizer must own (parameter slices and whole
    small parameters); :meth:`attach_grads` points their ``.grad`` at this step's gradients before the optimizer runs.
    """

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.rank = dist.get_rank(self.group) if self.world > 1 else 0
        backend = dist.get_backend(self.group) if self.active else None
        self._native_scatter = backend == "nccl"          # gloo has no reduce-scatter: all-reduce and keep the slice
        self._sharded, self._whole, self._slices = [], [], []
        for bucket in self.buckets:
            sharded = [p for p in bucket if p.numel() >= self.small_numel and p.numel() % self.world == 0
                       and p.data.is_contiguous()]
            ids = {id(p) for p in sharded}
            self._sharded.append(sharded)
            self._whole.append([p for p in bucket if id(p) not in ids])
            n = [p.numel() // self.world for p in sharded]
            self._slices.append([p.data.view(-1)[self.rank * m:(self.rank + 1) * m] for p, m in zip(sharded, n)])

    def update_tensors(self, k: int) -> list:
        return list(self._slices[k]) + list(self._whole[k])

    def attach_grads(self, k: int) -> None:
        for p, piece in zip(self._sharded[k], self._slices[k]):
            m = piece.numel()
            piece.grad = None if p.grad is None else p.grad.view(-1)[self.rank * m:(self.rank + 1) * m]

    def _reduce_on_current_stream(self, k: int, grads) -> None:
        sharded = [p for p in self._sharded[k] if p.grad is not None]
        for p in sharded:
            if not p.grad.is_contiguous():
                p.grad = p.grad.contiguous()
        whole = [p.grad for p in self._whole[k] if p.grad is not None]
        if self.active:
            flats = [p.grad.view(-1) for p in sharded]
            if self._native_scatter and flats:
                with dist._coalescing_manager(group=self.group):
                    for g in flats:
                        m = g.numel() // self.world
                        dist.reduce_scatter_tensor(g[self.rank * m:(self.rank + 1) * m], g, op=self._avg_op, group=self.group)
            elif flats:
                with dist._coalescing_manager(group=self.group):
                    for g in flats:
                        dist.all_reduce(g, op=self._avg_op, group=self.group)
                if self._divide:
                    torch._foreach_div_(flats, float(self.world))
            if whole:
                flat = torch.cat([g.reshape(-1) for g in whole])
                dist.all_reduce(flat, op=self._avg_op, group=self.group)
                if self._divide:
                    flat /= float(self.world)
                torch._foreach_copy_(whole, [v.view_as(g) for v, g in zip(flat.split([g.numel() for g in whole]), whole)])
        self.attach_grads(k)
        if self.on_bucket_reduced is not None:
            self.on_bucket_reduced(k)
        if self.active and sharded:
            with dist._coalescing_manager(group=self.group):
                for p in sharded:
                    d = p.data.view(-1)
                    m = d.numel() // self.world
                    dist.all_gather_into_tensor(d, d[self.rank * m:(self.rank + 1) * m], group=self.group)
