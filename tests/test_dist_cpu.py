"""The multi-rank part of the path on CPU: two gloo ranks shard a batch, compute the weight gradient of
their shard with the oracle, exchange it with ``allreduce_weight_grads`` and must reproduce the full-batch
gradient; a rank that fails before the exchange makes the other rank's collective end with an error
instead of hanging (host-side failure, short timeout)."""

import datetime
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sihc_oracle as O


def _worker(rank, world, port, tmp, fail):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from residual_stream_burden_b200.dist import allreduce_weight_grads, shard_batch
    try:
        torch.manual_seed(0)                                   # same full batch on every rank
        x = torch.randn(6, 8, 8, 16)
        alpha = 0.25 + 0.02 * torch.randn(2, 16, 4)
        g = [torch.randn(6, 16, 16) for _ in range(2)]
        lo, hi = shard_batch(6, rank, world)
        if fail and rank == 1:
            raise RuntimeError("injected host-side failure before the exchange")
        _, dalpha = O.read_backward(x[lo:hi], [t[lo:hi] for t in g], alpha)
        parts = [dalpha[0].clone(), dalpha[1].clone()]
        allreduce_weight_grads(parts, average=False)
        _, full = O.read_backward(x, g, alpha)
        torch.testing.assert_close(torch.stack(parts), full, atol=1e-5, rtol=1e-5)
        # one flat fp32 buffer (what the benchmark's kernels write into) is reduced where it lies, as a mean
        flat = dalpha.clone().float().contiguous()
        where = flat.data_ptr()
        allreduce_weight_grads([flat])
        assert flat.data_ptr() == where
        torch.testing.assert_close(flat, full / world, atol=1e-5, rtol=1e-5)
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    except Exception as exc:                                   # noqa: BLE001
        open(os.path.join(tmp, f"err{rank}"), "w").write(repr(exc))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                                      # noqa: BLE001
            pass


def _port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_reproduce_full_batch_weight_gradient(tmp_path):
    mp.spawn(_worker, args=(2, _port(), str(tmp_path), False), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists(), list(tmp_path.iterdir())


def test_rank_failure_surfaces_as_error_not_hang(tmp_path):
    mp.spawn(_worker, args=(2, _port(), str(tmp_path), True), nprocs=2, join=True)
    assert (tmp_path / "err1").exists()
    assert (tmp_path / "err0").exists() and not (tmp_path / "ok0").exists()   # rank 0's all-reduce raised


def test_shard_batch_partitions_exactly():
    from residual_stream_burden_b200.dist import shard_batch
    for batch in (1, 7, 32, 255):
        for world in (1, 2, 4, 8):
            spans = [shard_batch(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def _bucket_worker(rank, world, port, tmp, in_place):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    from residual_stream_burden_b200.dist import BucketedGradExchange, observe_ready_order, shard_batch
    try:
        torch.manual_seed(0)                                   # same model and full batch on every rank
        net = torch.nn.Sequential(torch.nn.Linear(12, 40), torch.nn.Tanh(), torch.nn.Linear(40, 40), torch.nn.Tanh(),
                                  torch.nn.Linear(40, 3))
        unused = torch.nn.Parameter(torch.ones(5))             # a parameter that never gets a gradient
        x, y = torch.randn(8, 12), torch.randn(8, 3)
        order = []
        params = list(net.parameters()) + [unused]
        ex = BucketedGradExchange(params, bucket_bytes=500, in_place=in_place, small_numel=100,
                                  on_bucket_reduced=order.append)
        assert len(ex.buckets) >= 3
        assert ex.buckets[0][0] is unused and ex.buckets[0][1] is net[4].bias          # reverse registration order
        # the order observed in a real backward pass: last layer first, the parameter without a gradient last
        seen = observe_ready_order(params, lambda: (net(x) - y).square().mean().backward())
        assert len(seen) == len(params) and {id(p) for p in seen} == {id(p) for p in params}
        layer_of = {id(p): k for k in (0, 2, 4) for p in net[k].parameters()}
        layers = [layer_of[id(p)] for p in seen[:-1]]
        assert layers == sorted(layers, reverse=True) and seen[-1] is unused
        for p in params:
            p.grad = None
        by_order = BucketedGradExchange(seen, bucket_bytes=500, ready_order=True)
        assert by_order.buckets[0][0] is seen[0] and by_order.buckets[-1][-1] is unused
        by_order.remove()
        for _ in range(2):                                     # two steps: the bookkeeping resets
            for p in params:
                p.grad = None
            order.clear()
            lo, hi = shard_batch(8, rank, world)
            ex.begin()
            (net(x[lo:hi]) - y[lo:hi]).square().mean().backward()
            launched_by_hooks = list(order)
            ex.finish()
            assert sorted(order) == list(range(len(ex.buckets)))
            assert launched_by_hooks == sorted(launched_by_hooks) and len(launched_by_hooks) >= len(ex.buckets) - 1
            got = [p.grad.clone() for p in net.parameters()]
            for p in net.parameters():
                p.grad = None
            (net(x) - y).square().mean().backward()            # full batch on one process = mean over the two shards
            for a, p in zip(got, net.parameters()):
                torch.testing.assert_close(a, p.grad, atol=1e-6, rtol=1e-5)
            assert unused.grad is None
        ex.remove()
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    except Exception as exc:                                   # noqa: BLE001
        import traceback
        open(os.path.join(tmp, f"err{rank}"), "w").write(traceback.format_exc())
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                                      # noqa: BLE001
            pass


@pytest.mark.parametrize("in_place", [True, False])
def test_bucketed_exchange_averages_gradients_during_backward(tmp_path, in_place):
    mp.spawn(_bucket_worker, args=(2, _port(), str(tmp_path), in_place), nprocs=2, join=True)
    errs = [p.read_text() for p in tmp_path.iterdir() if p.name.startswith("err")]
    assert not errs, errs[0]
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def _sharded_worker(rank, world, port, tmp):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    from residual_stream_burden_b200.dist import ShardedGradExchange, observe_ready_order, shard_batch
    try:
        torch.manual_seed(0)
        def make():
            torch.manual_seed(1)
            return torch.nn.Sequential(torch.nn.Linear(12, 40), torch.nn.Tanh(), torch.nn.Linear(40, 41), torch.nn.Tanh(),
                                       torch.nn.Linear(41, 3))
        net, ref = make(), make()
        x, y = torch.randn(8, 12), torch.randn(8, 3)
        params = list(net.parameters())
        order = observe_ready_order(params, lambda: (net(x) - y).square().mean().backward())
        for p in params:
            p.grad = None
        opts = []
        ex = ShardedGradExchange(order, ready_order=True, bucket_bytes=2000, small_numel=100,
                                 on_bucket_reduced=lambda k: opts[k].step())
        opts.extend(torch.optim.AdamW(ex.update_tensors(k), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.0)
                    for k in range(len(ex.buckets)))
        # 12x40 and 40x41 weights are sharded (even element counts), the 41x3 weight (123 elements) and biases are not
        assert sum(len(s) for s in ex._sharded) == 2 and sum(len(s) for s in ex._whole) == 4
        ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.0)
        lo, hi = shard_batch(8, rank, world)
        for _ in range(3):
            for p in params:
                p.grad = None
            ex.begin()
            (net(x[lo:hi]) - y[lo:hi]).square().mean().backward()
            ex.finish()
            ref_opt.zero_grad(set_to_none=True)
            (ref(x) - y).square().mean().backward()            # full batch = mean over the two shards
            ref_opt.step()
        for a, b in zip(net.parameters(), ref.parameters()):
            torch.testing.assert_close(a, b, atol=1e-6, rtol=1e-5)
        ex.remove()
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    except Exception:                                          # noqa: BLE001
        import traceback
        open(os.path.join(tmp, f"err{rank}"), "w").write(traceback.format_exc())
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                                      # noqa: BLE001
            pass


def test_sharded_update_equals_full_batch_adamw(tmp_path):
    """Reduce-scatter, update of each rank's slices, all-gather: after three steps both ranks hold the parameters a
    single process gets from AdamW on the full batch."""
    mp.spawn(_sharded_worker, args=(2, _port(), str(tmp_path)), nprocs=2, join=True)
    errs = [p.read_text() for p in tmp_path.iterdir() if p.name.startswith("err")]
    assert not errs, errs[0]
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
