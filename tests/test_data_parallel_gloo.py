"""world_size-2 test of the batch-sharding + gradient all-reduce logic on CPU ranks (gloo).

The compute inside each rank is the dense PyTorch backend; what is under test is the host logic:
row sharding, flat per-layer buckets, hooks that start the collective, and that the summed
shard gradients equal the gradients of the unsharded batch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torchsplinekan_b200 as sk
    torch.manual_seed(0)
    net = sk.KAN([6, 5, 3], backend="reference").double()
    x = torch.rand(37, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(1)) * 2 - 1
    full = sk.KAN([6, 5, 3], backend="reference").double()
    full.load_state_dict(net.state_dict())
    full(x).square().sum().backward()

    bucket = sk.GradientBucket(net.layers)
    a, b = sk.shard_rows(x.shape[0], world, rank)
    for step in range(2):                       # second step checks bucket reuse after zero_grad
        bucket.zero_grad()
        net(x[a:b]).square().sum().backward()
        bucket.finish()
        for p, q in zip(net.parameters(), full.parameters()):
            assert torch.allclose(p.grad, q.grad, rtol=1e-10, atol=1e-12), (rank, step)
    assert bucket.bucket_bytes() == sum(p.numel() for p in net.parameters()) * 8
    torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}.pt"))
    dist.destroy_process_group()


def test_sharded_gradients_equal_full_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}.pt").exists() for r in range(world))


def _reg_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torchsplinekan_b200 as sk
    torch.manual_seed(0)
    net = sk.KAN([6, 5, 3], backend="reference").double()
    x = torch.rand(37, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(1)) * 2 - 1
    full = sk.KAN([6, 5, 3], backend="reference").double()
    full.load_state_dict(net.state_dict())
    y, r = full.forward_with_regularization(x, 0.7, 1.3)
    (y.square().sum() + r).backward()

    bucket = sk.GradientBucket(net.layers)
    a, b = sk.shard_rows(x.shape[0], world, rank)            # 19 and 18 rows: ragged shards
    bucket.zero_grad()
    ys, rs = net.forward_with_regularization(x[a:b], 0.7, 1.3, reg_group=True)
    assert abs(float(rs.detach()) - float(r.detach())) <= 1e-12 * max(1.0, abs(float(r.detach()))), rank
    (ys.square().sum() + rs / world).backward()              # gradients are summed over the ranks
    bucket.finish()
    for p, q in zip(net.parameters(), full.parameters()):
        assert torch.allclose(p.grad, q.grad, rtol=1e-9, atol=1e-12), (rank, float((p.grad - q.grad).abs().max()))

    # per-shard penalties (the default) do NOT add up to the whole-batch penalty: the variant matters
    _, r_local = net.forward_with_regularization(x[a:b], 0.7, 1.3)
    both = torch.tensor([float(r_local.detach())], dtype=torch.float64)
    dist.all_reduce(both)
    assert abs(float(both) / world - float(r.detach())) > 1e-6

    # second derivatives go through the collective too
    h = x[a:b].clone().requires_grad_(True)
    _, r2 = net.forward_with_regularization(h, 0.7, 1.3, reg_group=dist.group.WORLD, reg_impl="dense")
    (g,) = torch.autograd.grad(r2, h, create_graph=True)
    g.square().sum().backward()
    assert h.grad is not None and torch.isfinite(h.grad).all()
    torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}.pt"))
    dist.destroy_process_group()


def test_global_batch_regulariser_equals_unsharded(tmp_path):
    """reg_group: every rank evaluates the penalty of the GLOBAL batch (one all-reduce of mean|phi|
    per layer, weighted by the ranks' row counts) and the summed shard gradients equal those of the
    unsharded batch, with ragged shards."""
    world = 2
    mp.spawn(_reg_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}.pt").exists() for r in range(world))
