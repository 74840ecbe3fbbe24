"""Multi-GPU tests (need at least 2 GPUs; skipped otherwise): the NVLink gradient all-reduce of
GradientBucket against single-process gradients of the whole batch, for the in-switch (multimem)
and the peer-load kernels and for NCCL."""
import os
import socket
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, transport_env, direct, out):
    import torch.distributed as dist
    import torchsplinekan_b200 as sk
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    if transport_env:
        os.environ["KAN_B200_ALLREDUCE"] = transport_env
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        torch.manual_seed(0)
        net = sk.KAN([24, 520, 6], backend="cuda").to(dev)
        g = torch.Generator().manual_seed(1)
        x = (torch.rand(1030, 24, generator=g) * 2 - 1)
        r0, r1 = sk.shard_rows(x.shape[0], world, rank)
        bucket = sk.GradientBucket(net.layers, transport="auto", direct=direct, chunks=3)
        for step in range(3):                              # the signal pad is reused across steps
            bucket.zero_grad()
            net(x[r0:r1].to(dev)).square().sum().backward()
            bucket.finish()
        bucket.check()
        torch.cuda.synchronize(dev)
        if rank == 0:
            out["transport"] = bucket.transport
            out["grads"] = [p.grad.detach().cpu() for p in net.parameters()]
            out["sinks"] = len(bucket._sinks)
            ref = sk.KAN([24, 520, 6], backend="cuda").to(dev)
            ref.load_state_dict(net.state_dict())
            ref(x.to(dev)).square().sum().backward()
            out["ref"] = [p.grad.detach().cpu() for p in ref.parameters()]
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("direct", [False, True])
@pytest.mark.parametrize("transport_env,expect", [("nvlink", "nvlink"), ("p2p", "nvlink-p2p"), ("", "nccl")])
def test_gradient_bucket_transports_match_whole_batch(transport_env, expect, direct):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), transport_env, direct, out), nprocs=world, join=True)
    assert out["transport"].startswith(expect), out["transport"]
    assert out["sinks"] == (2 if direct else 0)
    for got, want in zip(out["grads"], out["ref"]):
        err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
        assert err < 2e-5, err


def _reg_worker(rank, world, port, out):
    import torch.distributed as dist
    import torchsplinekan_b200 as sk
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        torch.manual_seed(0)
        net = sk.KAN([24, 40, 6], backend="cuda").to(dev)
        g = torch.Generator().manual_seed(1)
        x = (torch.rand(1031, 24, generator=g) * 2 - 1)          # ragged shards: 516 and 515 rows
        r0, r1 = sk.shard_rows(x.shape[0], world, rank)
        bucket = sk.GradientBucket(net.layers, transport="nccl")
        bucket.zero_grad()
        y, r = net.forward_with_regularization(x[r0:r1].to(dev), 0.7, 1.3, reg_group=True)
        (y.square().sum() + r / world).backward()                 # the bucket sums over the ranks
        bucket.finish()
        torch.cuda.synchronize(dev)
        if rank == 0:
            out["backends"] = [l.last_backend for l in net.layers]
            out["penalty"] = float(r.detach())
            out["grads"] = [p.grad.detach().cpu() for p in net.parameters()]
            ref = sk.KAN([24, 40, 6], backend="cuda").to(dev)
            ref.load_state_dict(net.state_dict())
            yw, rw = ref.forward_with_regularization(x.to(dev), 0.7, 1.3)
            (yw.square().sum() + rw).backward()
            out["penalty_ref"] = float(rw.detach())
            out["ref"] = [p.grad.detach().cpu() for p in ref.parameters()]
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_global_batch_regulariser_on_two_gpus():
    """reg_group on the native path: each rank's fused edge statistic is all-reduced (weighted by its
    row count) before the penalty, so the penalty and the summed gradients are those of the whole
    batch; tolerance 5e-5 of max|gradient| (float32, tensor-core products in different groupings)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_reg_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out["backends"] == ["cuda", "cuda"]
    assert abs(out["penalty"] - out["penalty_ref"]) <= 1e-5 * abs(out["penalty_ref"])
    for got, want in zip(out["grads"], out["ref"]):
        err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
        assert err < 5e-5, err
