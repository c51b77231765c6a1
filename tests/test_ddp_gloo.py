"""Data-parallel gradient averaging on CPU ranks (gloo, world size 2).

Checks the wrapper's contract against a single-process run on the concatenated batch:
parameters start from rank 0's values, every rank ends a step with the mean gradient, SGD
trajectories stay identical across ranks, and a rank that fails before its all-reduce makes
its peer error out (timeout) instead of hanging.
"""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _net(seed):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.Tanh(), torch.nn.Linear(32, 16),
                               torch.nn.Tanh(), torch.nn.Linear(16, 4))


def _worker(rank, world, port, out_dir, bucket_mb, fail_rank):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8 if fail_rank is not None else 60))
    from snn_gpu_training_bptt_b200.example.ddp import DistributedDataParallel as DDP
    torch.set_num_threads(1)
    model = _net(seed=100 + rank)                      # different init per rank on purpose
    ddp = DDP(model, bucket_mb=bucket_mb)
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    gen = torch.Generator().manual_seed(7)
    data = torch.randn(3, 8 * world, 12, generator=gen)
    target = torch.randn(3, 8 * world, 4, generator=gen)
    result = {"buckets": ddp.bucket_sizes()}
    try:
        for step in range(3):
            ddp.zero_grad()
            xb = data[step, rank * 8:(rank + 1) * 8]
            yb = target[step, rank * 8:(rank + 1) * 8]
            loss = ((ddp(xb) - yb) ** 2).mean()
            if fail_rank == rank and step == 1:
                raise RuntimeError("injected failure before backward")
            loss.backward()
            if step == 0:
                result["grad0"] = [p.grad.clone() for p in model.parameters()]
            opt.step()
        result["params"] = [p.detach().clone() for p in model.parameters()]
        result["status"] = "ok"
    except Exception as e:  # noqa: BLE001
        result["status"] = f"error: {type(e).__name__}: {e}"[:300]
    torch.save(result, os.path.join(out_dir, f"rank{rank}.pt"))
    if fail_rank is None:
        dist.destroy_process_group()


def _run(tmp_path, bucket_mb, fail_rank=None):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path), bucket_mb, fail_rank), nprocs=world, join=True)
    return [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]


@pytest.mark.parametrize("bucket_mb", [25.0, 0.001])
def test_mean_gradient_matches_single_process(tmp_path, bucket_mb):
    res = _run(tmp_path, bucket_mb)
    assert all(r["status"] == "ok" for r in res), [r["status"] for r in res]
    if bucket_mb < 1:
        assert len(res[0]["buckets"]) > 1          # several buckets exercised
    # single-process reference on the concatenated batch, starting from rank 0's init
    model = _net(seed=100)
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    gen = torch.Generator().manual_seed(7)
    data = torch.randn(3, 16, 12, generator=gen)
    target = torch.randn(3, 16, 4, generator=gen)
    for step in range(3):
        opt.zero_grad()
        loss = ((model(data[step]) - target[step]) ** 2).mean()
        loss.backward()
        if step == 0:
            for g_ref, g0, g1 in zip([p.grad for p in model.parameters()], res[0]["grad0"], res[1]["grad0"]):
                assert torch.allclose(g0, g_ref, rtol=1e-5, atol=1e-7)
                assert torch.equal(g0, g1)
        opt.step()
    for p_ref, p0, p1 in zip(model.parameters(), res[0]["params"], res[1]["params"]):
        assert torch.equal(p0, p1)                    # ranks stay in lock-step
        assert torch.allclose(p0, p_ref.detach(), rtol=1e-4, atol=1e-6)


def test_failed_rank_surfaces_as_error_not_hang(tmp_path):
    """Rank 1 raises before its second backward; rank 0's all-reduce must end with an error."""
    res = _run(tmp_path, 25.0, fail_rank=1)
    assert res[1]["status"].startswith("error: RuntimeError: injected")
    assert res[0]["status"].startswith("error")
