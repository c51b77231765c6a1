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


class _TwoHeads(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(5)
        self.trunk = torch.nn.Linear(6, 8)
        self.head_a = torch.nn.Linear(8, 3)
        self.head_b = torch.nn.Linear(8, 3)

    def forward(self, x, use_b):
        h = torch.tanh(self.trunk(x))
        return self.head_a(h) + (self.head_b(h) if use_b else 0.0)


def _skip_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from snn_gpu_training_bptt_b200.example.ddp import DistributedDataParallel as DDP
    torch.set_num_threads(1)
    model = _TwoHeads()
    ddp = DDP(model, bucket_mb=0.00001)                # every parameter its own bucket
    calls = []
    real = ddp._all_reduce_mean
    ddp._all_reduce_mean = lambda flat: (calls.append(flat.numel()), real(flat))[1]
    gen = torch.Generator().manual_seed(3)
    data = torch.randn(2, world, 4, 6, generator=gen)
    status, grads = "ok", []
    try:
        for step in range(2):
            ddp.zero_grad()
            # step 1: rank 1 takes a branch that leaves head_b (two whole buckets) without a gradient
            use_b = not (step == 1 and rank == 1)
            ddp(data[step, rank], use_b).square().mean().backward()
            grads.append({n: p.grad.clone() for n, p in model.named_parameters()})
    except Exception as e:  # noqa: BLE001
        status = f"error: {type(e).__name__}: {e}"[:300]
    torch.save({"status": status, "grads": grads, "calls": calls, "buckets": ddp.bucket_sizes()},
               os.path.join(out_dir, f"skip{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_rank_that_skips_a_parameter_issues_the_same_collectives(tmp_path):
    """One rank's backward leaves two buckets untouched: both ranks must still issue every bucket's
    all-reduce, in bucket order (otherwise NCCL would hang), and the untouched rank contributes zeros."""
    world, port = 2, _free_port()
    mp.spawn(_skip_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(str(tmp_path), f"skip{r}.pt")) for r in range(world)]
    assert all(r["status"] == "ok" for r in res), [r["status"] for r in res]
    assert res[0]["calls"] == res[1]["calls"] == res[0]["buckets"] * 2     # same sequence, both steps
    model = _TwoHeads()
    gen = torch.Generator().manual_seed(3)
    data = torch.randn(2, world, 4, 6, generator=gen)
    for step in range(2):
        want = {n: torch.zeros_like(p) for n, p in model.named_parameters()}
        for rank in range(world):
            model.zero_grad()
            model(data[step, rank], not (step == 1 and rank == 1)).square().mean().backward()
            for n, p in model.named_parameters():
                if p.grad is not None:
                    want[n] += p.grad / world
        for r in res:
            for n in want:
                assert torch.allclose(r["grads"][step][n], want[n], rtol=1e-5, atol=1e-7), (step, n)


def _syncbn_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from snn_gpu_training_bptt_b200 import snnlib_op as sop
    torch.set_num_threads(1)
    gen = torch.Generator().manual_seed(11)
    full = torch.randn(4, 2 * world, 6, 3, 3, generator=gen) * 2 + 0.5        # [T, B_total, C, H, W]
    mine = full[:, rank * 2:(rank + 1) * 2].contiguous()
    layer = sop.BnDist(6, (0, 1, 3, 4))
    n_calls = []
    real_all_reduce = dist.all_reduce
    dist.all_reduce = lambda t, *a, **k: (n_calls.append(tuple(t.shape)), real_all_reduce(t, *a, **k))[1]
    var1, mean1 = layer._statistics(mine)
    dist.all_reduce = real_all_reduce
    low = sop.BnDist(6, (0, 1, 3, 4))
    var_low, mean_low = low._statistics(mine.to(torch.bfloat16))               # 16-bit activations
    var2, mean2 = layer._statistics(mine * 0.5)                                # second step: running stats move on
    torch.save({"var1": var1, "mean1": mean1, "var2": var2, "mean2": mean2, "calls": n_calls,
                "var_low": var_low, "mean_low": mean_low,
                "running_var": layer.running_var.detach().clone(),
                "running_mean": layer.running_mean.detach().clone(),
                "world": layer.world_size, "ids": (id(layer.running_var), id(layer.running_mean))},
               os.path.join(out_dir, f"bn{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_sync_bn_statistics_over_two_ranks(tmp_path):
    """Host side of the sync-BN layers (reference snnlib_op.py:231-282): every rank normalises with
    the statistics of the whole batch (mean of the ranks' means and mean squares), and the running
    statistics follow the reference's update (momentum 0.05, unbiased correction with the LOCAL
    element count, as the reference computes its factor from the local tensor)."""
    world, port = 2, _free_port()
    mp.spawn(_syncbn_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f"bn{r}.pt")) for r in range(world)]
    gen = torch.Generator().manual_seed(11)
    full = torch.randn(4, 2 * world, 6, 3, 3, generator=gen) * 2 + 0.5
    dims = (0, 1, 3, 4)
    var_all, mean_all = torch.var_mean(full, dim=dims, unbiased=False)
    low_all = full.to(torch.bfloat16).float()
    var_low, mean_low = torch.var_mean(low_all, dim=dims, unbiased=False)
    for r in res:
        assert r["world"] == world
        assert r["calls"] == [(2, 6)]                    # both moments travel in one [2, C] message
        # 16-bit activations: statistics come out in fp32 and match an fp32 computation on the same values
        assert r["var_low"].dtype == r["mean_low"].dtype == torch.float32
        assert torch.allclose(r["mean_low"], mean_low, atol=1e-5)
        assert torch.allclose(r["var_low"], var_low, rtol=1e-4, atol=1e-5)
        assert torch.allclose(r["mean1"], mean_all, atol=1e-6)
        assert torch.allclose(r["var1"], var_all, rtol=1e-5, atol=1e-6)
        assert torch.allclose(r["mean2"], mean_all * 0.5, atol=1e-6)
        assert torch.allclose(r["var2"], var_all * 0.25, rtol=1e-5, atol=1e-6)
    count = full.numel() / world / 6                         # local elements per channel
    factor = count / (count - 1)
    rv, rm = torch.ones(6), torch.zeros(6)
    for scale in (1.0, 0.5):
        rv = rv * 0.95 + var_all * scale * scale * (0.05 * factor)
        rm = rm * 0.95 + mean_all * scale * 0.05
    for r in res:
        assert torch.allclose(r["running_var"], rv, rtol=1e-5, atol=1e-6)
        assert torch.allclose(r["running_mean"], rm, rtol=1e-5, atol=1e-6)
    assert torch.equal(res[0]["running_var"], res[1]["running_var"])
