"""Data-parallel training of a spiking CNN on synthetic images: samples/sec at 1..8 GPUs.

Follows the reference's trainers (snnlib/example/train_test_cifar.py:31-70 single GPU,
train_test_imagenet_alexnet_dist.py:26-105 one process per GPU over NCCL): SGD with momentum
0.9 and lr 1e-2, cross-entropy on the time-averaged output, ``zero_grad -> forward -> loss ->
backward -> step``. CIFAR / ImageNet are replaced by seeded synthetic data of the same shape:
3x32x32 images with pixels ~ U(0,1) and uniform-random labels in [0, 10).

Launch:  python -m snn_gpu_training_bptt_b200.example.train_synthetic --model vgg
         python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
                -m snn_gpu_training_bptt_b200.example.train_synthetic --model vgg

Every step copies its batch from pinned host memory to the GPU and reads the loss back when
it logs, so the throughput printed is end to end for the training loop.
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import models
from .ddp import BucketSGD, DistributedDataParallel


class SyntheticImages:
    """A fixed pool of pinned host batches cycled through; stands in for a DataLoader."""

    def __init__(self, batch, seed, pool=4, image=32, classes=10):
        gen = torch.Generator().manual_seed(seed)
        self.images = [torch.rand((batch, 3, image, image), generator=gen) for _ in range(pool)]
        self.labels = [torch.randint(0, classes, (batch,), generator=gen) for _ in range(pool)]
        if torch.cuda.is_available():
            self.images = [t.pin_memory() for t in self.images]
            self.labels = [t.pin_memory() for t in self.labels]
        self.bytes_per_batch = self.images[0].numel() * 4 + self.labels[0].numel() * 8

    def batch(self, step, device):
        k = step % len(self.images)
        return (self.images[k].to(device, non_blocking=True), self.labels[k].to(device, non_blocking=True))


def save_checkpoint(path, model, optimizer, step):
    """Parameters under the reference's key names plus what a resume needs (the reference saves
    only ``state_dict()`` of the best epoch, train_test_cifar.py:94-97)."""
    core = model.module if isinstance(model, DistributedDataParallel) else model
    torch.save({"model": core.state_dict(), "optimizer": optimizer.state_dict(), "step": step}, path)


def load_checkpoint(path, model, optimizer=None):
    core = model.module if isinstance(model, DistributedDataParallel) else model
    blob = torch.load(path, map_location="cpu")
    state = blob["model"] if "model" in blob else blob      # plain state dicts load too
    core.load_state_dict(state)
    if optimizer is not None and "optimizer" in blob:
        optimizer.load_state_dict(blob["optimizer"])
    return blob.get("step", 0) if isinstance(blob, dict) else 0


def run(model_name="vgg", time_steps=8, batch=64, steps=20, warmup=5, precision="bf16", lr=1e-2,
        bucket_mb=64.0, overlap=True, seed=0, log=False, checkpoint=None, graph=True,
        return_params=False, model_kwargs=None, communicate=True, bucket_sgd=False, prefetch_input=True):
    """Trains for warmup+steps steps; returns a dict with samples/sec (whole job) and timings.

    ``graph=True`` captures one whole training step (zero_grad, forward, loss, backward with its
    bucketed all-reduces on the side stream, SGD update) into a CUDA graph after the warm-up steps
    and replays it: a step is ~150 small launches, and at a few ms per step the Python/launch
    overhead of issuing them one by one is as large as the GPU time itself.

    ``bucket_sgd=True`` swaps ``torch.optim.SGD`` for ``ddp.BucketSGD`` (the update of the early
    buckets overlaps the last all-reduce). Measured on the VGG-style network it does not pay: the
    second, small optimizer step costs ~40 us of launches, about what the overlap saves at 8 GPUs."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    own_group = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_group = True

    act_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[precision]
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(seed)
    net = models.build(model_name, time_steps=time_steps, act_dtype=act_dtype, **(model_kwargs or {})).to(dev)
    # last bucket = the first layer only (<= 30 KB): the fastest of the tail layouts measured at 8 GPUs
    tail = tuple(float(v) for v in os.environ.get("SNN_DDP_TAIL_MB", "0.03").split(","))
    model = DistributedDataParallel(net, bucket_mb=bucket_mb, overlap=overlap, communicate=communicate,
                                    defer_wait=bucket_sgd, tail_mb=tail)
    if bucket_sgd:
        opt = BucketSGD(model, lr=lr, momentum=0.9)     # updates bucket by bucket as the all-reduces land
    else:
        opt = torch.optim.SGD(net.parameters(), lr=lr, momentum=0.9)
    data = SyntheticImages(batch, seed=1000 + rank)
    n_params = sum(p.numel() for p in net.parameters())

    static_images = torch.empty((batch, 3, 32, 32), device=dev)
    static_labels = torch.empty((batch,), dtype=torch.long, device=dev)
    # The next batch travels host -> device on its own stream while the current step computes (two
    # staging buffers); the step then starts with a device-to-device copy into the fixed buffers the
    # captured graph reads. With several ranks on one host link the upload is several times slower
    # than alone (measured 12 GB/s per rank at 8 GPUs against 49 GB/s), which would otherwise sit in
    # front of every step.
    copy_stream = torch.cuda.Stream(dev)
    staged = [(torch.empty_like(static_images), torch.empty_like(static_labels), torch.cuda.Event()) for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def prefetch(k):
        j, (img, lab, ready) = k % len(data.images), staged[k % 2]
        copy_stream.wait_event(consumed[k % 2])          # the step that last read this staging buffer
        with torch.cuda.stream(copy_stream):
            img.copy_(data.images[j], non_blocking=True)
            lab.copy_(data.labels[j], non_blocking=True)
            ready.record(copy_stream)

    state = {"prefetched": None}

    def load(k):
        """This step's batch: pinned host memory -> staging (prefetched during the step before) ->
        the fixed device buffers the step reads; then the upload of step k+1's batch is started."""
        if not prefetch_input:
            j = k % len(data.images)
            static_images.copy_(data.images[j], non_blocking=True)
            static_labels.copy_(data.labels[j], non_blocking=True)
            return
        if state["prefetched"] != k:
            prefetch(k)
        img, lab, ready = staged[k % 2]
        cur = torch.cuda.current_stream(dev)
        cur.wait_event(ready)
        static_images.copy_(img, non_blocking=True)
        static_labels.copy_(lab, non_blocking=True)
        consumed[k % 2].record(cur)
        prefetch(k + 1)
        state["prefetched"] = k + 1

    def compute():
        model.zero_grad()
        loss = F.cross_entropy(model(static_images), static_labels)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    captured = None
    if graph:
        # warm up on a side stream (cuDNN autotuning, lazy optimizer state), then capture
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for k in range(max(warmup, 3)):
                load(k)
                loss = compute()
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured, capture_error_mode="thread_local"):
            static_loss = compute()

        def one_step(k):
            load(k)
            captured.replay()
            return static_loss
    else:
        def one_step(k):
            load(k)
            return compute()

        for k in range(warmup):
            loss = one_step(k)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for k in range(steps):
        loss = one_step(warmup + k)
        if log and rank == 0 and (k + 1) % 10 == 0:
            print(f"step {k + 1}/{steps} loss {float(loss):.4f}", flush=True)
    final_loss = float(loss.detach())  # device -> host read of the step's result
    e1.record()
    barrier()
    wall = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([dev_ms, wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, wall = float(t[0]), float(t[1])
    if checkpoint and rank == 0:
        save_checkpoint(checkpoint, model, opt, warmup + steps)
    out = {
        "model": model_name, "time_steps": time_steps, "batch_per_gpu": batch, "n_gpus": world,
        "precision": precision, "params": n_params, "steps": steps,
        "ms_per_step": dev_ms / steps, "samples_per_s": batch * world * steps / (dev_ms / 1e3),
        "samples_per_s_wall": batch * world * steps / wall, "final_loss": final_loss,
        "h2d_bytes_per_step": data.bytes_per_batch, "d2h_bytes_per_step": 4,
        "grad_buckets": len(model.buckets), "overlap": overlap, "cuda_graph": bool(graph),
        "bucket_bytes": [b["flat"].numel() * b["flat"].element_size() for b in model.buckets],
        "communicate": communicate,
    }
    if return_params:
        out["params"] = [p.detach().float().cpu() for p in net.parameters()]
    # A captured step holds NCCL work that refers to the communicator: release the graph before
    # the process group goes away (tearing the group down under a live graph blocks forever).
    if captured is not None:
        torch.cuda.synchronize(dev)
        captured.reset()
        captured = None
    if own_group:
        dist.destroy_process_group()
    return out


def bucket_timeline(model_name="vgg", time_steps=8, batch=64, precision="bf16", bucket_mb=25.0, steps=3):
    """Per-bucket timing of the overlapped all-reduce over a few EAGER steps (CUDA events cannot be
    timed inside a captured graph): for every bucket, milliseconds from the start of the step to the
    moment its last gradient exists (ready), to the start and to the end of its all-reduce on the
    side stream, and the time at which backward itself ends. Medians over ``steps`` steps."""
    import statistics
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    own_group = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_group = True
    act_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[precision]
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(0)
    net = models.build(model_name, time_steps=time_steps, act_dtype=act_dtype).to(dev)
    model = DistributedDataParallel(net, bucket_mb=bucket_mb)
    opt = torch.optim.SGD(net.parameters(), lr=1e-2, momentum=0.9)
    images = torch.rand(batch, 3, 32, 32, device=dev)
    labels = torch.randint(0, 10, (batch,), device=dev)
    rows = []
    for k in range(5 + steps):
        model.trace = [] if k >= 5 else None
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        model.zero_grad()
        loss = F.cross_entropy(model(images), labels)
        e1.record()
        loss.backward()
        e2.record()
        opt.step()
        torch.cuda.synchronize(dev)
        if model.trace is not None:
            rows.append({"forward_end": e0.elapsed_time(e1), "backward_end": e0.elapsed_time(e2),
                         "buckets": [(b, e0.elapsed_time(ev[0]), e0.elapsed_time(ev[1]), e0.elapsed_time(ev[2]))
                                     for b, ev in model.trace]})
    med = lambda vals: round(statistics.median(vals), 3)
    out = {"model": model_name, "n_gpus": world, "bucket_mb": bucket_mb, "eager": True,
           "bucket_bytes": [b["flat"].numel() * b["flat"].element_size() for b in model.buckets],
           "forward_end_ms": med([r["forward_end"] for r in rows]), "backward_end_ms": med([r["backward_end"] for r in rows]),
           "buckets": [{"bucket": i, "ready_ms": med([r["buckets"][i][1] for r in rows]),
                        "allreduce_start_ms": med([r["buckets"][i][2] for r in rows]),
                        "allreduce_end_ms": med([r["buckets"][i][3] for r in rows])}
                       for i in range(len(rows[0]["buckets"]))] if rows and rows[0]["buckets"] else []}
    if own_group:
        dist.destroy_process_group()
    return out


def profile_steps(model_name, time_steps, batch, precision, steps=3):
    """Kernel-level table (torch.profiler) of a few eager training steps on one GPU."""
    from torch.profiler import ProfilerActivity, profile
    act_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[precision]
    torch.backends.cudnn.benchmark = True
    net = models.build(model_name, time_steps=time_steps, act_dtype=act_dtype).cuda()
    opt = torch.optim.SGD(net.parameters(), lr=1e-2, momentum=0.9)
    images = torch.rand(batch, 3, 32, 32, device="cuda")
    labels = torch.randint(0, 10, (batch,), device="cuda")

    def step():
        opt.zero_grad()
        F.cross_entropy(net(images), labels).backward()
        opt.step()

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            step()
        torch.cuda.synchronize()
    return prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=70)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="vgg", choices=["vgg", "resnet19"])
    ap.add_argument("--time-steps", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--bucket-mb", type=float, default=64.0)
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="issue every launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--log", action="store_true")
    ap.add_argument("--bucket-timeline", action="store_true",
                    help="print per-bucket ready / all-reduce start / end times of a few eager steps instead of timing")
    ap.add_argument("--profile", action="store_true",
                    help="print a torch.profiler kernel table of 3 eager single-GPU steps instead of timing")
    a = ap.parse_args()
    watchdog = os.environ.get("SNN_TRAIN_WATCHDOG_S")
    if watchdog:   # dump every thread's Python stack and exit if the run is still going after N seconds
        import faulthandler
        faulthandler.dump_traceback_later(int(watchdog), exit=True)
    T = a.time_steps or (8 if a.model == "vgg" else 16)
    B = a.batch or (64 if a.model == "vgg" else 128)
    if a.profile:
        print(profile_steps(a.model, T, B, a.precision))
        return
    if a.bucket_timeline:
        res = bucket_timeline(a.model, T, B, a.precision, a.bucket_mb)
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(res))
        return
    res = run(a.model, T, B, a.steps, a.warmup, a.precision, bucket_mb=a.bucket_mb,
              overlap=not a.no_overlap, log=a.log, checkpoint=a.checkpoint, graph=not a.no_graph)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
