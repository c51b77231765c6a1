#!/usr/bin/env python
"""Benchmark of the LIF fire forward+backward (BPTT) hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one forward (snn_lif_fwd) plus one backward (snn_lif_bwd) over one batch of
synthetic input currents / upstream gradients: fp32, T=8 time steps, 2^26 neurons per GPU
(2 GiB per tensor; the single-GPU bandwidth-sweep headline case). Inputs are i.i.d.
N(0.5, 1) currents and N(0, 1) gradients from a fixed seed, standing in for the CIFAR /
ImageNet activations the reference trains on.

Metric: achieved HBM GB/s, counting the ALGORITHMIC bytes of the pass,
20 B per neuron-timestep = forward (read x 4 + write spike 4) + backward (read x 4 +
read grad 4 + write grad_x 4). With N>1 GPUs every rank processes its own 2^26-neuron shard
(the neuron/batch axis shards with no exchange), so the aggregate is weak scaling.

Printed keys beyond the base contract:
  roofline          dominant kernel (the backward, 12 B/step) against the measured HBM copy peak
  cpu_baseline      the reference's own CPU path (its gold_op.py from oracle/_ref/, else the port in
                    oracle/), timed on this host's cores on a bounded sample
  e2e               same metric through the host-buffer API (pinned host -> device -> host)
  linear_lif        the fused synaptic linear + LIF layer (T=8, batch 256, 2048 -> 2048, bf16) forward and
                    BPTT backward on the tcgen05 kernels: microseconds, TFLOP/s, fraction of the bf16 peak
  trainer, trainer_resnet19
                    spiking-CNN training samples/s (VGG-style T=8 batch 64/GPU; ResNet-19-style T=16 batch
                    128/GPU), data-parallel over the N ranks, with the exposed all-reduce time at N > 1
  timed_blocks      the K-step block is repeated until >= 1 s is timed; the median block is reported
Flat scalar copies of the nested legs (linear_lif_*, trainer_*) sit at the top level too.

Other workloads (single measurements, not the contract line): --workload sweep | bn_lif | linear_lif |
host_link.  --impl reference times the reference's CPU implementation on the host cores.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T_STEPS = 8
NEURONS = 1 << 26
BYTES_FWD, BYTES_BWD = 8, 12          # algorithmic bytes per neuron-timestep, fp32
ALPHA, THRESH, BETA, INTERVAL = 0.25, 0.25, 1.0, 0.5
FALLBACK_HBM_GBS = 6650.0             # earlier measurement on this pool, used if no peaks file
NOMINAL_HBM_GBS = 8000.0
WORKLOAD = "lif_fire_fwd_bwd fp32 T=8 N=2^26 per GPU, x~N(0.5,1), grad~N(0,1), seed 1234"

# DRAM traffic of the backward kernel per neuron-timestep as measured by one ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum of snn::lif_bwd_kernel, T=8, N=2^24 -- 2 GiB on
# the device, inside the capture size rule -- divided by T*N; traffic is proportional to T*N,
# so a full launch is this figure x T*N).
NCU_BWD_TRAFFIC_BYTES_PER_STEP = 11.69


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, device copy)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    BAD = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown"}
    NOTE = {0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
            0x100: "display_clock_setting", 0x10: "sync_boost"}

    def __init__(self, index, period=0.02):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in {**self.BAD, **self.NOTE}.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# CPU legs (rank 0 only): the oracle's PyTorch-autograd port of the reference's gold op, and
# the plain-C loops, on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------
def cpu_torch_port_time(n_sample, reps, threads):
    import torch
    from oracle import lif_oracle as orc
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(1234)
    x = 0.5 + torch.randn((T_STEPS, 1, n_sample), generator=gen)
    g = torch.randn((T_STEPS, 1, n_sample), generator=gen)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.torch_fire_fwd_bwd(x, g)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_c_port_time(n_sample, reps):
    import numpy as np
    from oracle import lif_oracle as orc
    rng = np.random.default_rng(1234)
    x = (0.5 + rng.standard_normal((T_STEPS, 1, n_sample))).astype(np.float32)
    g = rng.standard_normal((T_STEPS, 1, n_sample)).astype(np.float32)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.c_lif_fwd(x)
        orc.c_lif_bwd(x, g)
        best = min(best, time.perf_counter() - t0)
    return best


def gbps(n_neurons, seconds):
    return (BYTES_FWD + BYTES_BWD) * T_STEPS * n_neurons / seconds / 1e9


def cpu_reference_time(gold, n_sample, reps, threads):
    import torch
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(1234)
    x = 0.5 + torch.randn((T_STEPS, 1, n_sample), generator=gen)
    g = torch.randn((T_STEPS, 1, n_sample), generator=gen)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        reference_fwd_bwd(gold, x, g)
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_baseline_block():
    cores = os.cpu_count() or 1
    n_sample = 1 << 22
    gold = reference_gold_op()
    if gold is not None:
        t_torch, kind = cpu_reference_time(gold, n_sample, reps=3, threads=cores), "reference"
        what = "the reference's own gold_op.py (gold_fire + autograd, from oracle/_ref)"
    else:
        t_torch, kind = cpu_torch_port_time(n_sample, reps=3, threads=cores), "port"
        what = "PyTorch-autograd port of the reference's gold_fire"
    t_c = cpu_c_port_time(1 << 24, reps=3)
    return {
        "value": round(gbps(n_sample, t_torch), 3), "unit": "GB/s", "cores": cores, "kind": kind,
        "sample": f"{what}, fwd+bwd, T=8, N=2^22 "
                  f"(1/16 of one GPU step), best of 3, {t_torch:.3f} s",
        "c_loops_value": round(gbps(1 << 24, t_c), 3),
        "c_loops_sample": f"plain-C OpenMP restatement, T=8, N=2^24, best of 3, {t_c:.3f} s",
    }


def reference_gold_op():
    """The reference's own CPU implementation of the path: its pure-PyTorch gold_op.py as installed,
    unmodified, into oracle/_ref/ by oracle/build_oracle.install_reference(). None when absent."""
    path = os.path.join(ROOT, "oracle", "_ref", "gold_op.py")
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("snn_reference_gold_op", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_fwd_bwd(gold, x, g):
    """One forward + backward of the reference's gold_fire (its globals set to this workload's
    constants; gold_fire reads the step count from its module global)."""
    gold.alpha, gold.beta, gold.interval, gold.thresh, gold.time_step = ALPHA, BETA, INTERVAL, THRESH, x.shape[0]
    xr = x.detach().requires_grad_(True)
    _, spikes = gold.gold_fire(xr)
    spikes.backward(g)
    return xr.grad


def run_reference_arm(args):
    """The reference's CPU implementation of the path on all host threads: its own gold_op.py when
    oracle/_ref/ holds it (kind "reference"), else the restatement in oracle/lif_oracle.py (kind
    "port"). Each step is a bounded sample of the GPU arm's 2^26-neuron step; GB/s is normalised by
    the sample's size."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import lif_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gold = reference_gold_op()
    kind = "reference" if gold is not None else "port"
    step_fn = (lambda x, g: reference_fwd_bwd(gold, x, g)) if gold is not None else (lambda x, g: orc.torch_fire_fwd_bwd(x, g))

    def inputs(n):
        gen = torch.Generator().manual_seed(1234)
        return (0.5 + torch.randn((T_STEPS, 1, n), generator=gen), torch.randn((T_STEPS, 1, n), generator=gen))

    x, g = inputs(1 << 18)
    step_fn(x, g)
    t0 = time.perf_counter()
    step_fn(x, g)
    probe = time.perf_counter() - t0                                   # seconds per 2^18 neurons
    budget = 90.0 / max(1, args.steps + args.warmup)                   # seconds per step
    n_sample = 1 << 18
    while n_sample < (1 << 23) and probe * (2 * n_sample / (1 << 18)) <= budget:
        n_sample *= 2
    x, g = inputs(n_sample)
    for _ in range(args.warmup):
        step_fn(x, g)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_fn(x, g)
    dt = (time.perf_counter() - t0) / args.steps
    value = round(gbps(n_sample, dt), 3)
    what = ("the reference's own snnlib/example/gold_op.py (gold_fire + autograd)" if gold is not None
            else "PyTorch-autograd port of the reference's gold_fire (oracle/_ref not installed)")
    sample = f"{what} on {cores} host threads, fwd+bwd, fp32, T=8, N=2^{n_sample.bit_length() - 1} neurons per step"
    print(json.dumps({
        "impl": "reference", "metric": "lif_fwd_bwd_hbm_gbps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD.replace("N=2^26 per GPU", f"N=2^{n_sample.bit_length() - 1} per step (a bounded sample "
                                                "of the GPU arm's 2^26-neuron step; GB/s is size-normalised)"),
                   "T": T_STEPS, "neurons_per_step": n_sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from snn_gpu_training_bptt_b200 import _capi
    from snn_gpu_training_bptt_b200.host_pipeline import HostLifPipeline

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path for the product arm")
    _capi.lib()  # fail loudly if the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    T, N = T_STEPS, 1 << args.log2n
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.randn((T, 1, N), device=dev, generator=gen).add_(0.5)
    g = torch.randn((T, 1, N), device=dev, generator=gen)
    spike = torch.empty_like(x)
    gx = torch.empty_like(x)
    L = _capi.lib()
    px, pg, ps, pgx = (_capi._ptr(t) for t in (x, g, spike, gx))
    stream = torch.cuda.current_stream(dev)
    sp = _capi._stream(dev)

    def step():
        _capi.check("snn_lif_fwd", L.snn_lif_fwd(px, ps, None, None, T, N, 0, ALPHA, THRESH, sp))
        _capi.check("snn_lif_bwd", L.snn_lif_bwd(px, pg, pgx, T, N, 0, ALPHA, THRESH, BETA, INTERVAL, None, 0, sp))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # The K timed steps take ~0.3 s at most; the K-step block (barrier + synchronize on both sides,
    # CUDA events on the launching stream) is repeated until at least MIN_TIMED_MS of device time has
    # been measured, so that the clock sampler sees the GPU under load, and the MEDIAN block is the
    # one reported. Every rank runs the same number of blocks (the decision uses the max over ranks).
    MIN_TIMED_MS, MAX_BLOCKS = 1000.0, 200
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    blocks, timed_ms = [], 0.0
    with ClockSampler(local) as clocks:
        while timed_ms < MIN_TIMED_MS and len(blocks) < MAX_BLOCKS:
            barrier()
            e_start.record(stream)
            for k in range(args.steps):
                ev[k][0].record(stream)
                _capi.check("snn_lif_fwd", L.snn_lif_fwd(px, ps, None, None, T, N, 0, ALPHA, THRESH, sp))
                ev[k][1].record(stream)
                _capi.check("snn_lif_bwd", L.snn_lif_bwd(px, pg, pgx, T, N, 0, ALPHA, THRESH, BETA, INTERVAL, None, 0, sp))
                ev[k][2].record(stream)
            e_end.record(stream)
            barrier()
            blk = [e_start.elapsed_time(e_end), statistics.mean(e[0].elapsed_time(e[1]) for e in ev),
                   statistics.mean(e[1].elapsed_time(e[2]) for e in ev)]
            if world > 1:
                t = torch.tensor(blk, device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                blk = [float(v) for v in t.tolist()]
            blocks.append(blk)
            timed_ms += blk[0]
    total_ms, fwd_ms, bwd_ms = sorted(blocks, key=lambda b: b[0])[len(blocks) // 2]
    ms_per_step = total_ms / args.steps
    value = gbps(N * world, ms_per_step / 1e3)

    # ---- end to end through the host-buffer API: pinned host -> device -> kernels -> host ----
    e2e = None
    e2e_steps = max(2, min(5, args.steps))
    for n_e2e in (() if args.no_e2e else (N, N // 4, N // 16)):
        try:
            hx = torch.empty((T, n_e2e), dtype=torch.float32).pin_memory()
            hg = torch.empty((T, n_e2e), dtype=torch.float32).pin_memory()
            hs = torch.empty((T, n_e2e), dtype=torch.float32).pin_memory()
            hgx = torch.empty((T, n_e2e), dtype=torch.float32).pin_memory()
        except RuntimeError:
            continue
        hx.copy_(x.view(T, N)[:, :n_e2e])
        hg.copy_(g.view(T, N)[:, :n_e2e])
        pipe = HostLifPipeline(T, n_e2e, torch.float32, chunk=1 << 22, lanes=3, device=dev)
        pipe.run(hx, hg, hs, hgx, ALPHA, THRESH, BETA, INTERVAL)       # warm-up
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            pipe.run(hx, hg, hs, hgx, ALPHA, THRESH, BETA, INTERVAL)
        torch.cuda.synchronize(dev)
        dt = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            tt = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        same = bool(torch.equal(hs[:, :4096].to(dev), spike.view(T, N)[:, :4096]))
        copy_ms = _host_link_copy_ms(hx, hg, hs, hgx, dev)
        e2e = {"value": round(gbps(n_e2e * world, dt), 2), "unit": "GB/s",
               "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
               "ms_per_step": round(dt * 1e3, 3), "neurons_per_gpu": n_e2e,
               "launches_per_step": pipe.launches_per_run, "matches_device_run": same,
               "how": "pinned host x,grad -> 3-stream chunked H2D (one pitched copy per [T, chunk] slab) / snn_lif_fwd / snn_lif_bwd / D2H of spike,grad_x",
               "host_link": {"copy_only_ms": round(copy_ms, 3),
                             "gbs_each_way": round(pipe.h2d_bytes / copy_ms / 1e6, 2),
                             "frac": round(copy_ms / (dt * 1e3), 4),
                             "what": "the same bytes copied H2D and D2H at once with no kernels (rank 0's "
                                     "link); frac = that time / the end-to-end step"}}
        del hx, hg, hs, hgx, pipe
        break

    # ---- fused synaptic linear + LIF layer (tensor-core leg), rank 0's GPU -----------------------
    linear_lif = None
    if not args.no_linear_lif:
        del x, g, spike, gx
        torch.cuda.empty_cache()
        if rank == 0:
            with ClockSampler(local) as lin_clocks:
                linear_lif = linear_lif_block(dev, 256, reps=40)
            linear_lif["clocks"] = lin_clocks.summary()
        barrier()

    # ---- second half of the metric: spiking-CNN training samples/sec (data-parallel) ----------
    trainer, trainer_resnet = None, None
    if not args.no_trainer:
        if args.no_linear_lif:
            del x, g, spike, gx
        torch.cuda.empty_cache()
        from snn_gpu_training_bptt_b200.example import train_synthetic

        def trainer_leg(name, time_steps, batch, steps, workload):
            tr = train_synthetic.run(name, time_steps=time_steps, batch=batch, steps=steps, warmup=5, precision="bf16",
                                     bucket_mb=args.bucket_mb)
            leg = {"metric": "spiking_cnn_train_samples_per_s", "value": round(tr["samples_per_s"], 1),
                   "unit": "samples/s", "ms_per_step": round(tr["ms_per_step"], 3),
                   "config": {"workload": workload,
                              "parallelism": f"dp{world}, bucketed NCCL all-reduce overlapped with backward"},
                   "steps": tr["steps"], "params": tr["params"], "final_loss": round(tr["final_loss"], 4),
                   "h2d_bytes_per_step": tr["h2d_bytes_per_step"], "d2h_bytes_per_step": tr["d2h_bytes_per_step"],
                   "grad_bucket_bytes": tr["bucket_bytes"]}
            if world > 1:
                # the same captured step with the all-reduces left out: the difference is the
                # communication time that backward does not hide
                quiet = train_synthetic.run(name, time_steps=time_steps, batch=batch, steps=steps, warmup=5,
                                            precision="bf16", communicate=False, bucket_mb=args.bucket_mb)
                leg["ms_per_step_without_allreduce"] = round(quiet["ms_per_step"], 3)
                leg["exposed_comm_ms"] = round(tr["ms_per_step"] - quiet["ms_per_step"], 3)
            return leg

        trainer = trainer_leg("vgg", 8, 64, args.trainer_steps,
                              "VGG-style spiking CNN (conv 128-128-P-256-256-P-512-512-P, fc 8192-1024-10, "
                              "LIF after every conv/fc), T=8, batch 64 per GPU, synthetic 3x32x32 U(0,1) "
                              "images, SGD momentum 0.9, bf16 synaptic ops + fp32 LIF state")
        if not args.no_resnet:
            trainer_resnet = trainer_leg("resnet19", 16, 128, max(5, args.trainer_steps // 3),
                                         "ResNet-19-style spiking network (3x3 stem, 3/3/2 residual blocks of "
                                         "128/256/512 channels, LIF after every conv and after each add), T=16, "
                                         "batch 128 per GPU, synthetic 3x32x32 U(0,1) images, SGD momentum 0.9, "
                                         "bf16 synaptic ops + fp32 LIF state")

    if rank == 0:
        peak, peak_src = measured_peak()
        bwd_gbs = BYTES_BWD * T * N / (bwd_ms / 1e3) / 1e9
        fwd_gbs = BYTES_FWD * T * N / (fwd_ms / 1e3) / 1e9
        traffic = (NCU_BWD_TRAFFIC_BYTES_PER_STEP * T * N) if NCU_BWD_TRAFFIC_BYTES_PER_STEP else None
        out = {
            "metric": "lif_fwd_bwd_hbm_gbps", "value": round(value, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD if N == NEURONS else WORKLOAD.replace("N=2^26", f"N=2^{args.log2n} (reduced case)"),
                       "T": T, "neurons_per_gpu": N,
                       "bytes_per_neuron_step": BYTES_FWD + BYTES_BWD,
                       "l2": f"inputs larger than L2 ({4 * 4 * T * N / 2**30:g} GiB working set per step, no flush needed)",
                       "parallelism": f"neuron-axis shards x{world}, no collective"},
            "pct_of_measured_hbm_peak": round(100 * value / world / peak, 2),
            "pct_of_nominal_8TBs": round(100 * value / world / NOMINAL_HBM_GBS, 2),
            "kernels": {"lif_fwd_ms": round(fwd_ms, 4), "lif_fwd_gbs": round(fwd_gbs, 1),
                        "lif_bwd_ms": round(bwd_ms, 4), "lif_bwd_gbs": round(bwd_gbs, 1)},
            "roofline": {"bound": "hbm", "kernel": "snn::lif_bwd_kernel<float,2,8>",
                         "achieved": round(bwd_gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(bwd_gbs / peak, 4), "traffic": traffic,
                         "algorithmic_bytes_per_launch": BYTES_BWD * T * N, "peak_source": peak_src},
            "clocks": clocks.summary(),
            "timed_blocks": len(blocks), "timed_region_ms": round(timed_ms, 1),
            "e2e": e2e,
            "gpu_launches": 2 * args.steps,
            "trainer": trainer,
            "trainer_resnet19": trainer_resnet,
            "linear_lif": linear_lif,
        }
        # flat copies of the nested legs (parsers that keep only top-level scalars still see them)
        if linear_lif is not None:
            for k in ("fwd_us", "bwd_us", "fwd_bwd_us", "fwd_tflops", "fwd_bwd_tflops", "fwd_frac", "fwd_bwd_frac"):
                out["linear_lif_" + k] = linear_lif[k]
        for prefix, leg in (("trainer", trainer), ("trainer_resnet19", trainer_resnet)):
            if leg is not None:
                out[prefix + "_samples_per_s"] = leg["value"]
                out[prefix + "_ms_per_step"] = leg["ms_per_step"]
                out[prefix + "_exposed_comm_ms"] = leg.get("exposed_comm_ms")
        if world == 1 and not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline_block()
            if trainer is not None:
                trainer["cpu_baseline"] = cpu_trainer_block()
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_trainer_block():
    """The trainer's network as a plain-PyTorch CPU restatement around the oracle's LIF, a few SGD
    steps at batch 8 on all host cores (the only CPU-runnable form of the reference's training)."""
    from oracle import cpu_trainer
    r = cpu_trainer.time_training(batch=8, steps=2, warmup=1, time_steps=8)
    return {"value": round(r["samples_per_s"], 2), "unit": "samples/s", "cores": r["cores"], "kind": "port",
            "sample": "same VGG-style network, T=8, plain PyTorch ops + autograd port of the reference's "
                      "gold_fire, fp32, batch 8, %d SGD steps, %.0f ms/step" % (r["steps"], r["ms_per_step"])}


# ----------------------------------------------------------------------------------------------
# secondary workloads (not the contract line): bandwidth sweep, BN-fused LIF, linear + LIF
# ----------------------------------------------------------------------------------------------
def _time_kernel(fn, reps, flush=None):
    """Median device time of fn() in ms over `reps` launches (CUDA events on the current stream).
    `flush` (a large tensor) is rewritten before each launch when the working set fits in L2."""
    import torch
    for _ in range(3):
        fn()
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def _host_link_copy_ms(hx, hg, hs, hgx, dev, reps=2, chunk=1 << 22, pitched=True):
    """Time of moving one end-to-end step's bytes over the host link and nothing else: the pinned
    inputs H2D on one stream while as many bytes go D2H into the pinned outputs on another.
    pitched = one transfer per [T, chunk] slab (as the pipeline copies), else T row copies."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi
    T, n = hx.shape
    chunk = min(n, chunk)
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    stage_in = torch.empty((2, T, chunk), dtype=hx.dtype, device=dev)
    stage_out = torch.zeros((2, T, chunk), dtype=hx.dtype, device=dev)
    torch.cuda.synchronize(dev)
    best = float("inf")
    for _ in range(reps + 1):                                   # first pass warms up
        t0 = time.perf_counter()
        for lo in range(0, n, chunk):
            m = min(chunk, n - lo)
            with torch.cuda.stream(up):
                if pitched:
                    _capi.copy_rows_(stage_in[0, :, :m], hx[:, lo:lo + m])
                    _capi.copy_rows_(stage_in[1, :, :m], hg[:, lo:lo + m])
                else:
                    for t in range(T):
                        stage_in[0, t, :m].copy_(hx[t, lo:lo + m], non_blocking=True)
                        stage_in[1, t, :m].copy_(hg[t, lo:lo + m], non_blocking=True)
            with torch.cuda.stream(down):
                if pitched:
                    _capi.copy_rows_(hs[:, lo:lo + m], stage_out[0, :, :m])
                    _capi.copy_rows_(hgx[:, lo:lo + m], stage_out[1, :, :m])
                else:
                    for t in range(T):
                        hs[t, lo:lo + m].copy_(stage_out[0, t, :m], non_blocking=True)
                        hgx[t, lo:lo + m].copy_(stage_out[1, t, :m], non_blocking=True)
        torch.cuda.synchronize(dev)
        best = min(best, (time.perf_counter() - t0) * 1e3)
    return best


def run_host_link(args):
    """What limits the end-to-end (host-buffer) number when several ranks share one host: the same
    host<->device traffic as the e2e leg (2^24 neurons per rank, T=8, fp32: 1 GiB each way per step),
    copies only and with the kernels, under four variants of how the host side is driven. Every
    figure is the max over ranks; GB/s is per rank and direction."""
    import torch
    import torch.distributed as dist
    from snn_gpu_training_bptt_b200.host_pipeline import HostLifPipeline
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, n = T_STEPS, 1 << 24
    cpus = sorted(os.sched_getaffinity(0))
    per = max(1, len(cpus) // max(world, 1))
    rows = []
    for name, pitched, chunk, pin_cpu in (("T row copies per slab, chunk 2^22", False, 1 << 22, False),
                                          ("one pitched copy per slab, chunk 2^22", True, 1 << 22, False),
                                          ("one pitched copy per slab, chunk 2^24", True, 1 << 24, False),
                                          ("pitched, chunk 2^22, rank bound to its own CPU cores before the "
                                           "pinned buffers are allocated and touched", True, 1 << 22, True)):
        if pin_cpu:
            os.sched_setaffinity(0, cpus[rank * per:(rank + 1) * per] or cpus)
        bufs = [torch.empty((T, n), dtype=torch.float32).pin_memory() for _ in range(4)]
        for b in bufs:
            b.zero_()
        bufs[0].normal_(0.5, 1.0)
        bufs[1].normal_(0.0, 1.0)
        if world > 1:
            dist.barrier()
        copy_ms = _host_link_copy_ms(*bufs, dev, reps=2, chunk=chunk, pitched=pitched)
        pipe = HostLifPipeline(T, n, torch.float32, chunk=chunk, lanes=3, device=dev, pitched=pitched)
        pipe.run(*bufs, ALPHA, THRESH, BETA, INTERVAL)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(3):
            pipe.run(*bufs, ALPHA, THRESH, BETA, INTERVAL)
        torch.cuda.synchronize(dev)
        e2e_ms = (time.perf_counter() - t0) / 3 * 1e3
        if world > 1:
            t = torch.tensor([copy_ms, e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            copy_ms, e2e_ms = float(t[0]), float(t[1])
        nbytes = 2 * T * n * 4
        rows.append({"variant": name, "copy_only_ms": round(copy_ms, 2), "copy_gbs_each_way_per_rank": round(nbytes / copy_ms / 1e6, 2),
                     "e2e_ms": round(e2e_ms, 2), "e2e_gbs_aggregate": round(gbps(n * world, e2e_ms / 1e3), 2)})
        del bufs, pipe
        if pin_cpu:
            os.sched_setaffinity(0, cpus)
    if rank == 0:
        print(json.dumps({"metric": "host_link_gbs", "n_gpus": world, "cpus_visible": len(cpus),
                          "config": {"workload": "host<->device traffic of the e2e leg, T=8, 2^24 neurons per rank, fp32"},
                          "rows": rows}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _time_graphed(fn, reps=20, per_graph=10):
    """Device time per call of fn() in ms with the host out of the picture: `per_graph` calls are
    captured into one CUDA graph and the graph is replayed `reps` times (median). For kernels of a
    few tens of microseconds the Python / launch overhead of an eager call is longer than the
    kernel, so eager event timing would measure the host."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(per_graph):
            fn()
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph.replay()
    for _ in range(reps):
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / per_graph)
    return statistics.median(times)


def run_sweep(args):
    """Single-GPU bandwidth sweep: T in {4,8,16} x N in {2^20,2^22,2^24,2^26}, fp32 and bf16 I/O.
    A case whose four tensors exceed 512 MiB is timed launch by launch (inputs larger than L2). A
    smaller case is timed as a stream of launches over R rotating sets of buffers that together
    exceed 768 MiB - every launch meets cold inputs, and the launch overhead of one call hides
    behind the execution of the call before it, as it does for the layers of a network - with
    `single_launch_*` = the same kernels timed one launch at a time after an L2 flush (which adds
    the ~5 us of an isolated launch to kernels of 10-20 us)."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi
    peak, peak_src = measured_peak()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    L, sp = _capi.lib(), _capi._stream(dev)
    for dtype, name, es in ((torch.float32, "f32", 4), (torch.bfloat16, "bf16", 2)):
        for T in (4, 8, 16):
            for lg in (20, 22, 24, 26):
                N = 1 << lg
                set_bytes = 4 * T * N * es
                small = set_bytes < (512 << 20)
                R = max(2, -(-(768 << 20) // set_bytes)) if small else 1
                gen = torch.Generator(device=dev).manual_seed(1234)
                sets = []
                for _ in range(R):
                    x = (torch.randn((T, 1, N), device=dev, generator=gen) + 0.5).to(dtype)
                    g = torch.randn((T, 1, N), device=dev, generator=gen).to(dtype)
                    sets.append((x, g, torch.empty_like(x), torch.empty_like(x)))
                code = _capi.DTYPE_CODE[dtype]
                ptrs = [tuple(_capi._ptr(t) for t in st) for st in sets]

                def fwd(k=0):
                    px, pg, ps, pgx = ptrs[k]
                    return L.snn_lif_fwd(px, ps, None, None, T, N, code, ALPHA, THRESH, sp)

                def bwd(k=0):
                    px, pg, ps, pgx = ptrs[k]
                    return L.snn_lif_bwd(px, pg, pgx, T, N, code, ALPHA, THRESH, BETA, INTERVAL, None, 0, sp)

                gb = lambda nbytes, ms: nbytes * T * N / ms / 1e6
                extra = {}
                if small:
                    def stream_ms(fn):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        times = []
                        for rep in range(6):
                            e0.record()
                            for k in range(R):
                                fn(k)
                            e1.record()
                            e1.synchronize()
                            if rep:                       # the first pass warms up
                                times.append(e0.elapsed_time(e1) / R)
                        return statistics.median(times)
                    t_f, t_b = stream_ms(fwd), stream_ms(bwd)
                    s_f, s_b = _time_kernel(fwd, 20, flush), _time_kernel(bwd, 20, flush)
                    extra = {"single_launch_fwd_ms": round(s_f, 4), "single_launch_bwd_ms": round(s_b, 4),
                             "single_launch_gbs": round(gb(5 * es, s_f + s_b), 1), "rotating_sets": R}
                else:
                    t_f, t_b = _time_kernel(fwd, 20), _time_kernel(bwd, 20)
                tot = gb(5 * es, t_f + t_b)
                print(json.dumps({
                    "metric": "lif_fwd_bwd_hbm_gbps", "value": round(tot, 1), "unit": "GB/s", "dtype": name,
                    "config": {"workload": f"lif sweep {name} T={T} N=2^{lg}",
                               "l2": f"{R} rotating buffer sets ({R * set_bytes >> 20} MiB) > L2, launches back to back"
                                     if small else "working set > L2"},
                    "fwd_ms": round(t_f, 4), "fwd_gbs": round(gb(2 * es, t_f), 1),
                    "bwd_ms": round(t_b, 4), "bwd_gbs": round(gb(3 * es, t_b), 1),
                    "frac_of_peak": round(tot / peak, 4), "peak": peak, "peak_source": peak_src, **extra}))
                del sets, ptrs


def run_bn_lif(args):
    """BN-fused LIF forward + two-pass backward, fp32, T=8, N = 2^26: contiguous [B=256, C=256, 32x32]
    images (channel runs of 1024 neurons) and the same tensor in channels-last memory order
    (every neuron its own channel run: the layout of the trainer's images and of [T, B, C] inputs)."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi
    peak, peak_src = measured_peak()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, B, C, HW = 8, 256 >> (26 - args.log2n), 256, 1024
    N = B * C * HW
    L, sp, P = _capi.lib(), _capi._stream(dev), _capi._ptr
    for layout, inner, shape, dims in (("contiguous [T,B,C,H,W], inner = H*W", HW, (T, B, C, 32, 32), (0, 1, 3, 4)),
                                       ("channels-last [T,B,H,W,C], inner = 1", 1, (T, B, 32, 32, C), (0, 1, 2, 3))):
        gen = torch.Generator(device=dev).manual_seed(1234)
        x = torch.randn(shape, device=dev, generator=gen) * 1.5 + 0.3
        g = torch.randn(shape, device=dev, generator=gen)
        w = torch.rand(C, device=dev, generator=gen) + 0.5
        b = torch.randn(C, device=dev, generator=gen) * 0.2
        var, mean = torch.var_mean(x, dim=dims, unbiased=False)
        out, gx = torch.empty_like(x), torch.empty_like(x)
        ivar = torch.empty_like(w)
        sums = torch.empty((2, C), device=dev)
        means = torch.empty((2, C), device=dev)
        fwd = lambda: L.snn_bn_lif_fwd(P(x), P(w), P(b), P(var), P(mean), 1e-5, P(out), None, P(ivar), T, N, C, inner, 0, 1,
                                       ALPHA, THRESH, sp)
        assert fwd() == 0

        def bwd():
            rc = L.snn_bn_lif_bwd_sums(P(x), P(g), P(w), P(b), P(ivar), P(mean), P(sums[0]), P(sums[1]), T, N, C, inner, 0, 1,
                                       ALPHA, THRESH, BETA, INTERVAL, sp)
            rc |= L.snn_bn_channel_means(P(sums[0]), P(sums[1]), P(w), P(means[0]), P(means[1]), C, float(T * N // C), sp)
            rc |= L.snn_bn_lif_bwd_input(P(x), P(g), P(w), P(b), P(ivar), P(mean), P(means[0]), P(means[1]), P(gx), T, N, C,
                                         inner, 0, 1, ALPHA, THRESH, BETA, INTERVAL, sp)
            assert rc == 0

        def sums_only():
            assert L.snn_bn_lif_bwd_sums(P(x), P(g), P(w), P(b), P(ivar), P(mean), P(sums[0]), P(sums[1]), T, N, C, inner, 0, 1,
                                         ALPHA, THRESH, BETA, INTERVAL, sp) == 0
        reps = args.steps if args.steps < 50 else 20
        t_f, t_b, t_s = _time_kernel(fwd, reps), _time_kernel(bwd, reps), _time_kernel(sums_only, reps)
        gb = lambda nbytes, ms: nbytes * T * N / ms / 1e6
        print(json.dumps({
            "metric": "bn_lif_fwd_bwd_hbm_gbps", "value": round(gb(28, t_f + t_b), 1), "unit": "GB/s", "dtype": "f32",
            "config": {"workload": f"bn_fire fwd + 2-pass bwd fp32 T=8 B={B} C=256 32x32 N=2^{args.log2n}, {layout}",
                       "bytes_per_neuron_step": "fwd 8, bwd sums pass 8 + input pass 12",
                       "l2": "working set > L2"},
            "fwd_ms": round(t_f, 4), "fwd_gbs": round(gb(8, t_f), 1), "bwd_ms": round(t_b, 4),
            "bwd_gbs": round(gb(20, t_b), 1), "bwd_sums_pass_ms": round(t_s, 4), "bwd_sums_pass_gbs": round(gb(8, t_s), 1),
            "frac_of_peak": round(gb(28, t_f + t_b) / peak, 4), "peak": peak, "peak_source": peak_src,
            "reference_traffic_bytes_per_neuron_step": "8 fwd + 8 (u rebuild) + 12 (sums) + 16 (input grad) = 44"}))
        del x, g, out, gx


def run_lif_add(args):
    """LIF of a sum of two currents (residual blocks), fused kernels against add -> LIF, one line per
    (dtype, T); N = 2^(log2n - 2) neurons so that every tensor is larger than L2."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi
    peak, peak_src = measured_peak()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    N = 1 << (args.log2n - 2)
    reps = args.steps if args.steps < 50 else 20
    for dtype, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        for T in (8, 16):
            gen = torch.Generator(device=dev).manual_seed(1234)
            a = (torch.randn((T, N), device=dev, generator=gen) * 0.7 + 0.3).to(dtype)
            b = (torch.randn((T, N), device=dev, generator=gen) * 0.7 + 0.2).to(dtype)
            g = torch.randn((T, N), device=dev, generator=gen).to(dtype)
            total = a + b
            spike = _capi.lif_add_fwd(a, b, ALPHA, THRESH)
            grad = _capi.lif_add_bwd(a, b, g, ALPHA, THRESH, BETA, INTERVAL)
            same = bool(torch.equal(spike, _capi.lif_fwd(total, ALPHA, THRESH)[0])
                        and torch.equal(grad, _capi.lif_bwd(total, g, ALPHA, THRESH, BETA, INTERVAL)))
            del spike, grad
            t_ff = _time_kernel(lambda: _capi.lif_add_fwd(a, b, ALPHA, THRESH), reps)
            t_fb = _time_kernel(lambda: _capi.lif_add_bwd(a, b, g, ALPHA, THRESH, BETA, INTERVAL), reps)
            t_uf = _time_kernel(lambda: _capi.lif_fwd(torch.add(a, b, out=total), ALPHA, THRESH), reps)
            t_ub = _time_kernel(lambda: _capi.lif_bwd(total, g, ALPHA, THRESH, BETA, INTERVAL), reps)
            es = a.element_size()
            gb = lambda elems, ms: elems * es * T * N / ms / 1e6
            print(json.dumps({
                "metric": "lif_add_fwd_bwd_hbm_gbps", "value": round(gb(7, t_ff + t_fb), 1), "unit": "GB/s", "dtype": name,
                "config": {"workload": f"LIF(a + b) fused fwd + bwd, {name}, T={T}, N=2^{args.log2n - 2}",
                           "elements_per_neuron_step": "fused fwd 3, bwd 4; unfused add 3 + fwd 2, bwd 3",
                           "l2": "every tensor larger than L2"},
                "equals_add_then_lif": same,
                "fwd_ms": round(t_ff, 4), "fwd_gbs": round(gb(3, t_ff), 1), "bwd_ms": round(t_fb, 4),
                "bwd_gbs": round(gb(4, t_fb), 1), "unfused_add_fwd_ms": round(t_uf, 4), "unfused_bwd_ms": round(t_ub, 4),
                "fused_over_unfused_time": round((t_ff + t_fb) / (t_uf + t_ub), 4),
                "frac_of_peak": round(gb(7, t_ff + t_fb) / peak, 4), "peak": peak, "peak_source": peak_src}))
            del a, b, g, total


def bf16_peak_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, cuBLAS burst)"
    except Exception:
        return 1590.0, "fallback (no MEASURED_PEAKS.json)"


def linear_lif_block(dev, batch=256, reps=20, with_library=False, eager_steps=0):
    """Fused synaptic linear + LIF layer (T=8, batch 256, 2048 -> 2048; Bernoulli(0.2) input spikes,
    Kaiming-uniform weights, bf16 operands): device time of the forward kernel, of the backward pair
    (dU kernel + the persistent kernel with both gradient GEMMs) and of both, through the C ABI,
    by CUDA-graph replay (a launch of ~15 us cannot be timed eagerly from Python)."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi
    T, B, K, M = 8, batch, 2048, 2048
    L, sp, P = _capi.lib(), _capi._stream(dev), _capi._ptr
    torch.manual_seed(1234)
    lin = torch.nn.Linear(K, M).to(dev)
    x = (torch.rand((T, B, K), device=dev) < 0.2).to(torch.bfloat16)
    w = lin.weight.detach().to(torch.bfloat16)
    bias = lin.bias.detach().float()
    gs = torch.randn((T, B, M), device=dev).to(torch.bfloat16)
    cur, spk = torch.empty((T, B, M), dtype=torch.bfloat16, device=dev), torch.empty((T, B, M), dtype=torch.bfloat16, device=dev)
    gx, gw, gb = torch.empty_like(x), torch.empty((M, K), device=dev), torch.empty(M, device=dev)
    need = L.snn_linear_lif_bwd_workspace_bytes(T, B, K, M, 1)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)

    def fwd():
        # torch.cuda.graph captures on a side stream: look the current stream up at call time
        rc = L.snn_linear_lif_fwd(P(x), P(w), P(bias), P(cur), P(spk), T, B, K, M, 1, ALPHA, THRESH, _capi._stream(dev))
        assert rc == 0, rc

    def bwd(want_gemms=True):
        rc = L.snn_linear_lif_bwd(P(x), P(w), P(cur), P(gs), P(gx) if want_gemms else None, P(gw) if want_gemms else None,
                                  P(gb) if want_gemms else None, T, B, K, M, 1, 0, ALPHA, THRESH, BETA, INTERVAL,
                                  P(ws), need, _capi._stream(dev))
        assert rc == 0, rc

    fwd()
    torch.cuda.synchronize(dev)
    if eager_steps:
        # a handful of plain launches and nothing else: the form a profiler capture wants
        for _ in range(eager_steps):
            fwd()
            bwd()
        torch.cuda.synchronize(dev)
        assert _capi.linear_lif_error() == 0
        return {"workload": "fc 2048->2048 + LIF, T=8, batch %d" % B, "eager_steps": eager_steps, "launches": 3 * eager_steps + 1}
    t_f = _time_graphed(fwd, reps)
    t_b = _time_graphed(bwd, reps)
    t_du = _time_graphed(lambda: bwd(False), reps)
    t_fb = _time_graphed(lambda: (fwd(), bwd()), reps)
    assert _capi.linear_lif_error() == 0
    peak, peak_src = bf16_peak_tflops()
    flops = 2.0 * T * B * K * M
    tf = lambda n, ms: n * flops / ms / 1e9
    out = {"workload": f"fc 2048->2048 + LIF, T=8, batch {B}, bf16 operands, fp32 accumulation and LIF state",
           "fwd_us": round(t_f * 1e3, 2), "bwd_us": round(t_b * 1e3, 2), "fwd_bwd_us": round(t_fb * 1e3, 2),
           "bwd_du_kernel_us": round(t_du * 1e3, 2),
           "fwd_tflops": round(tf(1, t_f), 1), "bwd_tflops": round(tf(2, t_b), 1), "fwd_bwd_tflops": round(tf(3, t_fb), 1),
           "fwd_frac": round(tf(1, t_f) / peak, 4), "bwd_frac": round(tf(2, t_b) / peak, 4),
           "fwd_bwd_frac": round(tf(3, t_fb) / peak, 4), "peak_tflops": peak, "peak_source": peak_src,
           "kernels": ["linear_lif_fwd_persistent_kernel<8,256>", "lif_du_kernel<8,8>", "bwd_gemm_pair_kernel"],
           "l2": "not flushed: the layer's ~50 MB of operands and outputs stay in the 126 MB L2 between replays, as "
                 "they do between adjacent layers of a training step",
           "launches_per_step": 3, "how": "CUDA-graph replay of 10 calls, median of %d replays" % reps}
    if with_library:
        xr, wr = x.view(T * B, K), w
        t_lib = _time_graphed(lambda: torch.nn.functional.linear(xr, wr), reps)
        out["cublas_gemm_alone_us"] = round(t_lib * 1e3, 2)
    return out


def run_linear_lif(args):
    """Synaptic linear followed by LIF (T=8, batch 256, 2048 -> 2048): the library's own kernels
    through the C ABI, then the same layer through the autograd ops (fused FcFire against the
    unfused library-GEMM composition) in bf16 and fp32."""
    import torch
    from snn_gpu_training_bptt_b200 import _capi, snnlib, snnlib_func as sf
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    if args.eager_steps:
        print(json.dumps(linear_lif_block(dev, args.batch, eager_steps=args.eager_steps)))
        return
    with ClockSampler(0) as clocks:
        block = linear_lif_block(dev, args.batch, with_library=True)
    block["clocks"] = clocks.summary()
    print(json.dumps({"metric": "linear_lif_fwd_bwd_tflops", "value": block["fwd_bwd_tflops"], "unit": "TFLOP/s",
                      "dtype": "bf16", "config": {"workload": block["workload"]}, "linear_lif": block}))
    T, B, K, M = 8, args.batch, 2048, 2048
    torch.manual_seed(1234)
    lin = torch.nn.Linear(K, M).to(dev)
    all_flops = 2.0 * T * B * K * M * 3
    peak_tf, _ = bf16_peak_tflops()
    for dtype, name in ((torch.bfloat16, "bf16"), (torch.float32, "fp32 (TF32 off)")):
        x = (torch.rand((T, B, K), device=dev) < 0.2).to(dtype).requires_grad_(True)
        w = lin.weight.detach().clone().requires_grad_(True)
        b = lin.bias.detach().clone().requires_grad_(True)
        gs = torch.randn((T, B, M), device=dev).to(dtype)
        for label, op in (("FcFire op (tcgen05 kernels where supported; fp32 master weight cast per step)", lambda: sf.fc_fire_func(x, w, b)),
                          ("fire_func(fc_func(x)) (library GEMMs + LIF kernels)", lambda: sf.fire_func(sf.fc_func(x, w, b)))):
            def step():
                x.grad = w.grad = b.grad = None
                op().backward(gs)
            ms = _time_graphed(step)
            tf = all_flops / ms / 1e9
            print(json.dumps({"metric": "linear_lif_fwd_bwd_tflops", "value": round(tf, 1), "unit": "TFLOP/s", "dtype": name,
                              "ms": round(ms, 4), "frac_of_bf16_burst_peak": round(tf / peak_tf, 4),
                              "config": {"workload": "fc 2048->2048 + LIF, T=8, batch %d" % B, "path": label}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--batch", type=int, default=256, help="batch size of --workload linear_lif (a multiple of 32)")
    ap.add_argument("--eager-steps", type=int, default=0,
                    help="--workload linear_lif only: run this many plain forward+backward steps and exit (for profiler captures)")
    ap.add_argument("--no-trainer", action="store_true", help="skip the spiking-CNN training legs")
    ap.add_argument("--no-resnet", action="store_true", help="skip the ResNet-19-style training leg")
    ap.add_argument("--bucket-mb", type=float, default=64.0,
                    help="gradient bucket size of the training legs (MB); 64 = one big bucket plus the small tail bucket, "
                         "the fastest of 25 / 40 / 64 measured at 8 GPUs (3.614 / 3.602 / 3.586 ms per step)")
    ap.add_argument("--no-linear-lif", action="store_true", help="skip the fused linear + LIF (tensor-core) leg")
    ap.add_argument("--trainer-steps", type=int, default=30)
    ap.add_argument("--log2n", type=int, default=26,
                    help="log2 of neurons per GPU (26 = the benchmark size; smaller only for profiler captures)")
    ap.add_argument("--workload", default="lif", choices=["lif", "sweep", "bn_lif", "linear_lif", "host_link", "lif_add"],
                    help="lif = the benchmark line; the others are secondary single-GPU measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "sweep":
        run_sweep(args)
    elif args.workload == "bn_lif":
        run_bn_lif(args)
    elif args.workload == "linear_lif":
        run_linear_lif(args)
    elif args.workload == "host_link":
        run_host_link(args)
    elif args.workload == "lif_add":
        run_lif_add(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
