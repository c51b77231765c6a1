"""CPU restatement of the benchmark's spiking VGG training step (test / baseline infrastructure).

The network of the trainer benchmark written with plain PyTorch ops, one time step at a time,
around the oracle's autograd LIF (``lif_oracle.torch_fire``, the port of the reference's
snnlib/example/gold_op.py:17-44): conv3x3 w1-w1-pool-w2-w2-pool-w3-w3-pool with a LIF after every
convolution and AvgPool2d(2) per time step, fc -> LIF -> fc on the time-averaged spikes,
cross-entropy loss, SGD with momentum. Layer structure and initialisation follow the reference's
``Conv`` / ``Fc`` modules (snnlib/example/snnlib_op.py:142-150, 213-228).

Only ``bench.py``'s CPU-baseline leg and the tests use this file; the library never imports it.
"""
import math
import os
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import lif_oracle as orc


def _fire(x):
    return orc.torch_fire(x)[1]


def _steps(fn, x):
    return torch.stack([fn(x[t]) for t in range(x.shape[0])])


class GoldSpikingVGG(nn.Module):
    def __init__(self, time_steps=8, num_classes=10, widths=(128, 256, 512), image=32, hidden=1024):
        super().__init__()
        self.T = time_steps
        chans = [3, widths[0], widths[0], widths[1], widths[1], widths[2], widths[2]]
        self.convs = nn.ModuleList()
        for cin, cout in zip(chans[:-1], chans[1:]):
            conv = nn.Conv2d(cin, cout, 3, padding=1)
            nn.init.normal_(conv.weight, 0.0, 0.75 / math.sqrt(cin))
            nn.init.zeros_(conv.bias)
            self.convs.append(conv)
        feat = widths[2] * (image // 8) ** 2
        self.fc1 = nn.Linear(feat, hidden)
        nn.init.normal_(self.fc1.weight, 0.0, 0.75 / math.sqrt(feat))
        nn.init.zeros_(self.fc1.bias)
        self.fc2 = nn.Linear(hidden, num_classes)

    def forward(self, images):
        x = torch.stack([images] * self.T)                       # direct encoding
        for i, conv in enumerate(self.convs):
            x = _fire(_steps(conv, x))
            if i % 2 == 1:
                x = _steps(lambda a: F.avg_pool2d(a, 2), x)
        x = x.reshape(x.shape[0], x.shape[1], -1)
        x = _fire(_steps(self.fc1, x))
        return self.fc2(x.mean(dim=0))


def time_training(batch=8, steps=3, warmup=1, time_steps=8, threads=None, seed=0, **model_kwargs):
    """Samples/s of SGD steps on synthetic U(0,1) 3x32x32 images with uniform labels.

    Returns {"samples_per_s", "ms_per_step", "cores", "batch", "steps", "final_loss"}.
    """
    threads = threads or os.cpu_count() or 1
    previous = torch.get_num_threads()
    torch.set_num_threads(threads)
    try:
        return _time_training(batch, steps, warmup, time_steps, threads, seed, model_kwargs)
    finally:
        torch.set_num_threads(previous)


def _time_training(batch, steps, warmup, time_steps, threads, seed, model_kwargs):
    gen = torch.Generator().manual_seed(seed)
    torch.manual_seed(seed)
    net = GoldSpikingVGG(time_steps=time_steps, **model_kwargs)
    image = model_kwargs.get("image", 32)
    opt = torch.optim.SGD(net.parameters(), lr=0.01, momentum=0.9)
    images = torch.rand((batch, 3, image, image), generator=gen)
    labels = torch.randint(0, 10, (batch,), generator=gen)
    loss = None
    t0 = time.perf_counter()
    for i in range(warmup + steps):
        if i == warmup:
            t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(net(images), labels)
        loss.backward()
        opt.step()
    dt = (time.perf_counter() - t0) / max(1, steps)
    return {"samples_per_s": batch / dt, "ms_per_step": dt * 1e3, "cores": threads, "batch": batch,
            "steps": steps, "final_loss": float(loss.detach())}
