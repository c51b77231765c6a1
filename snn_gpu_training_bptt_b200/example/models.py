"""Spiking networks built from the snnlib_op layers.

Conventions follow the reference's snnlib/example/models.py: the image batch is
direct-encoded by repeating it over T time steps (``torch.stack([x] * T)``, reference
models.py:42), every layer works on time-major [T, B, C, H, W] / [T, B, C] tensors, and the
classifier reads the time-averaged activity (``fc(x.mean(dim=0))``, reference models.py:59).

``SpikingVGG`` and ``SpikingResNet19`` are the BN-free benchmark networks (synthetic 3x32x32
images, 10 classes); their LIF layers are the plain ``Fire`` path. Activations run in
``act_dtype`` (bf16 by default: 16-bit synaptic convolutions / GEMMs through cuDNN / cuBLAS on
channels-last tensors, fp32 LIF state inside the kernels, fp32 master parameters).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import snnlib_func as sf
from .. import snnlib_op as sop


def _pool(x, k=2):
    """AvgPool2d(k) applied to every time step of [T, B, C, H, W]."""
    T, B = x.shape[0], x.shape[1]
    y = F.avg_pool2d(x.reshape((T * B,) + tuple(x.shape[2:])), k)
    return y.view((T, B) + tuple(y.shape[1:]))


def _encode(images, T, act_dtype):
    """[B, 3, H, W] -> direct-encoded [T, B, 3, H, W] in channels-last memory order."""
    x = images.to(act_dtype).contiguous(memory_format=torch.channels_last)
    B = x.shape[0]
    rep = x.unsqueeze(0).expand((T,) + tuple(x.shape)).reshape((T * B,) + tuple(x.shape[1:]))
    rep = rep.contiguous(memory_format=torch.channels_last)
    return rep.view((T, B) + tuple(x.shape[1:]))


class SpikingVGG(nn.Module):
    """conv3x3 128-128-pool-256-256-pool-512-512-pool, LIF after every conv, then
    fc 8192->1024 - LIF - fc 1024->classes on the time-averaged spikes."""

    def __init__(self, time_steps=8, num_classes=10, act_dtype=torch.bfloat16, widths=(128, 256, 512),
                 image=32, hidden=1024):
        super().__init__()
        self.T, self.act_dtype = time_steps, act_dtype
        w1, w2, w3 = widths
        self.conv1_1 = sop.Conv(3, w1)
        self.conv1_2 = sop.FireConv(w1, w1)        # LIF of conv1_1's current, then conv
        self.fire1 = sop.Fire()
        self.conv2_1 = sop.Conv(w1, w2)
        self.conv2_2 = sop.FireConv(w2, w2)
        self.fire2 = sop.Fire()
        self.conv3_1 = sop.Conv(w2, w3)
        self.conv3_2 = sop.FireConv(w3, w3)
        self.fire3 = sop.Fire()
        feat = w3 * (image // 8) ** 2
        self.fc1 = sop.Fc(feat, hidden)
        self.fire_fc = sop.Fire()
        self.fc2 = nn.Linear(hidden, num_classes)

    def forward(self, images):
        x = _encode(images, self.T, self.act_dtype)
        x = _pool(self.fire1(self.conv1_2(self.conv1_1(x))))
        x = _pool(self.fire2(self.conv2_2(self.conv2_1(x))))
        x = _pool(self.fire3(self.conv3_2(self.conv3_1(x))))
        x = x.reshape(x.shape[0], x.shape[1], -1)          # [T, B, C*H*W] in (C, H, W) order
        x = self.fire_fc(self.fc1(x))
        return self.fc2(x.mean(dim=0).float())


class _ResBlock(nn.Module):
    """conv-LIF-conv, add the shortcut current, LIF (a LIF after every conv and after the add)."""

    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1 = sop.Conv(cin, cout, stride=(stride, stride))
        self.conv2 = sop.FireConv(cout, cout)
        self.fire = sop.Fire()
        self.short = None
        if stride != 1 or cin != cout:
            self.short = sop.Conv(cin, cout, kernel_size=(1, 1), stride=(stride, stride), padding=(0, 0))

    def forward(self, spikes):
        cur = self.conv2(self.conv1(spikes))
        skip = spikes if self.short is None else self.short(spikes)
        return self.fire(cur + skip)


class SpikingResNet19(nn.Module):
    """ResNet-19-style: 3x3 stem (128), stages of 3/3/2 residual blocks with 128/256/512
    channels (stride 2 between stages), global average pool, fc 512->256 - LIF - fc->classes."""

    def __init__(self, time_steps=16, num_classes=10, act_dtype=torch.bfloat16, widths=(128, 256, 512),
                 blocks=(3, 3, 2), hidden=256):
        super().__init__()
        self.T, self.act_dtype = time_steps, act_dtype
        self.stem = sop.Conv(3, widths[0])
        self.stem_fire = sop.Fire()
        layers, cin = [], widths[0]
        for stage, (w, n) in enumerate(zip(widths, blocks)):
            for b in range(n):
                layers.append(_ResBlock(cin, w, 2 if (b == 0 and stage > 0) else 1))
                cin = w
        self.blocks = nn.ModuleList(layers)
        self.fc1 = sop.Fc(cin, hidden)
        self.fire_fc = sop.Fire()
        self.fc2 = nn.Linear(hidden, num_classes)

    def forward(self, images):
        x = self.stem_fire(self.stem(_encode(images, self.T, self.act_dtype)))
        for blk in self.blocks:
            x = blk(x)
        x = x.mean(dim=(3, 4))                              # global average pool -> [T, B, C]
        x = self.fire_fc(self.fc1(x))
        return self.fc2(x.mean(dim=0).float())


def build(name, **kw):
    if name == "vgg":
        return SpikingVGG(**kw)
    if name == "resnet19":
        return SpikingResNet19(**kw)
    raise ValueError(f"unknown model {name!r}")
