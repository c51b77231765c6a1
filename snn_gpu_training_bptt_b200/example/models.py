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
                 image=32, hidden=1024, fused_pool=True, fused_fc=True):
        super().__init__()
        self.T, self.act_dtype = time_steps, act_dtype
        self.fused_fc = fused_fc
        self.fused_pool = fused_pool and time_steps <= 16
        w1, w2, w3 = widths
        lif_pool = sop.FirePool if self.fused_pool else sop.Fire
        self.conv1_1 = sop.Conv(3, w1)
        self.conv1_2 = sop.FireConv(w1, w1)        # LIF of conv1_1's current, then conv
        self.fire1 = lif_pool()
        self.conv2_1 = sop.Conv(w1, w2)
        self.conv2_2 = sop.FireConv(w2, w2)
        self.fire2 = lif_pool()
        self.conv3_1 = sop.Conv(w2, w3)
        self.conv3_2 = sop.FireConv(w3, w3)
        self.fire3 = lif_pool()
        feat = w3 * (image // 8) ** 2
        # fc1 + its LIF as one op (the tcgen05 linear + LIF kernels for bf16 activations); the
        # parameters keep the names of an Fc layer either way
        self.fc1 = sop.FcFire(feat, hidden) if fused_fc else sop.Fc(feat, hidden)
        self.fire_fc = sop.Fire()
        self.fc2 = nn.Linear(hidden, num_classes)

    def forward(self, images):
        pool = (lambda t: t) if self.fused_pool else _pool      # FirePool already pooled
        x = _encode(images, self.T, self.act_dtype)
        x = pool(self.fire1(self.conv1_2(self.conv1_1(x))))
        x = pool(self.fire2(self.conv2_2(self.conv2_1(x))))
        x = pool(self.fire3(self.conv3_2(self.conv3_1(x))))
        x = x.reshape(x.shape[0], x.shape[1], -1)          # [T, B, C*H*W] in (C, H, W) order
        x = self.fc1(x) if self.fused_fc else self.fire_fc(self.fc1(x))
        return self.fc2(x.mean(dim=0).float())


class _ResBlock(nn.Module):
    """conv-LIF-conv, add the shortcut current, LIF (a LIF after every conv and after the add)."""

    def __init__(self, cin, cout, stride, fused_add=True):
        super().__init__()
        self.fused_add = fused_add
        self.conv1 = sop.Conv(cin, cout, stride=(stride, stride))
        self.conv2 = sop.FireConv(cout, cout)
        self.fire = sop.FireAdd() if fused_add else sop.Fire()
        self.short = None
        if stride != 1 or cin != cout:
            self.short = sop.Conv(cin, cout, kernel_size=(1, 1), stride=(stride, stride), padding=(0, 0))

    def forward(self, spikes):
        cur = self.conv2(self.conv1(spikes))
        skip = spikes if self.short is None else self.short(spikes)
        return self.fire(cur, skip) if self.fused_add else self.fire(cur + skip)


class SpikingResNet19(nn.Module):
    """ResNet-19-style: 3x3 stem (128), stages of 3/3/2 residual blocks with 128/256/512
    channels (stride 2 between stages), global average pool, fc 512->256 - LIF - fc->classes."""

    def __init__(self, time_steps=16, num_classes=10, act_dtype=torch.bfloat16, widths=(128, 256, 512),
                 blocks=(3, 3, 2), hidden=256, fused_fc=True, fused_add=True):
        super().__init__()
        self.T, self.act_dtype = time_steps, act_dtype
        self.fused_fc = fused_fc
        self.stem = sop.Conv(3, widths[0])
        self.stem_fire = sop.Fire()
        layers, cin = [], widths[0]
        for stage, (w, n) in enumerate(zip(widths, blocks)):
            for b in range(n):
                layers.append(_ResBlock(cin, w, 2 if (b == 0 and stage > 0) else 1, fused_add))
                cin = w
        self.blocks = nn.ModuleList(layers)
        self.fc1 = sop.FcFire(cin, hidden) if fused_fc else sop.Fc(cin, hidden)
        self.fire_fc = sop.Fire()
        self.fc2 = nn.Linear(hidden, num_classes)

    def forward(self, images):
        x = self.stem_fire(self.stem(_encode(images, self.T, self.act_dtype)))
        for blk in self.blocks:
            x = blk(x)
        x = x.mean(dim=(3, 4))                              # global average pool -> [T, B, C]
        x = self.fc1(x) if self.fused_fc else self.fire_fc(self.fc1(x))
        return self.fc2(x.mean(dim=0).float())


# ------------------------------------------------------------------------------------------
# The reference's own (batch-norm based) networks, with its attribute names so that state
# dicts saved by the reference's scripts load here and vice versa (reference models.py:8-191).
# T is read from snnlib_func.time_step at call time, as the reference does.
# ------------------------------------------------------------------------------------------
class _BnNet(nn.Module):
    """Shared: direct encoding over snnlib_func.time_step steps and the train_bn switch."""

    def _encode(self, images):
        return images.unsqueeze(0).expand((sf.time_step,) + tuple(images.shape)).contiguous()

    def _bn_layers(self):
        return [m for m in self.modules() if hasattr(m, "train_bn")]

    def set_bn(self, train_bn):
        """True: normalise with batch statistics and update the running ones; False: use the
        running statistics (reference models.py:37-39)."""
        for layer in self._bn_layers():
            layer.train_bn = train_bn


class CIFAR_BN(_BnNet):
    """9 conv (stride-2 convs instead of pooling) + 2 fc + BN-LIF + linear, 32x32 inputs.
    Reference: models.py:8-60."""

    def __init__(self):
        super().__init__()
        self.conv1_1 = sop.Conv(3, 128)
        plan = [("conv1_2", 128, 128, 1), ("conv1_3", 128, 128, 2), ("conv2_1", 128, 256, 1),
                ("conv2_2", 256, 256, 1), ("conv2_3", 256, 256, 2), ("conv3_1", 256, 512, 1),
                ("conv3_2", 512, 512, 1), ("conv3_3", 512, 512, 2)]
        for name, cin, cout, stride in plan:
            setattr(self, name, sop.BnFireConv(cin, cout, stride=(stride, stride)))
        self._conv_order = ["conv1_1"] + [p[0] for p in plan]
        self.fc1 = sop.BnFireFc(4 * 4 * 512, 1024, dim_bn=(0, 1, 3, 4), cin_bn=512)
        self.fc2 = sop.BnFireFc(1024, 512, dim_bn=(0, 1))
        self.bn = sop.BnFire(512, dim_bn=(0, 1))
        self.fc3 = nn.Linear(512, 10)

    def forward(self, images):
        x = self._encode(images)
        for name in self._conv_order:
            x = getattr(self, name)(x)
        x = self.bn(self.fc2(self.fc1(x)))
        return self.fc3(x.mean(dim=0))


class Alexnet_BN_DIST(_BnNet):
    """AlexNet-style, sync-BN layers, 224x224 inputs, 1000 classes. Reference: models.py:62-103."""

    def __init__(self):
        super().__init__()
        self.conv1 = sop.Conv(3, 64, stride=(2, 2))
        plan = [(64, 128, 2), (128, 256, 2), (256, 256, 2), (256, 384, 1), (384, 256, 1), (256, 256, 2)]
        for k, (cin, cout, stride) in enumerate(plan, start=2):
            setattr(self, f"conv{k}", sop.BnFireConvDist(cin, cout, stride=(stride, stride)))
        self.fc1 = sop.BnFireFcDist(7 * 7 * 256, 4096, dim_bn=(0, 1, 3, 4), cin_bn=256)
        self.fc2 = sop.BnFireFcDist(4096, 4096, dim_bn=(0, 1))
        self.fire = sop.Fire()
        self.fc3 = nn.Linear(4096, 1000)

    def forward(self, images):
        x = self._encode(images)
        for k in range(1, 8):
            x = getattr(self, f"conv{k}")(x)
        x = self.fire(self.fc2(self.fc1(x)))
        return self.fc3(x.mean(dim=0))


class ResidualDist(nn.Module):
    """LIF-conv, BN-LIF-conv, BN, plus the (optionally projected) input. Reference: models.py:107-128."""

    def __init__(self, cin, cout, stride=(1, 1), downsample=None):
        super().__init__()
        self.conv1 = sop.FireConv(cin, cout, stride=stride)
        self.conv2 = sop.BnFireConvDist(cout, cout)
        self.bn2 = sop.BnDist(cout, dim_bn=(0, 1, 3, 4))
        self.downsample = downsample

    def forward(self, current):
        out = self.bn2(self.conv2(self.conv1(current)))
        return out + (self.downsample(current) if self.downsample is not None else current)


class Resnet_DIST(_BnNet):
    """ResNet-34 layout (3-4-6-3 blocks), sync-BN, 224x224 inputs. Reference: models.py:132-191."""

    def __init__(self):
        super().__init__()
        self.pre_conv = sop.Conv(3, 64, kernel_size=(7, 7), stride=(2, 2), padding=(3, 3))
        self.pre_bn = sop.BnDist(64, dim_bn=(0, 1, 3, 4))
        cin = 64
        for k, (cout, blocks) in enumerate(((64, 3), (128, 4), (256, 6), (512, 3)), start=1):
            setattr(self, f"layer{k}", self._stage(cin, cout, blocks))
            cin = cout
        self.fire = sop.Fire()
        self.fc = nn.Linear(512, 1000)

    @staticmethod
    def _stage(cin, cout, blocks, stride=(2, 2)):
        project = nn.Sequential(sop.FireConv(cin, cout, kernel_size=(1, 1), stride=stride, padding=(0, 0)),
                                sop.BnDist(cout, (0, 1, 3, 4)))
        return nn.Sequential(ResidualDist(cin, cout, stride, project),
                             *[ResidualDist(cout, cout) for _ in range(1, blocks)])

    def forward(self, images):
        x = self.pre_bn(self.pre_conv(self._encode(images)))
        for k in range(1, 5):
            x = getattr(self, f"layer{k}")(x)
        x = self.fire(x).mean(dim=0)
        return self.fc(F.avg_pool2d(x, 7).flatten(1))


def build(name, **kw):
    if name == "vgg":
        return SpikingVGG(**kw)
    if name == "resnet19":
        return SpikingResNet19(**kw)
    if name in ("cifar_bn", "alexnet_bn_dist", "resnet_dist"):
        return {"cifar_bn": CIFAR_BN, "alexnet_bn_dist": Alexnet_BN_DIST, "resnet_dist": Resnet_DIST}[name]()
    raise ValueError(f"unknown model {name!r}")
