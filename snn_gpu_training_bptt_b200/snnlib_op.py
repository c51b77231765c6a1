"""Layer modules of a spiking network on time-major tensors [T, B, C] / [T, B, C, H, W].

Host-side mirror of the reference's snnlib/example/snnlib_op.py: the same twelve classes
(Fire, Bn, BnFire, BnFireFc, FireFc, Fc, BnFireConv, FireConv, Conv, BnDist, BnFireFcDist,
BnFireConvDist) with the same constructor arguments, parameter names (``weight_bn``,
``bias_bn``, ``running_var``, ``running_mean``, ``weight_fc``, ``bias_fc``, ``weight_conv``,
``bias_conv`` - so reference state dicts load), initialisations and ``train_bn`` switch.

One deliberate difference: the reference re-wraps ``running_var`` / ``running_mean`` in a
brand-new ``nn.Parameter`` on every training forward (reference lines 45-46, 79-80, ...),
which changes the module's parameter identities each step and forces data-parallel wrappers
to rebuild their buckets. Here the running statistics keep their identity and are updated
in place (same values, same state-dict keys, ``requires_grad=False``).
"""
import math

import torch
import torch.nn as nn

from . import snnlib_func as sf


class Fire(nn.Module):
    """LIF layer. Reference: snnlib_op.py:11-16."""

    def forward(self, x):
        return sf.fire_func(x)


class FireAdd(nn.Module):
    """LIF layer on the sum of two currents, fused (not in the reference's layer set; identical to
    ``Fire()(current + shortcut)``)."""

    def forward(self, current, shortcut):
        return sf.fire_add_func(current, shortcut)


class FirePool(nn.Module):
    """LIF layer followed by AvgPool2d(2) per time step, fused (not in the reference's layer set;
    numerically identical to ``Fire`` then pooling each x[t])."""

    def forward(self, x):
        return sf.fire_pool_func(x)


class FcFire(nn.Module):
    """Synaptic linear followed by LIF as one op (``Fc`` then ``Fire`` of the reference; fused on
    the tensor cores for bf16 inputs with tile-aligned sizes). Parameters as ``Fc``."""

    def __init__(self, cin, cout):
        super().__init__()
        self.weight_fc = nn.Parameter(torch.zeros(cout, cin).normal_(0, 0.75 / math.sqrt(cin)))
        self.bias_fc = nn.Parameter(torch.zeros(cout))

    def forward(self, x):
        return sf.fc_fire_func(x, self.weight_fc, self.bias_fc)


# ------------------------------------------------------------------------------------------
# shared batch-norm bookkeeping
# ------------------------------------------------------------------------------------------
class _BnStats(nn.Module):
    """Affine BN parameters + running statistics over a time-major tensor.

    ``momentum`` is the weight of the new batch statistic: 0.1 for the single-GPU layers
    (reference lines 45-46), 0.05 for the sync-BN layers (reference lines 274-275). The
    running variance gets the unbiased correction n/(n-1) (reference lines 37-38).
    """

    def _init_bn(self, channels, dim_bn, eps_bn, momentum, distributed):
        self.dim_bn = dim_bn
        self.eps_bn = eps_bn
        self.weight_bn = nn.Parameter(torch.ones(channels))
        self.bias_bn = nn.Parameter(torch.zeros(channels))
        self.running_var = nn.Parameter(torch.ones(channels), requires_grad=False)
        self.running_mean = nn.Parameter(torch.zeros(channels), requires_grad=False)
        self.factor = None
        self.train_bn = True
        self._bn_channels = channels
        self._momentum = momentum
        self._distributed = distributed
        if distributed:
            self.ReduceOp = torch.distributed.ReduceOp
            self.process_group = None
            self.world_size = None

    def _reduce_arg(self):
        return [self.ReduceOp, self.process_group, self.world_size]

    def _statistics(self, x):
        """Returns (var, mean) to normalise with and updates the running statistics."""
        if self.factor is None:
            count = x.numel() / self._bn_channels
            self.factor = count / (count - 1)
            if self._distributed:
                self.process_group = torch.distributed.group.WORLD
                self.world_size = torch.distributed.get_world_size(self.process_group)
        if not self.train_bn:
            return self.running_var, self.running_mean
        # Statistics are always fp32, whatever the activation dtype (the kernels take fp32
        # var / mean beside bf16 / fp16 tensors; E[x^2] - E[x]^2 in 16 bits would be unusable).
        low = x.dtype in (torch.bfloat16, torch.float16)
        if self._distributed:
            # one [2, C] message carries both moments (the reference sends two [C] messages,
            # snnlib_op.py:268-269); same arithmetic: mean of the ranks' means and mean squares
            moments = torch.stack((self._mean32(x), self._mean_sq32(x)))
            torch.distributed.all_reduce(moments, self.ReduceOp.SUM, self.process_group)
            mean = moments[0] / self.world_size
            var = moments[1] / self.world_size - mean ** 2
        elif low:
            mean = self._mean32(x)
            var = (self._mean_sq32(x) - mean ** 2).clamp(min=0.0)
        else:
            var, mean = torch.var_mean(x, dim=self.dim_bn, unbiased=False)
        m = self._momentum
        with torch.no_grad():
            self.running_var.mul_(1 - m).add_(var.detach() * (m * self.factor))
            self.running_mean.mul_(1 - m).add_(mean.detach() * m)
        return var, mean


    def _mean32(self, x):
        return torch.mean(x, dim=self.dim_bn, dtype=torch.float32)

    def _mean_sq32(self, x):
        """E[x^2] per channel, accumulated in fp32 without an fp32 copy of a 16-bit activation."""
        if x.dtype == torch.float32:
            return torch.mean(x * x, dim=self.dim_bn)
        count = x.numel() / self._bn_channels
        return torch.linalg.vector_norm(x, 2, dim=self.dim_bn, dtype=torch.float32).square() / count


class Bn(_BnStats):
    """Reference: snnlib_op.py:19-50."""

    def __init__(self, cin, dim_bn, eps_bn=1e-5):
        super().__init__()
        self.cin = cin
        self._init_bn(cin, dim_bn, eps_bn, 0.1, False)

    def forward(self, x):
        var, mean = self._statistics(x)
        return sf.bn_func(x, self.weight_bn, self.bias_bn, var, mean, self.dim_bn, self.eps_bn)


class BnFire(_BnStats):
    """Reference: snnlib_op.py:53-84."""

    def __init__(self, cin, dim_bn, eps_bn=1e-5):
        super().__init__()
        self.cin = cin
        self._init_bn(cin, dim_bn, eps_bn, 0.1, False)

    def forward(self, x):
        var, mean = self._statistics(x)
        return sf.bn_fire_func(x, self.weight_bn, self.bias_bn, var, mean, self.dim_bn, self.eps_bn)


def _linear_params(cin, cout):
    """nn.Linear's default initialisation, as the BN-bearing FC layers use (reference lines 107-109)."""
    fc = nn.Linear(cin, cout, bias=True)
    return nn.Parameter(fc.weight.detach().clone()), nn.Parameter(fc.bias.detach().clone())


def _conv_params(cin, cout, kernel_size, stride, padding):
    """nn.Conv2d's default initialisation (reference lines 168-170)."""
    conv = nn.Conv2d(cin, cout, kernel_size, stride, padding)
    return nn.Parameter(conv.weight.detach().clone()), nn.Parameter(conv.bias.detach().clone())


class BnFireFc(_BnStats):
    """Reference: snnlib_op.py:87-128. ``cin_bn`` = BN channel count when the input is 5-D."""

    _DIST = False

    def __init__(self, cin, cout, dim_bn, eps_bn=1e-5, cin_bn=None):
        super().__init__()
        self.cin = cin
        self.cin_bn = cin if cin_bn is None else cin_bn
        self._init_bn(self.cin_bn, dim_bn, eps_bn, 0.05 if self._DIST else 0.1, self._DIST)
        self.weight_fc, self.bias_fc = _linear_params(cin, cout)

    def forward(self, x):
        var, mean = self._statistics(x)
        if self._DIST:
            return sf.bn_fire_fc_dist_func(x, self.weight_bn, self.bias_bn, var, mean, self.dim_bn,
                                           self.eps_bn, self.weight_fc, self.bias_fc, self._reduce_arg())
        return sf.bn_fire_fc_func(x, self.weight_bn, self.bias_bn, var, mean, self.dim_bn,
                                  self.eps_bn, self.weight_fc, self.bias_fc)


class FireFc(nn.Module):
    """Reference: snnlib_op.py:131-139 (normal init, std 0.75/sqrt(cin); zero bias)."""

    def __init__(self, cin, cout):
        super().__init__()
        self.weight_fc = nn.Parameter(torch.zeros(cout, cin).normal_(0, 0.75 / math.sqrt(cin)))
        self.bias_fc = nn.Parameter(torch.zeros(cout))

    def forward(self, x):
        return sf.fire_fc_func(x, self.weight_fc, self.bias_fc)


class Fc(nn.Module):
    """Reference: snnlib_op.py:142-150."""

    def __init__(self, cin, cout):
        super().__init__()
        self.weight_fc = nn.Parameter(torch.zeros(cout, cin).normal_(0, 0.75 / math.sqrt(cin)))
        self.bias_fc = nn.Parameter(torch.zeros(cout))

    def forward(self, x):
        return sf.fc_func(x, self.weight_fc, self.bias_fc)


class BnFireConv(_BnStats):
    """Reference: snnlib_op.py:153-192."""

    _DIST = False

    def __init__(self, cin, cout, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), eps_bn=1e-5,
                 if_bias_conv=True):
        super().__init__()
        self.cin = cin
        self.stride = stride
        self.padding = padding
        self.if_bias_conv = if_bias_conv
        self._init_bn(cin, (0, 1, 3, 4), eps_bn, 0.05 if self._DIST else 0.1, self._DIST)
        self.weight_conv, self.bias_conv = _conv_params(cin, cout, kernel_size, stride, padding)

    def forward(self, x):
        var, mean = self._statistics(x)
        if self._DIST:
            return sf.bn_fire_conv_dist_func(
                x, self.weight_bn, self.bias_bn, var, mean, self.eps_bn, self.weight_conv,
                self.bias_conv, self.stride, self.padding, self.if_bias_conv, self._reduce_arg())
        return sf.bn_fire_conv_func(x, self.weight_bn, self.bias_bn, var, mean, self.eps_bn,
                                    self.weight_conv, self.bias_conv, self.stride, self.padding,
                                    self.if_bias_conv)


class FireConv(nn.Module):
    """Reference: snnlib_op.py:195-210."""

    def __init__(self, cin, cout, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), if_bias_conv=True):
        super().__init__()
        self.cin = cin
        self.stride = stride
        self.padding = padding
        self.if_bias_conv = if_bias_conv
        self.weight_conv, self.bias_conv = _conv_params(cin, cout, kernel_size, stride, padding)

    def forward(self, x):
        return sf.fire_conv_func(x, self.weight_conv, self.bias_conv, self.stride, self.padding,
                                 self.if_bias_conv)


class Conv(nn.Module):
    """Reference: snnlib_op.py:213-228 (normal init, std 0.75/sqrt(cin); zero bias)."""

    def __init__(self, cin, cout, kernel_size=(3, 3), stride=(1, 1), padding=(1, 1), if_bias_conv=True):
        super().__init__()
        self.cin = cin
        self.stride = stride
        self.padding = padding
        self.if_bias_conv = if_bias_conv
        shape = (cout, cin, kernel_size[0], kernel_size[1])
        self.weight_conv = nn.Parameter(torch.zeros(shape).normal_(0, 0.75 / math.sqrt(cin)))
        self.bias_conv = nn.Parameter(torch.zeros(cout))

    def forward(self, x):
        return sf.conv_func(x, self.weight_conv, self.bias_conv, self.stride, self.padding,
                            self.if_bias_conv)


class BnDist(_BnStats):
    """Sync-BN over the process group. Reference: snnlib_op.py:231-282."""

    def __init__(self, cin, dim_bn, eps_bn=1e-5):
        super().__init__()
        self.cin = cin
        self._init_bn(cin, dim_bn, eps_bn, 0.05, True)

    def forward(self, x):
        var, mean = self._statistics(x)
        return sf.bn_dist_func(x, self.weight_bn, self.bias_bn, var, mean, self.dim_bn, self.eps_bn,
                               self._reduce_arg())


class BnFireFcDist(BnFireFc):
    """Reference: snnlib_op.py:285-345."""

    _DIST = True


class BnFireConvDist(BnFireConv):
    """Reference: snnlib_op.py:348-406."""

    _DIST = True
