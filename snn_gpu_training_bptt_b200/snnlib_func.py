"""Autograd Functions over the ``snnlib`` op table, plus the hyper-parameter globals.

Host-side mirror of the reference's snnlib/example/snnlib_func.py: same module-level names
(``alpha, beta, interval, thresh, time_step, conv_benchmark``, reference lines 11-17), same
``XFunc`` classes and ``x_func = XFunc.apply`` callables with the same positional arguments
and the same tuple of returned gradients, so snnlib_op-style modules and models written
against the reference work unchanged. The globals are read at call time, as in the
reference, so ``snnlib_func.thresh = 0.5`` takes effect on the next forward.

Each forward saves only its inputs (the reference's choice, e.g. FireFunc at reference
lines 25-28): membrane potentials are never stored, the backward kernel rebuilds them.
"""
import torch

from . import _capi, snnlib
from ._capi import as_time_major_dense

# hyper-parameters (reference snnlib_func.py:11-17)
alpha = 0.25
beta = 1.0
interval = 0.5
thresh = 0.25
time_step = 6

conv_benchmark = False  # accepted for compatibility; cuDNN autotuning is torch's global switch

_DILATION, _GROUPS = (1, 1), 1
_DIM_FC = (0, 1)
_DIM_CONV = (0, 1, 3, 4)


def _nones(n):
    return (None,) * n


class FireFunc(torch.autograd.Function):
    """spike = LIF(spatial). Reference: snnlib_func.py:22-36."""

    @staticmethod
    def forward(ctx, spatial):
        spatial = as_time_major_dense(spatial)   # no copy for contiguous or channels-last inputs
        ctx.save_for_backward(spatial)
        return snnlib.fire_s_fp(spatial, alpha, thresh)

    @staticmethod
    def backward(ctx, grad_spike):
        (spatial,) = ctx.saved_tensors
        return snnlib.fire_bp(spatial, grad_spike, alpha, thresh, beta, interval)


fire_func = FireFunc.apply


class FireAddFunc(torch.autograd.Function):
    """spike = LIF(current + shortcut) without the sum in memory (an addition to the reference's set
    of Functions; equals ``fire_func(current + shortcut)`` bit for bit, spikes and gradients)."""

    @staticmethod
    def forward(ctx, current, shortcut):
        current, shortcut = _capi.lif_add_operands(current, shortcut)
        ctx.save_for_backward(current, shortcut)
        return _capi.lif_add_fwd(current, shortcut, alpha, thresh)

    @staticmethod
    def backward(ctx, grad_spike):
        current, shortcut = ctx.saved_tensors
        grad = _capi.lif_add_bwd(current, shortcut, grad_spike, alpha, thresh, beta, interval)
        return (grad if ctx.needs_input_grad[0] else None, grad if ctx.needs_input_grad[1] else None)


def fire_add_func(current, shortcut):
    """LIF of the sum of two currents; falls back to add -> ``fire_func`` where the fused backward
    does not apply (more than 16 time steps, float64)."""
    if current.shape[0] > _capi.LIF_ADD_MAX_T or current.dtype == torch.float64:
        return fire_func(current + shortcut)
    return FireAddFunc.apply(current, shortcut)


class FirePoolFunc(torch.autograd.Function):
    """LIF followed by AvgPool2d(2) on every time step, as one kernel each way (an addition to the
    reference's set of Functions; equals ``avg_pool2d(fire_func(x))`` applied per time step)."""

    @staticmethod
    def forward(ctx, spatial):
        dense, pooled = _capi.lif_pool_fwd(spatial, alpha, thresh)
        ctx.save_for_backward(dense)
        return pooled

    @staticmethod
    def backward(ctx, grad_pooled):
        (dense,) = ctx.saved_tensors
        return _capi.lif_pool_bwd(dense, grad_pooled, alpha, thresh, beta, interval)


fire_pool_func = FirePoolFunc.apply


class BnFunc(torch.autograd.Function):
    """Time-major batch-norm with externally supplied statistics. Reference: snnlib_func.py:42-60."""

    @staticmethod
    def forward(ctx, x_bn, weight_bn, bias_bn, var, mean, dim_bn, eps_bn):
        ivar, y_bn = snnlib.bn_fp(x_bn, weight_bn, bias_bn, var, mean, eps_bn)
        ctx.save_for_backward(x_bn, weight_bn, bias_bn, ivar, mean)
        ctx.dim_bn = dim_bn
        return y_bn

    @staticmethod
    def backward(ctx, grad_y_bn):
        x_bn, weight_bn, bias_bn, ivar, mean = ctx.saved_tensors
        gx, gw, gb = snnlib.bn_bp(x_bn, weight_bn, bias_bn, ivar, mean, ctx.dim_bn, grad_y_bn)
        return (gx, gw, gb) + _nones(4)


bn_func = BnFunc.apply


class BnFireFunc(torch.autograd.Function):
    """Batch-norm folded into the LIF input. Reference: snnlib_func.py:67-85."""

    @staticmethod
    def forward(ctx, spatial, weight_bn, bias_bn, var, mean, dim_bn, eps_bn):
        ivar, spike = snnlib.bn_fire_s_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, alpha, thresh)
        ctx.save_for_backward(spatial, weight_bn, bias_bn, ivar, mean)
        ctx.dim_bn = dim_bn
        return spike

    @staticmethod
    def backward(ctx, grad_spike):
        spatial, weight_bn, bias_bn, ivar, mean = ctx.saved_tensors
        gx, gw, gb = snnlib.bn_fire_bp(spatial, weight_bn, bias_bn, ivar, mean, ctx.dim_bn,
                                       grad_spike, alpha, thresh, beta, interval)
        return (gx, gw, gb) + _nones(4)


bn_fire_func = BnFireFunc.apply


class BnFireFcFunc(torch.autograd.Function):
    """BN + LIF + synaptic linear. Reference: snnlib_func.py:91-110."""

    @staticmethod
    def forward(ctx, spatial, weight_bn, bias_bn, var, mean, dim_bn, eps_bn, weight_fc, bias_fc):
        ivar, fc = snnlib.bn_fire_fc_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn,
                                        weight_fc, bias_fc, alpha, thresh)
        ctx.save_for_backward(spatial, weight_bn, bias_bn, ivar, mean, weight_fc, bias_fc)
        ctx.dim_bn = dim_bn
        return fc

    @staticmethod
    def backward(ctx, grad_fc):
        spatial, weight_bn, bias_bn, ivar, mean, weight_fc, bias_fc = ctx.saved_tensors
        gx, gwb, gbb, gwf, gbf = snnlib.bn_fire_fc_bp(
            spatial, weight_bn, bias_bn, ivar, mean, ctx.dim_bn, grad_fc, weight_fc, bias_fc,
            _DIM_FC, alpha, thresh, beta, interval)
        return (gx, gwb, gbb) + _nones(4) + (gwf, gbf)


bn_fire_fc_func = BnFireFcFunc.apply


class FireFcFunc(torch.autograd.Function):
    """LIF + synaptic linear. Reference: snnlib_func.py:116-132."""

    @staticmethod
    def forward(ctx, spatial, weight_fc, bias_fc):
        ctx.save_for_backward(spatial, weight_fc, bias_fc)
        return snnlib.fire_fc_fp(spatial, weight_fc, bias_fc, alpha, thresh)

    @staticmethod
    def backward(ctx, grad_fc):
        spatial, weight_fc, bias_fc = ctx.saved_tensors
        return tuple(snnlib.fire_fc_bp(spatial, grad_fc, weight_fc, bias_fc, _DIM_FC,
                                       alpha, thresh, beta, interval))


fire_fc_func = FireFcFunc.apply


class FcFunc(torch.autograd.Function):
    """Synaptic linear applied at every time step. Reference: snnlib_func.py:138-155."""

    @staticmethod
    def forward(ctx, spatial, weight_fc, bias_fc):
        ctx.save_for_backward(spatial, weight_fc, bias_fc)
        return snnlib.fc_fp(spatial, weight_fc, bias_fc)

    @staticmethod
    def backward(ctx, grad_fc):
        spatial, weight_fc, bias_fc = ctx.saved_tensors
        return tuple(snnlib.fc_bp(spatial, grad_fc, weight_fc, bias_fc, _DIM_FC))


fc_func = FcFunc.apply


class FcFireFunc(torch.autograd.Function):
    """Synaptic linear followed by LIF: ``fire_func(fc_func(x, W, b))`` as one op (an addition to
    the reference's set of Functions). For bf16 problems the tcgen05 kernels cover, forward is a
    single fused GEMM + LIF-epilogue launch and backward is the library's own pair of launches
    (LIF reverse pass, then both gradient GEMMs in one persistent tcgen05 kernel); otherwise one
    library GEMM and the LIF kernels each way. The LIF input current is saved (bf16 / input dtype)
    for the backward pass, and so is the bf16 copy of an fp32 master weight, so the weight is cast
    once per step."""

    @staticmethod
    def forward(ctx, spatial, weight_fc, bias_fc):
        fused = spatial.dim() == 3 and _capi.linear_lif_supported(spatial, weight_fc)
        if fused:
            weight_op = weight_fc if weight_fc.dtype == torch.bfloat16 else weight_fc.to(torch.bfloat16)
            current, spike = _capi.linear_lif_fwd(spatial, weight_op, bias_fc, alpha, thresh)
        else:
            weight_op = weight_fc
            current = snnlib.fc_fp(spatial, weight_fc, bias_fc)
            spike = snnlib.fire_s_fp(current, alpha, thresh)
        ctx.save_for_backward(spatial, weight_op, bias_fc, current)
        ctx.fused = fused and _capi.linear_lif_bwd_supported(spatial, weight_op)
        ctx.weight_dtype = weight_fc.dtype
        return spike

    @staticmethod
    def backward(ctx, grad_spike):
        spatial, weight_op, bias_fc, current = ctx.saved_tensors
        if ctx.fused:
            need_x, need_w, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1], \
                bias_fc is not None and ctx.needs_input_grad[2]
            out_dtype = ctx.weight_dtype if ctx.weight_dtype in (torch.float32, torch.bfloat16) else torch.float32
            gx, gw, gb = _capi.linear_lif_bwd(spatial, weight_op, current, grad_spike, alpha, thresh, beta,
                                              interval, need_x, need_w, need_b, out_dtype)
            if gw is not None and gw.dtype != ctx.weight_dtype:
                gw = gw.to(ctx.weight_dtype)
            if gb is not None and gb.dtype != bias_fc.dtype:
                gb = gb.to(bias_fc.dtype)
            return gx, (gw if need_w else None), gb
        grad_current = snnlib.fire_bp(current, grad_spike, alpha, thresh, beta, interval)
        gx, gw, gb = snnlib.fc_bp(spatial, grad_current, weight_op, bias_fc, _DIM_FC)
        return gx, gw.to(ctx.weight_dtype), (gb if bias_fc is not None else None)


fc_fire_func = FcFireFunc.apply


def _conv_grad_tuple(grads, head, if_bias_conv, tail):
    """(input/bn grads..., Nones, grad_w, grad_b or None, Nones): layout of reference lines 183-191."""
    gw, gb = grads[-2], grads[-1]
    return tuple(grads[:-2]) + _nones(head) + (gw, gb if if_bias_conv else None) + _nones(tail)


class BnFireConvFunc(torch.autograd.Function):
    """BN + LIF + convolution. Reference: snnlib_func.py:161-191."""

    @staticmethod
    def forward(ctx, spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_conv, bias_conv,
                stride, padding, if_bias_conv):
        ivar, conv = snnlib.bn_fire_conv_fp(
            spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_conv, bias_conv, stride,
            padding, _DILATION, _GROUPS, conv_benchmark, False, alpha, thresh)
        ctx.save_for_backward(spatial, weight_bn, bias_bn, ivar, mean, weight_conv, bias_conv)
        ctx.cfg = (stride, padding, if_bias_conv)
        return conv

    @staticmethod
    def backward(ctx, grad_conv):
        spatial, weight_bn, bias_bn, ivar, mean, weight_conv, _ = ctx.saved_tensors
        stride, padding, if_bias_conv = ctx.cfg
        grads = snnlib.bn_fire_conv_bp(
            spatial.contiguous(), weight_bn, bias_bn, ivar, mean, _DIM_CONV, grad_conv.contiguous(),
            weight_conv, stride, padding, _DILATION, _GROUPS, conv_benchmark, False, True,
            _DIM_CONV, alpha, thresh, beta, interval)
        return _conv_grad_tuple(grads, 3, if_bias_conv, 3)


bn_fire_conv_func = BnFireConvFunc.apply


class FireConvFunc(torch.autograd.Function):
    """LIF + convolution. Reference: snnlib_func.py:197-223."""

    @staticmethod
    def forward(ctx, spatial, weight_conv, bias_conv, stride, padding, if_bias_conv):
        ctx.save_for_backward(spatial, weight_conv, bias_conv)
        ctx.cfg = (stride, padding, if_bias_conv)
        return snnlib.fire_conv_fp(spatial, weight_conv, bias_conv, stride, padding, _DILATION,
                                   _GROUPS, conv_benchmark, False, alpha, thresh)

    @staticmethod
    def backward(ctx, grad_conv):
        spatial, weight_conv, _ = ctx.saved_tensors
        stride, padding, if_bias_conv = ctx.cfg
        grads = snnlib.fire_conv_bp(
            spatial, grad_conv, weight_conv, stride, padding, _DILATION,
            _GROUPS, conv_benchmark, False, True, _DIM_CONV, alpha, thresh, beta, interval)
        return _conv_grad_tuple(grads, 0, if_bias_conv, 3)


fire_conv_func = FireConvFunc.apply


class ConvFunc(torch.autograd.Function):
    """Convolution applied at every time step. Reference: snnlib_func.py:229-255."""

    @staticmethod
    def forward(ctx, spatial, weight_conv, bias_conv, stride, padding, if_bias_conv):
        ctx.save_for_backward(spatial, weight_conv, bias_conv)
        ctx.cfg = (stride, padding, if_bias_conv)
        return snnlib.conv_fp(spatial, weight_conv, bias_conv, stride, padding, _DILATION,
                              _GROUPS, conv_benchmark, False)

    @staticmethod
    def backward(ctx, grad_conv):
        spatial, weight_conv, _ = ctx.saved_tensors
        stride, padding, if_bias_conv = ctx.cfg
        grads = snnlib.conv_bp(spatial, grad_conv, weight_conv, stride,
                               padding, _DILATION, _GROUPS, conv_benchmark, False, True, _DIM_CONV)
        return _conv_grad_tuple(grads, 0, if_bias_conv, 3)


conv_func = ConvFunc.apply


# ------------------------------------------------------------------------------------------
# sync-BN variants: backward is split around two all-reduces of per-channel sums
# (reference snnlib_func.py:261-379). reduce_op = [ReduceOp enum, process group, world size].
# ------------------------------------------------------------------------------------------
def _allreduce_channel_sums(local_xhat, local_xhatx, reduce_op):
    """Mean over ranks of the two per-channel vectors, as one [2, C] all-reduce (the reference
    sends them as two messages, snnlib_func.py:278-279; the arithmetic is the same)."""
    op, group, world = reduce_op
    base = local_xhat._base
    if (base is not None and base is local_xhatx._base and base.dim() == 2 and base.shape[0] == 2
            and base.is_contiguous() and local_xhat.data_ptr() == base.data_ptr()
            and local_xhatx.data_ptr() == base[1].data_ptr()):
        both = base                      # the two rows of the buffer the means kernel wrote: no copy
    else:
        both = torch.stack((local_xhat, local_xhatx))
    torch.distributed.all_reduce(both, op.SUM, group)
    both /= world
    return both[0], both[1]


class BnDistFunc(torch.autograd.Function):
    """Reference: snnlib_func.py:261-290."""

    @staticmethod
    def forward(ctx, x_bn, weight_bn, bias_bn, var, mean, dim_bn, eps_bn, reduce_op):
        ivar, y_bn = snnlib.bn_fp(x_bn, weight_bn, bias_bn, var, mean, eps_bn)
        ctx.save_for_backward(x_bn, weight_bn, bias_bn, ivar, mean)
        ctx.dim_bn, ctx.reduce_op = dim_bn, reduce_op
        return y_bn

    @staticmethod
    def backward(ctx, grad_y_bn):
        x_bn, weight_bn, bias_bn, ivar, mean = ctx.saved_tensors
        x_bn, grad_y_bn = x_bn.contiguous(), grad_y_bn.contiguous()
        lx, lxx, gw, gb = snnlib.bn_bp_dist1(x_bn, weight_bn, bias_bn, ivar, mean, ctx.dim_bn, grad_y_bn)
        gxhat, gxhatx = _allreduce_channel_sums(lx, lxx, ctx.reduce_op)
        gx = snnlib.bn_bp_dist2(x_bn, weight_bn, bias_bn, ivar, mean, ctx.dim_bn, grad_y_bn, gxhat, gxhatx)
        return (gx, gw, gb) + _nones(5)


bn_dist_func = BnDistFunc.apply


class BnFireFcDistFunc(torch.autograd.Function):
    """Reference: snnlib_func.py:297-332."""

    @staticmethod
    def forward(ctx, spatial, weight_bn, bias_bn, var, mean, dim_bn, eps_bn, weight_fc, bias_fc,
                reduce_op):
        ivar, fc = snnlib.bn_fire_fc_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn,
                                        weight_fc, bias_fc, alpha, thresh)
        ctx.save_for_backward(spatial, weight_bn, bias_bn, ivar, mean, weight_fc, bias_fc)
        ctx.dim_bn, ctx.reduce_op = dim_bn, reduce_op
        return fc

    @staticmethod
    def backward(ctx, grad_fc):
        spatial, weight_bn, bias_bn, ivar, mean, weight_fc, bias_fc = ctx.saved_tensors
        spatial = spatial.contiguous()
        gspike, lx, lxx, gwb, gbb, gwf, gbf = snnlib.bn_fire_fc_bp_dist1(
            spatial, weight_bn, bias_bn, ivar, mean, ctx.dim_bn, grad_fc.contiguous(), weight_fc,
            bias_fc, _DIM_FC, alpha, thresh, beta, interval)
        gxhat, gxhatx = _allreduce_channel_sums(lx, lxx, ctx.reduce_op)
        gx = snnlib.bn_fire_bp_dist2(spatial, weight_bn, bias_bn, ivar, mean, gspike.contiguous(),
                                     gxhat, gxhatx, alpha, thresh, beta, interval)
        return (gx, gwb, gbb) + _nones(4) + (gwf, gbf, None)


bn_fire_fc_dist_func = BnFireFcDistFunc.apply


class BnFireConvDistFunc(torch.autograd.Function):
    """Reference: snnlib_func.py:339-379."""

    @staticmethod
    def forward(ctx, spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_conv, bias_conv,
                stride, padding, if_bias_conv, reduce_op):
        ivar, conv = snnlib.bn_fire_conv_fp(
            spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_conv, bias_conv, stride,
            padding, _DILATION, _GROUPS, conv_benchmark, False, alpha, thresh)
        ctx.save_for_backward(spatial, weight_bn, bias_bn, ivar, mean, weight_conv, bias_conv)
        ctx.cfg = (stride, padding, if_bias_conv, reduce_op)
        return conv

    @staticmethod
    def backward(ctx, grad_conv):
        spatial, weight_bn, bias_bn, ivar, mean, weight_conv, _ = ctx.saved_tensors
        stride, padding, if_bias_conv, reduce_op = ctx.cfg
        spatial = spatial.contiguous()
        gspike, lx, lxx, gwb, gbb, gwc, gbc = snnlib.bn_fire_conv_bp_dist1(
            spatial, weight_bn, bias_bn, ivar, mean, _DIM_CONV, grad_conv.contiguous(), weight_conv,
            stride, padding, _DILATION, _GROUPS, conv_benchmark, False, True, _DIM_CONV,
            alpha, thresh, beta, interval)
        gxhat, gxhatx = _allreduce_channel_sums(lx, lxx, reduce_op)
        gx = snnlib.bn_fire_bp_dist2(spatial, weight_bn, bias_bn, ivar, mean, gspike.contiguous(),
                                     gxhat, gxhatx, alpha, thresh, beta, interval)
        return _conv_grad_tuple((gx, gwb, gbb, gwc, gbc), 3, if_bias_conv, 4)


bn_fire_conv_dist_func = BnFireConvDistFunc.apply
