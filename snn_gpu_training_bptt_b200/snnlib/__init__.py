"""Drop-in for the reference's compiled extension module ``snnlib``.

The reference builds ``snnlib`` from snnlib/cuda/snn.cpp (pybind11 table at snn.cpp:798-830)
and its only caller is snnlib/example/snnlib_func.py. This package exposes the same function
names with the same positional arguments and return values, backed by libsnn_b200.so
(hand-written sm_100a kernels behind a C ABI, see include/snn_b200.h) for the LIF fire path and
the batch-norm family, and by one library GEMM / convolution over the merged [T*B, ...] batch
where the reference issues T separate cuBLAS / cuDNN calls.

Make it importable under the reference's name with either
``snn_gpu_training_bptt_b200.install_as_snnlib()`` or by putting this package's parent
directory on ``sys.path``; the reference's own snnlib_func.py / snnlib_op.py / models.py
then run unchanged.

Differences from the reference, all on the strict side: inputs are validated (CUDA, floating
dtype, shapes) and errors are raised instead of producing garbage; kernels launch on
torch's current stream instead of the legacy default stream; bf16 / fp16 tensors are
accepted (state is still carried in fp32); 64-bit indexing.
"""
import torch
import torch.nn.functional as F

from .. import _capi

__all__ = [
    "fire_s_fp", "bn_fire_s_fp", "bn_fp", "bn_bp", "bn_fire_fc_fp", "fire_fc_fp", "fc_fp",
    "bn_fire_conv_fp", "fire_conv_fp", "conv_fp", "fire_bp", "bn_fire_bp", "bn_fire_fc_bp",
    "fire_fc_bp", "fc_bp", "bn_fire_conv_bp", "fire_conv_bp", "conv_bp", "bn_bp_dist1",
    "bn_bp_dist2", "bn_fire_bp_dist1", "bn_fire_bp_dist2", "bn_fire_fc_bp_dist1",
    "bn_fire_conv_bp_dist1",
]


# ------------------------------------------------------------------------------------------
# LIF fire (the hot path)
# ------------------------------------------------------------------------------------------
def fire_s_fp(spatial, alpha, thresh):
    """LIF forward, returns the 0/1 spike tensor (same shape and dtype as ``spatial``).

    Reference: fire_s_fp, snnlib/cuda/snn.cpp:11-17 -> snn_kernel_fp.cu:55-73.
    """
    spike, _, _ = _capi.lif_fwd(spatial, alpha, thresh)
    return spike


def fire_bp(spatial, grad_spike, alpha, thresh, beta, interval):
    """LIF backward through time; returns grad w.r.t. ``spatial``.

    Reference: fire_bp, snnlib/cuda/snn.cpp:270-279 -> snn_kernel_bp.cu:141-168.
    """
    return _capi.lif_bwd(spatial, grad_spike, alpha, thresh, beta, interval)


# ------------------------------------------------------------------------------------------
# synaptic linear over time (one GEMM over the merged T*B rows)
# ------------------------------------------------------------------------------------------
def _cast(param, like):
    """Parameters may be kept in fp32 while activations run in bf16/fp16: the synaptic op then
    runs in the activation dtype (weights cast on the fly, gradients returned in the
    parameter's dtype). With matching dtypes this is the identity."""
    return param if param is None or param.dtype == like.dtype else param.to(like.dtype)


def _add_bias(y, bias):
    """y[:, c] += bias[c] in place with the library's channel kernel (fp32 bias, any activation
    dtype); torch's own add for the combinations that kernel does not cover."""
    if bias is None:
        return y
    if y.is_cuda and bias.dtype == torch.float32 and y.dtype in (torch.float32, torch.bfloat16, torch.float16) \
            and _capi._channel_geometry(y) is not None:
        return _capi.channel_bias_add_(y, bias)
    return y.add_(bias.to(y.dtype).view((1, -1) + (1,) * (y.dim() - 2)))


def _bias_grad(g, dtype):
    """Sum of g ([N, C, ...]) over everything but channels, in the bias's dtype."""
    if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16, torch.float16):
        return _capi.channel_sum(g).to(dtype)
    return torch.sum(g, dim=[d for d in range(g.dim()) if d != 1], dtype=dtype)


def _rows(t):
    """[T, B, ...] -> [T*B, features] view (reference flattens C,H,W: snn_kernel_fp.cu:349)."""
    return t.reshape(t.shape[0] * t.shape[1], -1)


def fc_fp(spatial, weight_fc, bias_fc):
    """fc[t] = spatial[t] @ W^T + b for every t. Reference: snn.cpp:130-136 -> snn_kernel_fp.cu:332-357."""
    T, B = spatial.shape[0], spatial.shape[1]
    y = F.linear(_rows(spatial), _cast(weight_fc, spatial))
    return _add_bias(y, bias_fc).view(T, B, weight_fc.shape[0])


def _fc_grads(inp_rows, grad_fc, weight_fc, dim_fc):
    g = _rows(grad_fc)
    grad_in = g @ _cast(weight_fc, g)            # [T*B, in]
    grad_w = (g.t() @ inp_rows).to(weight_fc.dtype)   # [out, in], summed over t and b
    return grad_in, grad_w, _bias_grad(g, weight_fc.dtype)


def fc_bp(spatial, grad_fc, weight_fc, bias_fc, dim_fc):
    """Returns [grad_spatial, grad_weight_fc, grad_bias_fc]. Reference: snn.cpp:594-602 -> snn_kernel_bp.cu:1131-1173."""
    grad_in, grad_w, grad_b = _fc_grads(_rows(spatial), grad_fc, weight_fc, dim_fc)
    return [grad_in.view(spatial.shape), grad_w, grad_b]


def fire_fc_fp(spatial, weight_fc, bias_fc, alpha, thresh):
    """LIF on the incoming current, then the synaptic linear. Reference: snn.cpp:112-120 -> snn_kernel_fp.cu:295-329."""
    spike = fire_s_fp(spatial, alpha, thresh)
    return fc_fp(spike, weight_fc, bias_fc)


def fire_fc_bp(spatial, grad_fc, weight_fc, bias_fc, dim_fc, alpha, thresh, beta, interval):
    """Returns [grad_spatial, grad_weight_fc, grad_bias_fc]. Reference: snn.cpp:569-582 -> snn_kernel_bp.cu:1065-1128.

    The reference re-materialises both u and s; here only the spikes are rebuilt (they are a
    GEMM operand) and u is recomputed inside the backward kernel's registers.
    """
    spike = fire_s_fp(spatial, alpha, thresh)
    grad_spike, grad_w, grad_b = _fc_grads(_rows(spike), grad_fc, weight_fc, dim_fc)
    grad_spatial = fire_bp(spatial, grad_spike.view(spatial.shape), alpha, thresh, beta, interval)
    return [grad_spatial, grad_w, grad_b]


# ------------------------------------------------------------------------------------------
# synaptic convolution over time (one cuDNN call over the merged T*B images)
# ------------------------------------------------------------------------------------------
def _images(t):
    return t.reshape((t.shape[0] * t.shape[1],) + tuple(t.shape[2:]))


def conv_fp(spatial, weight_conv, bias_conv, stride, padding, dilation, groups, benchmark,
            deterministic):
    """conv[t] = conv2d(spatial[t]). Reference: snn.cpp:239-253 -> snn_kernel_fp.cu:457-479."""
    T, B = spatial.shape[0], spatial.shape[1]
    y = F.conv2d(_images(spatial), _cast(weight_conv, spatial), None, tuple(stride), tuple(padding),
                 tuple(dilation), groups)
    return _add_bias(y, bias_conv).view((T, B) + tuple(y.shape[1:]))


def _conv_grads(inp, grad_conv, weight_conv, stride, padding, dilation, groups, dim_conv):
    g = _images(grad_conv)
    x = _images(inp)
    grad_in, grad_w = torch.ops.aten.convolution_backward(
        g, x, _cast(weight_conv, g), None, list(stride), list(padding), list(dilation), False,
        [0, 0], groups, [True, True, False])[:2]
    return grad_in, grad_w.to(weight_conv.dtype), _bias_grad(g, weight_conv.dtype)


def conv_bp(spatial, grad_conv, weight_conv, stride, padding, dilation, groups, benchmark,
            deterministic, allow_tf32, dim_conv):
    """Returns [grad_spatial, grad_weight_conv, grad_bias_conv]. Reference: snn.cpp:779-794 -> snn_kernel_bp.cu:1404-1436."""
    grad_in, grad_w, grad_b = _conv_grads(spatial, grad_conv, weight_conv, stride, padding,
                                          dilation, groups, dim_conv)
    return [grad_in.view(spatial.shape), grad_w, grad_b]


def fire_conv_fp(spatial, weight_conv, bias_conv, stride, padding, dilation, groups, benchmark,
                 deterministic, alpha, thresh):
    """LIF then convolution. Reference: snn.cpp:206-223 -> snn_kernel_fp.cu:413-454."""
    spike = fire_s_fp(spatial, alpha, thresh)
    return conv_fp(spike, weight_conv, bias_conv, stride, padding, dilation, groups, benchmark,
                   deterministic)


def fire_conv_bp(spatial, grad_conv, weight_conv, stride, padding, dilation, groups, benchmark,
                 deterministic, allow_tf32, dim_conv, alpha, thresh, beta, interval):
    """Returns [grad_spatial, grad_weight_conv, grad_bias_conv]. Reference: snn.cpp:740-762 -> snn_kernel_bp.cu:1344-1401."""
    spike = fire_s_fp(spatial, alpha, thresh)
    grad_spike, grad_w, grad_b = _conv_grads(spike, grad_conv, weight_conv, stride, padding,
                                             dilation, groups, dim_conv)
    grad_spatial = fire_bp(spatial, grad_spike.view(spatial.shape), alpha, thresh, beta, interval)
    return [grad_spatial, grad_w, grad_b]


# ------------------------------------------------------------------------------------------
# batch-norm family. Statistics (var, mean) come from the caller, as in the reference, where
# snnlib_op computes them with torch.var_mean / all-reduced means before calling in.
# ------------------------------------------------------------------------------------------
def bn_fp(x_bn, weight_bn, bias_bn, var, mean, eps_bn):
    """Returns [ivar, y_bn]. Reference: snn.cpp:30-39 -> snn_kernel_fp.cu:124-150."""
    ivar, y, _ = _capi.bn_lif_fwd(x_bn, weight_bn, bias_bn, var, mean, eps_bn, 0.0, 0.0, fire=False)
    return [ivar, y]


def bn_fire_s_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, alpha, thresh):
    """Returns [ivar, spike]. Reference: snn.cpp:55-66 -> snn_kernel_fp.cu:212-240."""
    ivar, spike, _ = _capi.bn_lif_fwd(spatial, weight_bn, bias_bn, var, mean, eps_bn, alpha, thresh)
    return [ivar, spike]


def _bn_backward(x, grad, weight_bn, bias_bn, ivar, mean, consts, fire):
    """Two-pass backward: per-channel sums, channel means, input gradient."""
    alpha, thresh, beta, interval = consts
    x, g, sum_g, sum_gx, count = _capi.bn_lif_bwd_sums(x, grad, weight_bn, bias_bn, ivar, mean, alpha,
                                                       thresh, beta, interval, fire=fire)
    gxhat, gxhatx = _capi.bn_channel_means(sum_g, sum_gx, weight_bn, count)
    gx = _capi.bn_lif_bwd_input(x, g, weight_bn, bias_bn, ivar, mean, gxhat, gxhatx, alpha, thresh,
                                beta, interval, fire=fire)
    return gx, sum_gx, sum_g          # grad_x, grad_weight_bn, grad_bias_bn


def _bn_backward_local(x, grad, weight_bn, bias_bn, ivar, mean, consts, fire):
    """First half for sync-BN: local channel means (to be all-reduced) and local parameter sums."""
    alpha, thresh, beta, interval = consts
    _, _, sum_g, sum_gx, count = _capi.bn_lif_bwd_sums(x, grad, weight_bn, bias_bn, ivar, mean, alpha,
                                                       thresh, beta, interval, fire=fire)
    gxhat, gxhatx = _capi.bn_channel_means(sum_g, sum_gx, weight_bn, count)
    return gxhat, gxhatx, sum_gx, sum_g


def bn_bp(x_bn, weight_bn, bias_bn, ivar, mean, dim_bn, grad_y_bn):
    """Returns [grad_x_bn, grad_weight_bn, grad_bias_bn]. Reference: snn.cpp:293-303 -> snn_kernel_bp.cu:288-345."""
    return list(_bn_backward(x_bn, grad_y_bn, weight_bn, bias_bn, ivar, mean, (0.0, 0.0, 0.0, 0.0), False))


def bn_fire_bp(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_spike, alpha, thresh, beta, interval):
    """Returns [grad_spatial, grad_weight_bn, grad_bias_bn]. Reference: snn.cpp:373-387 -> snn_kernel_bp.cu:679-750."""
    return list(_bn_backward(spatial, grad_spike, weight_bn, bias_bn, ivar, mean,
                             (alpha, thresh, beta, interval), True))


def bn_bp_dist1(x_bn, weight_bn, bias_bn, ivar, mean, dim_bn, grad_y_bn):
    """Returns [local_grad_xhat, local_grad_xhatx, grad_weight_bn, grad_bias_bn]. Reference: snn.cpp:317-327 -> snn_kernel_bp.cu:348-392."""
    return list(_bn_backward_local(x_bn, grad_y_bn, weight_bn, bias_bn, ivar, mean, (0.0, 0.0, 0.0, 0.0), False))


def bn_bp_dist2(x_bn, weight_bn, bias_bn, ivar, mean, dim_bn, grad_y_bn, grad_xhat, grad_xhatx):
    """Returns grad_x_bn from all-reduced channel means. Reference: snn.cpp:343-355 -> snn_kernel_bp.cu:394-425."""
    return _capi.bn_lif_bwd_input(x_bn, grad_y_bn, weight_bn, bias_bn, ivar, mean, grad_xhat, grad_xhatx,
                                  0.0, 0.0, 0.0, 0.0, fire=False)


def bn_fire_bp_dist1(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_spike, alpha, thresh, beta, interval):
    """Returns [local_grad_xhat, local_grad_xhatx, grad_weight_bn, grad_bias_bn]. Reference: snn.cpp:405-421 -> snn_kernel_bp.cu:753-806."""
    return list(_bn_backward_local(spatial, grad_spike, weight_bn, bias_bn, ivar, mean,
                                   (alpha, thresh, beta, interval), True))


def bn_fire_bp_dist2(spatial, weight_bn, bias_bn, ivar, mean, grad_spike, grad_xhat, grad_xhatx,
                     alpha, thresh, beta, interval):
    """Returns grad_spatial from all-reduced channel means. Reference: snn.cpp:442-460 -> snn_kernel_bp.cu:808-854."""
    return _capi.bn_lif_bwd_input(spatial, grad_spike, weight_bn, bias_bn, ivar, mean, grad_xhat,
                                  grad_xhatx, alpha, thresh, beta, interval, fire=True)


def _bn_spikes_again(spatial, weight_bn, bias_bn, ivar, mean, alpha, thresh):
    """Spikes rebuilt at backward time with w' = weight*ivar (reference: bn_fire_us_fp_kernel,
    snn_kernel_bp.cu:481-530); only the spikes are materialised, they are a GEMM / conv operand."""
    return _capi.bn_lif_fwd(spatial, weight_bn, bias_bn, None, mean, 0.0, alpha, thresh, ivar=ivar)[1]


def bn_fire_fc_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_fc, bias_fc, alpha, thresh):
    """Returns [ivar, fc]. Reference: snn.cpp:85-101 -> snn_kernel_fp.cu:244-291."""
    ivar, spike = bn_fire_s_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, alpha, thresh)
    return [ivar, fc_fp(spike, weight_fc, bias_fc)]


def bn_fire_fc_bp(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_fc, weight_fc, bias_fc, dim_fc,
                  alpha, thresh, beta, interval):
    """Returns [grad_spatial, grad_weight_bn, grad_bias_bn, grad_weight_fc, grad_bias_fc]. Reference: snn.cpp:484-504 -> snn_kernel_bp.cu:860-962."""
    spike = _bn_spikes_again(spatial, weight_bn, bias_bn, ivar, mean, alpha, thresh)
    grad_spike, grad_w, grad_b = _fc_grads(_rows(spike), grad_fc, weight_fc, dim_fc)
    gx, gwb, gbb = _bn_backward(spatial, grad_spike.view(spatial.shape), weight_bn, bias_bn, ivar, mean,
                                (alpha, thresh, beta, interval), True)
    return [gx, gwb, gbb, grad_w, grad_b]


def bn_fire_fc_bp_dist1(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_fc, weight_fc, bias_fc,
                        dim_fc, alpha, thresh, beta, interval):
    """Returns [grad_spike, local_grad_xhat, local_grad_xhatx, grad_weight_bn, grad_bias_bn, grad_weight_fc, grad_bias_fc]. Reference: snn.cpp:528-551 -> snn_kernel_bp.cu:966-1061."""
    spike = _bn_spikes_again(spatial, weight_bn, bias_bn, ivar, mean, alpha, thresh)
    grad_spike, grad_w, grad_b = _fc_grads(_rows(spike), grad_fc, weight_fc, dim_fc)
    grad_spike = grad_spike.view(spatial.shape)
    gxhat, gxhatx, gwb, gbb = _bn_backward_local(spatial, grad_spike, weight_bn, bias_bn, ivar, mean,
                                                 (alpha, thresh, beta, interval), True)
    return [grad_spike, gxhat, gxhatx, gwb, gbb, grad_w, grad_b]


def bn_fire_conv_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, weight_conv, bias_conv, stride,
                    padding, dilation, groups, benchmark, deterministic, alpha, thresh):
    """Returns [ivar, conv]. Reference: snn.cpp:162-187 -> snn_kernel_fp.cu:361-410."""
    ivar, spike = bn_fire_s_fp(spatial, weight_bn, bias_bn, var, mean, eps_bn, alpha, thresh)
    return [ivar, conv_fp(spike, weight_conv, bias_conv, stride, padding, dilation, groups, benchmark,
                          deterministic)]


def bn_fire_conv_bp(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_conv, weight_conv, stride,
                    padding, dilation, groups, benchmark, deterministic, allow_tf32, dim_conv,
                    alpha, thresh, beta, interval):
    """Returns [grad_spatial, grad_weight_bn, grad_bias_bn, grad_weight_conv, grad_bias_conv]. Reference: snn.cpp:630-658 -> snn_kernel_bp.cu:1180-1262."""
    spike = _bn_spikes_again(spatial, weight_bn, bias_bn, ivar, mean, alpha, thresh)
    grad_spike, grad_w, grad_b = _conv_grads(spike, grad_conv, weight_conv, stride, padding, dilation,
                                             groups, dim_conv)
    gx, gwb, gbb = _bn_backward(spatial, grad_spike.view(spatial.shape), weight_bn, bias_bn, ivar, mean,
                                (alpha, thresh, beta, interval), True)
    return [gx, gwb, gbb, grad_w, grad_b]


def bn_fire_conv_bp_dist1(spatial, weight_bn, bias_bn, ivar, mean, dim_bn, grad_conv, weight_conv, stride,
                          padding, dilation, groups, benchmark, deterministic, allow_tf32, dim_conv,
                          alpha, thresh, beta, interval):
    """Returns [grad_spike, local_grad_xhat, local_grad_xhatx, grad_weight_bn, grad_bias_bn, grad_weight_conv, grad_bias_conv]. Reference: snn.cpp:687-716 -> snn_kernel_bp.cu:1265-1340."""
    spike = _bn_spikes_again(spatial, weight_bn, bias_bn, ivar, mean, alpha, thresh)
    grad_spike, grad_w, grad_b = _conv_grads(spike, grad_conv, weight_conv, stride, padding, dilation,
                                             groups, dim_conv)
    grad_spike = grad_spike.view(spatial.shape)
    gxhat, gxhatx, gwb, gbb = _bn_backward_local(spatial, grad_spike, weight_bn, bias_bn, ivar, mean,
                                                 (alpha, thresh, beta, interval), True)
    return [grad_spike, gxhat, gxhatx, gwb, gbb, grad_w, grad_b]
