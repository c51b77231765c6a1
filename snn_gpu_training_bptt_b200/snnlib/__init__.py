"""Drop-in for the reference's compiled extension module ``snnlib``.

The reference builds ``snnlib`` from snnlib/cuda/snn.cpp (pybind11 table at snn.cpp:798-830)
and its only caller is snnlib/example/snnlib_func.py. This package exposes the same function
names with the same positional arguments and return values, backed by libsnn_b200.so
(hand-written sm_100a kernels behind a C ABI, see include/snn_b200.h) for the LIF fire path
and by one library GEMM / convolution over the merged [T*B, ...] batch where the reference
issues T separate cuBLAS / cuDNN calls.

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


def _rows(t):
    """[T, B, ...] -> [T*B, features] view (reference flattens C,H,W: snn_kernel_fp.cu:349)."""
    return t.reshape(t.shape[0] * t.shape[1], -1)


def fc_fp(spatial, weight_fc, bias_fc):
    """fc[t] = spatial[t] @ W^T + b for every t. Reference: snn.cpp:130-136 -> snn_kernel_fp.cu:332-357."""
    T, B = spatial.shape[0], spatial.shape[1]
    return F.linear(_rows(spatial), _cast(weight_fc, spatial), _cast(bias_fc, spatial)).view(
        T, B, weight_fc.shape[0])


def _fc_grads(inp_rows, grad_fc, weight_fc, dim_fc):
    g = _rows(grad_fc)
    grad_in = g @ _cast(weight_fc, g)            # [T*B, in]
    grad_w = (g.t() @ inp_rows).to(weight_fc.dtype)   # [out, in], summed over t and b
    grad_b = torch.sum(grad_fc, dim=tuple(dim_fc), dtype=weight_fc.dtype)
    return grad_in, grad_w, grad_b


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
    y = F.conv2d(_images(spatial), _cast(weight_conv, spatial), _cast(bias_conv, spatial),
                 tuple(stride), tuple(padding), tuple(dilation), groups)
    return y.view((T, B) + tuple(y.shape[1:]))


def _conv_grads(inp, grad_conv, weight_conv, stride, padding, dilation, groups, dim_conv):
    g = _images(grad_conv)
    x = _images(inp)
    grad_in, grad_w = torch.ops.aten.convolution_backward(
        g, x, _cast(weight_conv, g), None, list(stride), list(padding), list(dilation), False,
        [0, 0], groups, [True, True, False])[:2]
    grad_b = torch.sum(grad_conv, dim=tuple(dim_conv), dtype=weight_conv.dtype)
    return grad_in, grad_w.to(weight_conv.dtype), grad_b


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
# batch-norm family: names of the reference's table that are not built yet
# ------------------------------------------------------------------------------------------
def _not_built(name, where):
    def stub(*args, **kwargs):
        raise NotImplementedError(
            f"snnlib.{name} (reference: snnlib/cuda/snn.cpp:{where}) is outside the LIF fire "
            "path this library implements; no substitute implementation is provided")
    stub.__name__ = name
    return stub


bn_fp = _not_built("bn_fp", "30-39")
bn_bp = _not_built("bn_bp", "293-303")
bn_fire_s_fp = _not_built("bn_fire_s_fp", "55-66")
bn_fire_bp = _not_built("bn_fire_bp", "373-387")
bn_fire_fc_fp = _not_built("bn_fire_fc_fp", "85-101")
bn_fire_fc_bp = _not_built("bn_fire_fc_bp", "484-504")
bn_fire_conv_fp = _not_built("bn_fire_conv_fp", "162-187")
bn_fire_conv_bp = _not_built("bn_fire_conv_bp", "630-658")
bn_bp_dist1 = _not_built("bn_bp_dist1", "317-327")
bn_bp_dist2 = _not_built("bn_bp_dist2", "343-355")
bn_fire_bp_dist1 = _not_built("bn_fire_bp_dist1", "405-421")
bn_fire_bp_dist2 = _not_built("bn_fire_bp_dist2", "442-460")
bn_fire_fc_bp_dist1 = _not_built("bn_fire_fc_bp_dist1", "528-551")
bn_fire_conv_bp_dist1 = _not_built("bn_fire_conv_bp_dist1", "687-716")
