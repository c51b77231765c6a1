"""ctypes binding of libsnn_b200.so (C ABI declared in include/snn_b200.h).

There is exactly one backend. If the shared library has not been built, or a call returns
a non-zero status, this module raises; it never falls back to another implementation.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libsnn_b200.so")

SNN_OK = 0
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3}
STATE_DTYPE = {torch.float32: torch.float32, torch.bfloat16: torch.float32,
               torch.float16: torch.float32, torch.float64: torch.float64}

# every symbol include/snn_b200.h declares: (restype, argtypes)
_vp, _i64, _f32, _int, _sz = (ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int,
                              ctypes.c_size_t)
SIGNATURES = {
    "snn_version": (_int, []),
    "snn_status_string": (ctypes.c_char_p, [_int]),
    "snn_last_cuda_error": (_int, []),
    "snn_lif_fwd": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _f32, _f32, _vp]),
    "snn_lif_bwd_workspace_bytes": (_i64, [_i64, _i64, _int]),
    "snn_lif_bwd": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _f32, _f32, _f32, _f32, _vp, _sz, _vp]),
    "snn_spike_unpack": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "snn_copy_rows_async": (_int, [_vp, _sz, _vp, _sz, _sz, _i64, _int, _vp]),
    "snn_lif_bwd_noalloc": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _f32, _f32, _f32, _f32, _vp]),
    "snn_lif_add_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _f32, _f32, _vp]),
    "snn_lif_add_bwd": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _f32, _f32, _f32, _f32, _vp]),
    "snn_lif_pool_fwd": (_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _f32, _f32, _vp]),
    "snn_lif_pool_bwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _int, _f32, _f32, _f32, _f32, _vp]),
    "snn_linear_lif_fwd_supported": (_int, [_i64, _i64, _i64, _i64, _int]),
    "snn_linear_lif_fwd_plan": (_int, [_i64, _i64, _i64, _i64, _int, _int]),
    "snn_linear_lif_fwd": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _f32, _f32, _vp]),
    "snn_linear_lif_error": (_int, [_int]),
    "snn_linear_lif_bwd_supported": (_int, [_i64, _i64, _i64, _i64, _int]),
    "snn_linear_lif_bwd_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _int]),
    "snn_linear_lif_bwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _int,
                                  _f32, _f32, _f32, _f32, _vp, _sz, _vp]),
    "snn_channel_bias_add": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "snn_channel_sum": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "snn_bn_lif_fwd": (_int, [_vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                              _int, _int, _f32, _f32, _vp]),
    "snn_bn_lif_bwd_sums": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                   _int, _int, _f32, _f32, _f32, _f32, _vp]),
    "snn_bn_channel_means": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, ctypes.c_double, _vp]),
    "snn_bn_lif_bwd_input": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                    _i64, _int, _int, _f32, _f32, _f32, _f32, _vp]),
}
STATIC_SCRATCH_BYTES = 64 * 1024 * 1024


# NVTX ranges around every op (and, in example/ddp.py, around every gradient bucket's all-reduce), so
# that a timeline tool shows which layer's kernels and which bucket a span belongs to. Off unless
# SNN_NVTX=1: a range push/pop per op is host work the hot loop does not need. The reference's DDP
# has the same hooks behind its `prof` switch (apex/parallel/distributed.py:359-360, 516-517).
NVTX = os.environ.get("SNN_NVTX", "0") == "1"


def nvtx_range(name):
    """Decorator: run the function inside an NVTX range called ``name`` when SNN_NVTX=1."""
    def wrap(fn):
        if not NVTX:
            return fn
        import functools

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        return inner
    return wrap


class SnnError(RuntimeError):
    """A C-ABI call returned a non-zero snn_status."""

    def __init__(self, fn, status, detail):
        super().__init__(f"{fn} failed: status {status} ({detail})")
        self.status = status


_lib = None


def lib():
    """Load libsnn_b200.so once; raise if it is missing (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with "
                "`python -m snn_gpu_training_bptt_b200.build` (needs nvcc). "
                "There is no CPU or PyTorch fallback for these ops.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = restype, argtypes
        _lib = handle
    return _lib


def check(fn_name, status):
    if status != SNN_OK:
        L = lib()
        detail = L.snn_status_string(status).decode()
        if status == 7:
            detail += f", cudaError {L.snn_last_cuda_error()}"
        raise SnnError(fn_name, status, detail)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(t, name):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if t.dtype not in DTYPE_CODE:
        raise TypeError(f"{name}: unsupported dtype {t.dtype}; use float32, bfloat16, float16 or float64")
    if t.dim() < 2:
        raise ValueError(f"{name} must be time-major [T, B, ...]")
    if t.shape[0] < 1:
        raise ValueError(f"{name} has an empty time axis")


def is_time_major_dense(t):
    """True if ``t`` can be handed to the kernels as it is: element (time, neuron) lives at
    time * (numel / T) + f(neuron) for some fixed one-to-one layout f of the neurons of one
    time step. That holds for contiguous tensors and equally for e.g. a channels-last batch
    of images viewed as [T, B, C, H, W]: neurons are independent, so their order inside a
    time step does not matter as long as every time step uses the same one."""
    T = t.shape[0]
    step = t.numel() // T if T else 0
    if T > 1 and t.stride(0) != step:
        return False
    expect = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(t.shape[1:], t.stride()[1:]) if sz > 1),
                               key=lambda p: p[1]):
        if stride != expect:
            return False
        expect *= size
    return expect == step or step == 0


def as_time_major_dense(t):
    return t if is_time_major_dense(t) else t.contiguous()


def like_layout(t, ref):
    """``t`` with exactly ``ref``'s strides (copying only if they differ)."""
    if t.stride() == ref.stride():
        return t
    out = torch.empty_strided(ref.shape, ref.stride(), dtype=t.dtype, device=t.device)
    out.copy_(t)
    return out


def bits_dtype(T):
    if T > 32:
        raise ValueError("packed spike words cover at most 32 time steps")
    return torch.uint8 if T <= 8 else (torch.int16 if T <= 16 else torch.int32)


@nvtx_range("snn.lif_fwd")
def lif_fwd(x, alpha, thresh, want_spike=True, want_mem=False, want_bits=False):
    """Run snn_lif_fwd on a [T, ...] CUDA tensor; returns (spike, mem, bits) with None for
    outputs not requested. Launches on torch's current stream of x's device."""
    _require_cuda(x, "spatial")
    x = as_time_major_dense(x)
    T = x.shape[0]
    N = x.numel() // T
    with torch.cuda.device(x.device):
        spike = torch.empty_like(x) if want_spike else None
        mem = torch.empty_like(x, dtype=STATE_DTYPE[x.dtype]) if want_mem else None
        bits = torch.empty_like(x[0], dtype=bits_dtype(T)) if want_bits else None
        if N == 0:
            return spike, mem, bits
        rc = lib().snn_lif_fwd(_ptr(x), _ptr(spike), _ptr(mem), _ptr(bits), T, N,
                               DTYPE_CODE[x.dtype], float(alpha), float(thresh), _stream(x.device))
    check("snn_lif_fwd", rc)
    return spike, mem, bits


@nvtx_range("snn.lif_bwd")
def lif_bwd(x, grad_spike, alpha, thresh, beta, interval):
    """Run snn_lif_bwd; returns grad_x shaped like x."""
    _require_cuda(x, "spatial")
    _require_cuda(grad_spike, "grad_spike")
    if grad_spike.shape != x.shape:
        raise ValueError(f"grad_spike shape {tuple(grad_spike.shape)} != spatial shape {tuple(x.shape)}")
    if grad_spike.dtype != x.dtype or grad_spike.device != x.device:
        raise TypeError("grad_spike must have spatial's dtype and device")
    x = as_time_major_dense(x)
    g = like_layout(grad_spike, x)
    T = x.shape[0]
    N = x.numel() // T
    code = DTYPE_CODE[x.dtype]
    with torch.cuda.device(x.device):
        need = lib().snn_lif_bwd_workspace_bytes(T, N, code)
        if need < 0:
            check("snn_lif_bwd_workspace_bytes", -need)
        ws = torch.empty(need, dtype=torch.uint8, device=x.device) if need > 0 else None
        gx = torch.empty_like(x)
        if N == 0:
            return gx
        rc = lib().snn_lif_bwd(_ptr(x), _ptr(g), _ptr(gx), T, N, code, float(alpha), float(thresh),
                               float(beta), float(interval), _ptr(ws), need, _stream(x.device))
    check("snn_lif_bwd", rc)
    return gx


LIF_ADD_MAX_T = 16


def lif_add_operands(a, b):
    """(a, b) made time-major dense with IDENTICAL strides (b is copied into a's layout if it
    differs), after the checks shared by both directions."""
    _require_cuda(a, "current")
    _require_cuda(b, "shortcut")
    if a.shape != b.shape or a.dtype != b.dtype or a.device != b.device:
        raise ValueError("lif_add: the two currents must agree in shape, dtype and device")
    a = as_time_major_dense(a)
    return a, like_layout(b, a)


@nvtx_range("snn.lif_add_fwd")
def lif_add_fwd(a, b, alpha, thresh):
    """snn_lif_add_fwd: spikes of LIF(a + b) for two [T, ...] tensors already in one layout."""
    T = a.shape[0]
    N = a.numel() // T
    with torch.cuda.device(a.device):
        spike = torch.empty_like(a)
        if N == 0:
            return spike
        rc = lib().snn_lif_add_fwd(_ptr(a), _ptr(b), _ptr(spike), T, N, DTYPE_CODE[a.dtype], float(alpha),
                                   float(thresh), _stream(a.device))
    check("snn_lif_add_fwd", rc)
    return spike


@nvtx_range("snn.lif_add_bwd")
def lif_add_bwd(a, b, grad_spike, alpha, thresh, beta, interval):
    """snn_lif_add_bwd: dL/d(a + b), shaped and laid out like a."""
    _require_cuda(grad_spike, "grad_spike")
    if grad_spike.shape != a.shape or grad_spike.dtype != a.dtype or grad_spike.device != a.device:
        raise ValueError("grad_spike must have the currents' shape, dtype and device")
    g = like_layout(grad_spike, a)
    T = a.shape[0]
    N = a.numel() // T
    with torch.cuda.device(a.device):
        gx = torch.empty_like(a)
        if N == 0:
            return gx
        rc = lib().snn_lif_add_bwd(_ptr(a), _ptr(b), _ptr(g), _ptr(gx), T, N, DTYPE_CODE[a.dtype], float(alpha),
                                   float(thresh), float(beta), float(interval), _stream(a.device))
    check("snn_lif_add_bwd", rc)
    return gx


def copy_rows_(dst, src):
    """One pitched transfer between a host and a device 2-D tensor view (rows may be strided, the
    elements of a row must be contiguous): dst[r, :] = src[r, :] on torch's current stream."""
    if dst.dim() != 2 or src.dim() != 2 or dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError("copy_rows_: dst and src must be 2-D views of the same shape and dtype")
    if dst.is_cuda == src.is_cuda:
        raise ValueError("copy_rows_: one side must be host memory, the other device memory")
    rows, cols = dst.shape
    if rows and cols and (dst.stride(1) != 1 or src.stride(1) != 1):
        raise ValueError("copy_rows_: rows must be contiguous")
    es = dst.element_size()
    dev = dst.device if dst.is_cuda else src.device
    with torch.cuda.device(dev):
        rc = lib().snn_copy_rows_async(_ptr(dst), dst.stride(0) * es if rows > 1 else cols * es, _ptr(src),
                                       src.stride(0) * es if rows > 1 else cols * es, cols * es, rows,
                                       1 if dst.is_cuda else 0, _stream(dev))
    check("snn_copy_rows_async", rc)
    return dst


def spike_unpack(bits, T, dtype=torch.float32):
    """Expand packed spike words [B, ...] into a dense [T, B, ...] 0/1 tensor."""
    if not bits.is_cuda:
        raise ValueError("bits must be a CUDA tensor")
    if bits.dtype != bits_dtype(T):
        raise TypeError(f"bits dtype {bits.dtype} does not match T={T}")
    if not is_time_major_dense(bits.unsqueeze(0)):
        bits = bits.contiguous()
    N = bits.numel()
    with torch.cuda.device(bits.device):
        out = torch.empty_strided((T,) + tuple(bits.shape), (N,) + tuple(bits.stride()),
                                  dtype=dtype, device=bits.device)
        rc = lib().snn_spike_unpack(_ptr(bits), _ptr(out), T, N, DTYPE_CODE[dtype], _stream(bits.device))
    check("snn_spike_unpack", rc)
    return out


def lif_bwd_noalloc(x, grad_spike, grad_x, alpha, thresh, beta, interval):
    """snn_lif_bwd_noalloc: backward into the caller's ``grad_x`` with the membrane scratch held
    inside the library, for callers that must not allocate on the device. All three tensors must
    already be dense, time-major, of one dtype and layout; nothing is allocated or copied here.
    Raises SnnError (status 8) if T*N*state bytes exceed STATIC_SCRATCH_BYTES."""
    for name, t in (("spatial", x), ("grad_spike", grad_spike), ("grad_x", grad_x)):
        _require_cuda(t, name)
        if not is_time_major_dense(t):
            raise ValueError(f"{name} must be dense and time-major (no copy is made on this path)")
    if not (x.shape == grad_spike.shape == grad_x.shape and x.stride() == grad_spike.stride() == grad_x.stride()):
        raise ValueError("spatial, grad_spike and grad_x must share shape and layout")
    if not (x.dtype == grad_spike.dtype == grad_x.dtype):
        raise TypeError("spatial, grad_spike and grad_x must share a dtype")
    T = x.shape[0]
    N = x.numel() // T
    with torch.cuda.device(x.device):
        rc = lib().snn_lif_bwd_noalloc(_ptr(x), _ptr(grad_spike), _ptr(grad_x), T, N, DTYPE_CODE[x.dtype],
                                       float(alpha), float(thresh), float(beta), float(interval),
                                       _stream(x.device))
    check("snn_lif_bwd_noalloc", rc)
    return grad_x


# ----------------------------------------------------------------------------------------------
# batch-norm family
# ----------------------------------------------------------------------------------------------
def _bn_geometry(x):
    """(x made dense, T, N, C, inner) for a [T, B, C] or [T, B, C, H, W] tensor. ``inner`` is the
    number of consecutive neurons that share a channel: H*W for the contiguous layout, 1 for
    [T, B, C] and for channels-last images."""
    x = as_time_major_dense(x)
    T, C = x.shape[0], x.shape[2]
    N = x.numel() // T
    if x.dim() == 3 or x.numel() == 0:
        return x, T, N, C, 1
    if x.is_contiguous():
        return x, T, N, C, N // (x.shape[1] * C)
    if x.stride(2) == 1:                       # channels-last: channel is the fastest axis
        return x, T, N, C, 1
    x = x.contiguous()
    return x, T, N, C, N // (x.shape[1] * C)


def _f32c(t, C, name):
    if t.dtype != torch.float32 or not t.is_cuda or t.numel() != C:
        raise TypeError(f"{name} must be a float32 CUDA tensor with {C} elements")
    return t.contiguous()


@nvtx_range("snn.bn_lif_fwd")
def bn_lif_fwd(x, weight, bias, var, mean, eps, alpha, thresh, fire=True, want_mem=False, ivar=None):
    """snn_bn_lif_fwd. Returns (ivar, out, mem): out = spikes (fire) or the normalised tensor.
    Pass ``var=None, ivar=<tensor>`` to rebuild with w' = weight*ivar (backward-time form)."""
    _require_cuda(x, "spatial")
    if x.dtype == torch.float64:
        raise TypeError("the batch-norm family supports float32, bfloat16 and float16")
    x, T, N, C, inner = _bn_geometry(x)
    w, b, m = (_f32c(t, C, n) for t, n in ((weight, "weight_bn"), (bias, "bias_bn"), (mean, "mean")))
    v = _f32c(var, C, "var") if var is not None else None
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        mem = torch.empty_like(x, dtype=torch.float32) if (want_mem and fire) else None
        ivar = torch.empty_like(w) if v is not None else _f32c(ivar, C, "ivar")
        if N == 0:
            return ivar, out, mem
        rc = lib().snn_bn_lif_fwd(_ptr(x), _ptr(w), _ptr(b), _ptr(v), _ptr(m), float(eps), _ptr(out),
                                  _ptr(mem), _ptr(ivar), T, N, C, inner, DTYPE_CODE[x.dtype], int(fire),
                                  float(alpha), float(thresh), _stream(x.device))
    check("snn_bn_lif_fwd", rc)
    return ivar, out, mem


@nvtx_range("snn.bn_lif_bwd_sums")
def bn_lif_bwd_sums(x, grad, weight, bias, ivar, mean, alpha, thresh, beta, interval, fire=True):
    """snn_bn_lif_bwd_sums. Returns (x_dense, grad_dense, sum_g, sum_gx, count) where count is the
    number of values per channel (T*B*inner)."""
    _require_cuda(x, "spatial")
    _require_cuda(grad, "grad")
    x, T, N, C, inner = _bn_geometry(x)
    g = like_layout(grad, x)
    w, b, iv, m = (_f32c(t, C, n) for t, n in ((weight, "weight_bn"), (bias, "bias_bn"), (ivar, "ivar"), (mean, "mean")))
    with torch.cuda.device(x.device):
        sums = torch.empty((2, C), dtype=torch.float32, device=x.device)
        rc = lib().snn_bn_lif_bwd_sums(_ptr(x), _ptr(g), _ptr(w), _ptr(b), _ptr(iv), _ptr(m), _ptr(sums[0]),
                                       _ptr(sums[1]), T, N, C, inner, DTYPE_CODE[x.dtype], int(fire),
                                       float(alpha), float(thresh), float(beta), float(interval),
                                       _stream(x.device))
    check("snn_bn_lif_bwd_sums", rc)
    return x, g, sums[0], sums[1], T * N // C


def bn_channel_means(sum_g, sum_gx, weight, count):
    C = sum_g.numel()
    with torch.cuda.device(sum_g.device):
        out = torch.empty((2, C), dtype=torch.float32, device=sum_g.device)
        rc = lib().snn_bn_channel_means(_ptr(sum_g), _ptr(sum_gx), _ptr(_f32c(weight, C, "weight_bn")),
                                        _ptr(out[0]), _ptr(out[1]), C, float(count), _stream(sum_g.device))
    check("snn_bn_channel_means", rc)
    return out[0], out[1]


@nvtx_range("snn.bn_lif_bwd_input")
def bn_lif_bwd_input(x, grad, weight, bias, ivar, mean, gxhat, gxhatx, alpha, thresh, beta, interval,
                     fire=True):
    """snn_bn_lif_bwd_input. Returns grad_x laid out like x."""
    _require_cuda(x, "spatial")
    x, T, N, C, inner = _bn_geometry(x)
    g = like_layout(grad, x)
    w, b, iv, m, gh, ghx = (_f32c(t, C, n) for t, n in (
        (weight, "weight_bn"), (bias, "bias_bn"), (ivar, "ivar"), (mean, "mean"),
        (gxhat.reshape(-1), "grad_xhat"), (gxhatx.reshape(-1), "grad_xhatx")))
    with torch.cuda.device(x.device):
        gx = torch.empty_like(x)
        if N == 0:
            return gx
        rc = lib().snn_bn_lif_bwd_input(_ptr(x), _ptr(g), _ptr(w), _ptr(b), _ptr(iv), _ptr(m), _ptr(gh),
                                        _ptr(ghx), _ptr(gx), T, N, C, inner, DTYPE_CODE[x.dtype], int(fire),
                                        float(alpha), float(thresh), float(beta), float(interval),
                                        _stream(x.device))
    check("snn_bn_lif_bwd_input", rc)
    return gx


# ----------------------------------------------------------------------------------------------
# LIF + 2x2 average pool, fused (channels-last images)
# ----------------------------------------------------------------------------------------------
def _channels_last_5d(x):
    """[T, B, C, H, W] tensor whose memory order is (T, B, H, W, C); copies only if it is not."""
    T, B, C, H, W = x.shape
    want = (B * H * W * C, H * W * C, 1, W * C, C)
    if tuple(x.stride()) == want:
        return x
    out = torch.empty_strided(x.shape, want, dtype=x.dtype, device=x.device)
    out.copy_(x)
    return out


@nvtx_range("snn.lif_pool_fwd")
def lif_pool_fwd(x, alpha, thresh):
    """Pooled spikes [T, B, C, H/2, W/2] (channels-last memory order) of the LIF of x."""
    _require_cuda(x, "spatial")
    if x.dim() != 5 or x.shape[3] % 2 or x.shape[4] % 2:
        raise ValueError("fused LIF+pool needs [T, B, C, H, W] with even H and W")
    x = _channels_last_5d(x)
    T, B, C, H, W = x.shape
    with torch.cuda.device(x.device):
        out = torch.empty_strided((T, B, C, H // 2, W // 2),
                                  (B * (H // 2) * (W // 2) * C, (H // 2) * (W // 2) * C, 1, (W // 2) * C, C),
                                  dtype=x.dtype, device=x.device)
        rc = lib().snn_lif_pool_fwd(_ptr(x), _ptr(out), T, B, H, W, C, DTYPE_CODE[x.dtype], float(alpha),
                                    float(thresh), _stream(x.device))
    check("snn_lif_pool_fwd", rc)
    return x, out


@nvtx_range("snn.lif_pool_bwd")
def lif_pool_bwd(x, grad_out, alpha, thresh, beta, interval):
    """grad w.r.t. x (channels-last, as produced by lif_pool_fwd's first return value)."""
    T, B, C, H, W = x.shape
    g = _channels_last_5d(grad_out)
    with torch.cuda.device(x.device):
        gx = torch.empty_like(x)
        rc = lib().snn_lif_pool_bwd(_ptr(x), _ptr(g), _ptr(gx), T, B, H, W, C, DTYPE_CODE[x.dtype],
                                    float(alpha), float(thresh), float(beta), float(interval), _stream(x.device))
    check("snn_lif_pool_bwd", rc)
    return gx


# ----------------------------------------------------------------------------------------------
# per-channel bias add / bias-gradient sum for [N, C, ...] activations (dim 1 = channels)
# ----------------------------------------------------------------------------------------------
def _channel_geometry(t):
    """(outer, C, inner) if ``t`` ([N, C, ...]) is laid out as (o*C + c)*inner + i, else None."""
    C = t.shape[1]
    if t.numel() == 0:
        return 0, C, 1
    if t.is_contiguous():
        inner = t.numel() // (t.shape[0] * C)
        return t.shape[0], C, inner
    if t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last):
        return t.numel() // C, C, 1
    return None


@nvtx_range("snn.channel_bias_add")
def channel_bias_add_(y, bias):
    """y[:, c] += bias[c] in place (y: [N, C, ...] contiguous or channels-last; bias fp32 [C])."""
    geo = _channel_geometry(y)
    if geo is None or y.dtype not in DTYPE_CODE or y.dtype == torch.float64 or bias.dtype != torch.float32:
        raise TypeError("channel_bias_add_: needs a dense f32/bf16/f16 activation and an fp32 bias")
    outer, C, inner = geo
    with torch.cuda.device(y.device):
        rc = lib().snn_channel_bias_add(_ptr(y), _ptr(bias.contiguous()), outer, C, inner, DTYPE_CODE[y.dtype],
                                        _stream(y.device))
    check("snn_channel_bias_add", rc)
    return y


@nvtx_range("snn.channel_sum")
def channel_sum(grad):
    """fp32 [C] sums of grad ([N, C, ...]) over every axis but the channel axis."""
    geo = _channel_geometry(grad)
    if geo is None:
        grad = grad.contiguous()
        geo = _channel_geometry(grad)
    outer, C, inner = geo
    with torch.cuda.device(grad.device):
        out = torch.empty(C, dtype=torch.float32, device=grad.device)
        rc = lib().snn_channel_sum(_ptr(grad), _ptr(out), outer, C, inner, DTYPE_CODE[grad.dtype],
                                   _stream(grad.device))
    check("snn_channel_sum", rc)
    return out


# ----------------------------------------------------------------------------------------------
# fused synaptic linear + LIF forward (tcgen05)
# ----------------------------------------------------------------------------------------------
def linear_lif_supported(x, weight):
    """True if the tcgen05 kernel covers this problem (bf16, 2 <= T <= 16, tile-aligned sizes)."""
    if x.dim() != 3 or weight.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    T, B, K = x.shape
    return bool(lib().snn_linear_lif_fwd_supported(T, B, K, weight.shape[0], DTYPE_CODE[x.dtype]))


@nvtx_range("snn.linear_lif_fwd")
def linear_lif_fwd(x, weight, bias, alpha, thresh, want_current=True):
    """(current, spike) of ``LIF(x @ weight^T + bias)`` in one kernel. x [T, B, K] bf16, weight
    [M, K] (cast to bf16 if needed), bias fp32 [M] or None."""
    if not linear_lif_supported(x, weight):
        raise ValueError("linear_lif_fwd: unsupported problem (needs bf16, 2 <= T <= 16, B a multiple of "
                         "128 / (T rounded up to 2, 4, 8 or 16), K % 64 == 0, M % 128 == 0)")
    x = x.contiguous()
    w = weight.to(torch.bfloat16).contiguous()
    b = bias.float().contiguous() if bias is not None else None
    T, B, K = x.shape
    M = w.shape[0]
    if b is not None and b.numel() != M:
        raise ValueError("linear_lif_fwd: bias must have one entry per output neuron")
    with torch.cuda.device(x.device):
        spike = torch.empty((T, B, M), dtype=torch.bfloat16, device=x.device)
        current = torch.empty_like(spike) if want_current else None
        rc = lib().snn_linear_lif_fwd(_ptr(x), _ptr(w), _ptr(b), _ptr(current), _ptr(spike), T, B, K, M,
                                      DTYPE_CODE[x.dtype], float(alpha), float(thresh), _stream(x.device))
    check("snn_linear_lif_fwd", rc)
    return current, spike


def linear_lif_bwd_supported(x, weight):
    """True if the tcgen05 backward covers this problem (bf16 x, T <= 16, T*B >= 128, K >= 64, M >= 128)."""
    if x.dim() != 3 or weight.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    T, B, K = x.shape
    return bool(lib().snn_linear_lif_bwd_supported(T, B, K, weight.shape[0], DTYPE_CODE[x.dtype]))


@nvtx_range("snn.linear_lif_bwd")
def linear_lif_bwd(x, weight, current, grad_spike, alpha, thresh, beta, interval, need_grad_x=True,
                   need_grad_weight=True, need_grad_bias=True, grad_weight_dtype=torch.float32):
    """(grad_x, grad_weight, grad_bias) of ``LIF(x @ weight^T + bias)`` from the saved LIF input
    ``current`` and the upstream ``grad_spike``: the LIF reverse pass and both gradient GEMMs on the
    library's own kernels (snn_linear_lif_bwd). x [T, B, K], current / grad_spike [T, B, M] and
    weight [M, K] in bf16; grad_weight comes out in ``grad_weight_dtype`` (fp32 or bf16), grad_bias
    in fp32. Entries that are not needed are None."""
    if not linear_lif_bwd_supported(x, weight):
        raise ValueError("linear_lif_bwd: unsupported problem (needs bf16, T <= 16, T*B >= 128, K >= 64, "
                         "M >= 128, K % 64 == 0, M % 64 == 0)")
    if weight.dtype != torch.bfloat16 or current.dtype != torch.bfloat16:
        raise TypeError("linear_lif_bwd: weight and current must be bfloat16")
    if grad_weight_dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("linear_lif_bwd: grad_weight_dtype must be float32 or bfloat16")
    x, weight, current = x.contiguous(), weight.contiguous(), current.contiguous()
    grad_spike = grad_spike.to(torch.bfloat16).contiguous()
    T, B, K = x.shape
    M = weight.shape[0]
    if current.shape != (T, B, M) or grad_spike.shape != (T, B, M) or weight.shape[1] != K:
        raise ValueError("linear_lif_bwd: shape mismatch")
    need_grad_weight = need_grad_weight or need_grad_bias
    L = lib()
    with torch.cuda.device(x.device):
        need = L.snn_linear_lif_bwd_workspace_bytes(T, B, K, M, DTYPE_CODE[x.dtype])
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        gx = torch.empty_like(x) if need_grad_x else None
        gw = torch.empty((M, K), dtype=grad_weight_dtype, device=x.device) if need_grad_weight else None
        gb = torch.empty(M, dtype=torch.float32, device=x.device) if need_grad_bias else None
        rc = L.snn_linear_lif_bwd(_ptr(x), _ptr(weight), _ptr(current), _ptr(grad_spike), _ptr(gx), _ptr(gw),
                                  _ptr(gb), T, B, K, M, DTYPE_CODE[x.dtype], DTYPE_CODE[grad_weight_dtype],
                                  float(alpha), float(thresh), float(beta), float(interval), _ptr(ws), need,
                                  _stream(x.device))
    check("snn_linear_lif_bwd", rc)
    return gx, gw, gb


def linear_lif_error(reset=True):
    """0, or the code of a bounded wait that expired inside the fused kernel (synchronises)."""
    return lib().snn_linear_lif_error(1 if reset else 0)
