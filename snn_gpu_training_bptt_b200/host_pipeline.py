"""LIF forward+backward for tensors that live in HOST memory.

The C ABI works on device buffers. A caller whose currents and upstream gradients sit in
(pinned) host memory pays PCIe both ways; this helper hides as much of that as the bus
allows by cutting the neuron axis into chunks (neurons are independent, so chunking is
exact) and running chunks round-robin on a few CUDA streams: while one stream computes or
drains its results, another is already uploading the next chunk, so host->device and
device->host copies run concurrently with each other and with the kernels.
"""
import torch

from . import _capi


class HostLifPipeline:
    """Reusable staging buffers + streams for ``run``.

    T, N: time steps and neurons of the full [T, N] problem; ``chunk`` neurons per piece;
    ``lanes`` concurrent streams (each owns one set of device staging buffers).
    """

    def __init__(self, T, N, dtype=torch.float32, chunk=1 << 22, lanes=3, device=None, pitched=True):
        if T > 32:
            raise ValueError("the host pipeline covers T <= 32 (longer time axes need a scratch tensor)")
        self.T, self.N, self.dtype = T, N, dtype
        self.pitched = pitched          # one pitched copy per [T, chunk] slab instead of T row copies
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.chunk = min(chunk, N)
        self.lanes = []
        for _ in range(max(1, min(lanes, (N + self.chunk - 1) // self.chunk))):
            bufs = [torch.empty((T, self.chunk), dtype=dtype, device=self.device) for _ in range(4)]
            self.lanes.append((torch.cuda.Stream(self.device), bufs))
        self.h2d_bytes = 2 * T * N * torch.empty(0, dtype=dtype).element_size()
        self.d2h_bytes = self.h2d_bytes
        self.launches_per_run = 2 * ((N + self.chunk - 1) // self.chunk)

    def run(self, x_host, g_host, spike_host, gx_host, alpha, thresh, beta, interval):
        """x_host, g_host -> spike_host, gx_host; all [T, N] host tensors (pinned for overlap).
        Returns after every copy has landed."""
        T, N = self.T, self.N
        caller = torch.cuda.current_stream(self.device)
        lib = _capi.lib()
        code = _capi.DTYPE_CODE[self.dtype]
        for lane_stream, _ in self.lanes:
            lane_stream.wait_stream(caller)
        for k, lo in enumerate(range(0, N, self.chunk)):
            n = min(self.chunk, N - lo)
            stream, (xd, gd, sd, gxd) = self.lanes[k % len(self.lanes)]
            with torch.cuda.stream(stream):
                if n == self.chunk:
                    xv, gv, sv, gxv = xd, gd, sd, gxd
                else:  # ragged last chunk: dense [T, n] views at the front of the buffers
                    xv, gv, sv, gxv = (b.view(-1)[:T * n].view(T, n) for b in (xd, gd, sd, gxd))
                if self.pitched:
                    _capi.copy_rows_(xv, x_host[:, lo:lo + n])
                    _capi.copy_rows_(gv, g_host[:, lo:lo + n])
                else:
                    for t in range(T):
                        xv[t].copy_(x_host[t, lo:lo + n], non_blocking=True)
                        gv[t].copy_(g_host[t, lo:lo + n], non_blocking=True)
                sp = _capi._stream(self.device)
                _capi.check("snn_lif_fwd", lib.snn_lif_fwd(
                    _capi._ptr(xv), _capi._ptr(sv), None, None, T, n, code, float(alpha),
                    float(thresh), sp))
                _capi.check("snn_lif_bwd", lib.snn_lif_bwd(
                    _capi._ptr(xv), _capi._ptr(gv), _capi._ptr(gxv), T, n, code, float(alpha),
                    float(thresh), float(beta), float(interval), None, 0, sp))
                if self.pitched:
                    _capi.copy_rows_(spike_host[:, lo:lo + n], sv)
                    _capi.copy_rows_(gx_host[:, lo:lo + n], gxv)
                else:
                    for t in range(T):
                        spike_host[t, lo:lo + n].copy_(sv[t], non_blocking=True)
                        gx_host[t, lo:lo + n].copy_(gxv[t], non_blocking=True)
        for lane_stream, _ in self.lanes:
            caller.wait_stream(lane_stream)
        caller.synchronize()
