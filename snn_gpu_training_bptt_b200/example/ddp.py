"""Data-parallel gradient averaging overlapped with backward.

Behaviour to match: the reference trains with apex's ``DistributedDataParallel``
(snnlib/example/apex/parallel/distributed.py:129-639, used at
snnlib/example/train_test_imagenet_alexnet_dist.py:66): rank 0's parameters are broadcast
when the wrapper is built (distributed.py:253) and every step all ranks end up with
``sum(grad) * (1 / world_size)`` (distributed.py:449-454). As shipped, the reference never
actually overlaps that all-reduce with backward (its BN layers re-create parameters every
forward, which sends apex down its flat end-of-backward fallback, distributed.py:491-510).

This wrapper keeps the numerics and does overlap:
  * parameters are grouped, in reverse registration order (the order gradients become ready),
    into buckets of about ``bucket_mb`` megabytes;
  * every ``param.grad`` is a view into its bucket's flat buffer, so nothing is packed or
    unpacked;
  * a post-accumulate-grad hook counts arrivals; when a bucket is complete its all-reduce is
    issued on a side stream that waits only for the work recorded so far, so NCCL runs over
    NVLink while the remaining layers' BPTT kernels keep the SMs busy;
  * buckets are always reduced in bucket order, every bucket exactly once per backward, so every
    rank issues the same sequence of collectives whatever subset of its parameters received a
    gradient (a bucket that completes early waits for the buckets before it; ``finish()`` reduces
    what is left, untouched buckets included - their gradients are the zeros ``zero_grad()`` left).
    apex's fallback has the same property: it always reduces the whole flat gradient set
    (distributed.py:491-510). Ranks that issued different numbers of all-reduces would hang NCCL;
  * ``finish()`` (called automatically at the end of backward through an autograd engine
    callback) also makes the compute stream wait for the outstanding reductions - or, with
    ``defer_wait=True``, leaves that to whoever consumes the gradients: ``wait_bucket(k)`` makes
    the compute stream wait for bucket k only, so ``BucketSGD`` below updates the parameters of
    the early buckets while the last (unhidable) all-reduce is still in flight.
On CPU tensors (gloo) the same logic runs without streams.
"""
import os

import torch
import torch.distributed as dist

from .. import _capi


class DistributedDataParallel(torch.nn.Module):
    def __init__(self, module, bucket_mb=25.0, process_group=None, overlap=True, communicate=True, tail_mb=1.0,
                 defer_wait=False):
        """``communicate=False`` keeps all the bookkeeping but issues no all-reduce (a measuring aid:
        the step-time difference against the normal wrapper is the communication time that backward
        does not hide; gradients are then NOT averaged)."""
        super().__init__()
        self.module = module
        self.communicate = communicate
        self.defer_wait = defer_wait
        self.trace = None           # set to [] to record (bucket, ready, start, end) CUDA events per reduction
        self.group = process_group
        self.world_size = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.overlap = overlap
        self.params = [p for p in module.parameters() if p.requires_grad]
        self._broadcast_parameters()
        self._build_buckets(bucket_mb, tail_mb)
        self._pending = []          # indices of buckets whose reduction runs on the side stream
        self._next_bucket = 0       # buckets [0, _next_bucket) have been reduced in this backward
        self._callback_queued = False
        self._comm_stream = None
        dev = self.params[0].device if self.params else torch.device("cpu")
        if dev.type == "cuda":
            # SNN_DDP_COMM_PRIORITY=-1 runs the reductions on a high-priority stream
            prio = int(os.environ.get("SNN_DDP_COMM_PRIORITY", "0"))
            self._comm_stream = torch.cuda.Stream(dev, priority=prio)
        # NCCL averages in the reduction itself; gloo needs sum followed by a scale
        backend = dist.get_backend(process_group) if dist.is_initialized() else ""
        self._avg_op = dist.ReduceOp.AVG if backend == "nccl" else None
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._on_grad_ready)

    # ---- construction ------------------------------------------------------------------------
    def _broadcast_parameters(self):
        """Everyone starts from rank 0's parameters and buffers-as-parameters (running stats)."""
        if self.world_size == 1:
            return
        with torch.no_grad():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                dist.broadcast(t.data, src=0, group=self.group)

    def _build_buckets(self, bucket_mb, tail_mb):
        """``tail_mb`` (a number or a sequence of decreasing numbers): the LAST bucket holds the parameters of the first layers, whose gradients
        exist only when backward ends, so its all-reduce is the one nothing can hide. It is cut
        down to at most ``tail_mb`` megabytes (its other parameters become a bucket of their own
        that is ready earlier): measured on the VGG-style network at 2 GPUs, an 18 MB last bucket
        exposed 0.14 ms of a 3.4 ms step."""
        cap = int(bucket_mb * 1024 * 1024)
        self.buckets = []           # dict(flat=Tensor, params=[...], ready=int)
        self._bucket_of = {}
        current, size = [], 0
        order = list(reversed(self.params))
        groups = []
        for p in order:
            nbytes = p.numel() * p.element_size()
            if current and (size + nbytes > cap or p.dtype != current[0].dtype
                            or p.device != current[0].device):
                groups.append(current)
                current, size = [], 0
            current.append(p)
            size += nbytes
        if current:
            groups.append(current)
        caps = [] if tail_mb is None else ([tail_mb] if isinstance(tail_mb, (int, float)) else list(tail_mb))
        for cap_mb in caps:             # several caps cut the tail repeatedly: (1.0, 0.03) -> ..., <= 1 MB, <= 30 KB
            if not groups or len(groups[-1]) <= 1:
                break
            tail_cap = int(cap_mb * 1024 * 1024)
            last, tail, size = groups[-1], [], 0
            while len(last) > 1 and size + last[-1].numel() * last[-1].element_size() <= tail_cap:
                size += last[-1].numel() * last[-1].element_size()
                tail.insert(0, last.pop())
            if tail and sum(p.numel() * p.element_size() for p in last) > tail_cap:
                groups.append(tail)
            else:
                last.extend(tail)
        for k, plist in enumerate(groups):
            total = sum(p.numel() for p in plist)
            flat = torch.zeros(total, dtype=plist[0].dtype, device=plist[0].device)
            offset = 0
            for p in plist:
                p.grad = flat[offset:offset + p.numel()].view_as(p)
                offset += p.numel()
                self._bucket_of[p] = k
            done = torch.cuda.Event() if flat.is_cuda else None     # recorded after the bucket's all-reduce
            self.buckets.append({"flat": flat, "params": plist, "ready": 0, "done": done})

    # ---- per-step ----------------------------------------------------------------------------
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def zero_grad(self, set_to_none=False):
        """Zero the flat buffers; gradients stay views into them (never set to None)."""
        for b in self.buckets:
            b["flat"].zero_()
            b["ready"] = 0
        self._next_bucket = 0

    def _on_grad_ready(self, param):
        k = self._bucket_of[param]
        b = self.buckets[k]
        if param.grad.data_ptr() != b["flat"].data_ptr() + self._offset_bytes(param, b):
            # something replaced .grad (e.g. zero_grad(set_to_none=True)): copy back into the view
            view = self._view_of(param, b)
            view.copy_(param.grad)
            param.grad = view
        b["ready"] += 1
        if not self._callback_queued:
            torch.autograd.Variable._execution_engine.queue_callback(self.finish)
            self._callback_queued = True
        self._reduce_complete_prefix()

    def _reduce_complete_prefix(self):
        """Issue, in bucket order, the reductions of the leading buckets that are complete."""
        while self._next_bucket < len(self.buckets):
            b = self.buckets[self._next_bucket]
            if b["ready"] < len(b["params"]):
                break
            self._reduce_bucket(self._next_bucket)
            self._next_bucket += 1

    def _offset_bytes(self, param, b):
        off = 0
        for p in b["params"]:
            if p is param:
                return off * b["flat"].element_size()
            off += p.numel()
        raise KeyError("parameter not in bucket")

    def _view_of(self, param, b):
        off = self._offset_bytes(param, b) // b["flat"].element_size()
        return b["flat"][off:off + param.numel()].view_as(param)

    def _reduce_bucket(self, k):
        flat = self.buckets[k]["flat"]
        if self.world_size == 1 or not self.communicate:
            return
        if flat.is_cuda and self.overlap:
            compute = torch.cuda.current_stream(flat.device)
            events = None
            if self.trace is not None:       # eager steps only: events cannot be timed inside a captured graph
                events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                events[0].record(compute)    # the bucket's last gradient exists
            self._comm_stream.wait_stream(compute)
            with torch.cuda.stream(self._comm_stream):
                if events is not None:
                    events[1].record(self._comm_stream)
                self._all_reduce_mean(flat)
                if events is not None:
                    events[2].record(self._comm_stream)
                    self.trace.append((k, events))
                self.buckets[k]["done"].record(self._comm_stream)
            self._pending.append(k)
        else:
            self._all_reduce_mean(flat)

    def _all_reduce_mean(self, flat):
        if _capi.NVTX and flat.is_cuda:
            torch.cuda.nvtx.range_push("snn.ddp.allreduce %d bytes" % (flat.numel() * flat.element_size()))
            try:
                self._all_reduce_mean_impl(flat)
            finally:
                torch.cuda.nvtx.range_pop()
        else:
            self._all_reduce_mean_impl(flat)

    def _all_reduce_mean_impl(self, flat):
        if self._avg_op is not None:
            dist.all_reduce(flat, op=self._avg_op, group=self.group)
        else:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
            flat.mul_(1.0 / self.world_size)

    def finish(self):
        """Join the side stream; gradients are averaged once work queued after this runs."""
        self._callback_queued = False
        # whatever has not been reduced yet (a parameter, or a whole bucket, took no part in this
        # backward on this rank): reduce it now, in order, so the collective sequence is the same
        # on every rank
        while self._next_bucket < len(self.buckets):
            self._reduce_bucket(self._next_bucket)
            self._next_bucket += 1
        for b in self.buckets:
            b["ready"] = 0
        self._next_bucket = 0
        if self._pending and not self.defer_wait:
            flat = self.buckets[self._pending[0]]["flat"]
            torch.cuda.current_stream(flat.device).wait_stream(self._comm_stream)
            self._pending.clear()

    def wait_bucket(self, k):
        """Make the current stream wait for bucket k's all-reduce of this backward (a no-op when
        that reduction ran inline). Only needed with ``defer_wait=True``."""
        if k in self._pending:
            torch.cuda.current_stream(self.buckets[k]["flat"].device).wait_event(self.buckets[k]["done"])
            self._pending.remove(k)

    def bucket_sizes(self):
        return [b["flat"].numel() for b in self.buckets]


class BucketSGD:
    """``torch.optim.SGD`` with momentum that does not wait for the LAST all-reduce before it starts:
    the parameters of all buckets but the last are updated first (after waiting for their reductions
    only), then the last bucket's - the first layers, whose all-reduce cannot start before backward
    ends and so cannot hide behind backward; it hides behind the first update instead. Two
    ``torch.optim.SGD`` instances do the arithmetic, so the trajectory is that of the reference's
    ``optim.SGD(..., momentum=0.9)`` (snnlib/example/train_test_cifar.py:36). Build the wrapper
    with ``defer_wait=True``."""

    def __init__(self, ddp, lr=1e-2, momentum=0.9):
        self.ddp = ddp
        n = len(ddp.buckets)
        cut = n - 1 if n > 1 else n
        self.groups = []                 # (index of the last bucket to wait for, optimizer of those buckets)
        for lo, hi in ((0, cut), (cut, n)):
            params = [p for b in ddp.buckets[lo:hi] for p in b["params"]]
            if params:
                self.groups.append((hi - 1, torch.optim.SGD(params, lr=lr, momentum=momentum)))

    def zero_grad(self, set_to_none=False):
        self.ddp.zero_grad()

    def step(self):
        done = 0
        for last, opt in self.groups:
            for k in range(done, last + 1):
                self.ddp.wait_bucket(k)
            done = last + 1
            opt.step()

    def state_dict(self):
        return {"groups": [opt.state_dict() for _, opt in self.groups]}

    def load_state_dict(self, state):
        for (_, opt), saved in zip(self.groups, state["groups"]):
            opt.load_state_dict(saved)
