"""Host-resident entry point: inputs and results live in pinned host memory, transfers overlap the kernels.

The sequences of a batch are independent in the Triadic GDN core (cute_triadic_gdn/ops/gdn_joint.py:45-90 loops over
the batch rows; the kernels here run one CTA chain per (batch row, head)), so the batch is cut into slices and pushed
through a three-stage pipeline on three CUDA streams:

    upload slice i+1   |   forward (+ backward) of slice i   |   download slice i-1

With PCIe carrying both directions at once, a step costs about max(upload, compute, download) instead of their sum.
The results are bitwise those of one `gdn_joint_call` over the whole batch.
"""
from __future__ import annotations

import torch

from .joint_torch_ops import gdn_joint_call

_NAMES = ("q", "k", "v", "k2", "q2", "g", "beta")


def _check_host(t, name):
    if t.device.type != "cpu":
        raise ValueError(f"{name} must be a host tensor")
    if not t.is_pinned():
        raise ValueError(f"{name} must be in pinned host memory (tensor.pin_memory())")


class HostPipeline:
    """Reusable buffers and streams for `run`; build once per shape, call every step.

    `inputs` are the seven host tensors (q, k, v, k2, q2, g, beta) in the layouts `gdn_joint_call` takes; `do` is the
    upstream gradient (None: forward only).  `slices` must divide the batch.
    """

    def __init__(self, inputs, do=None, *, scale=None, slices=None, device=None):
        if len(inputs) != 7:
            raise ValueError("expected (q, k, v, k2, q2, g, beta)")
        for t, n in zip(inputs, _NAMES):
            _check_host(t, n)
        if do is not None:
            _check_host(do, "do")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        B = inputs[0].shape[0]
        self.slices = B if slices is None else int(slices)
        if self.slices < 1 or B % self.slices:
            raise ValueError(f"slices={self.slices} must divide the batch {B}")
        self.rows = B // self.slices
        self.scale = scale
        self.backward = do is not None
        dev = self.device
        # two device-side input sets (upload of slice i+1 overlaps the kernels of slice i)
        self._in = [[torch.empty((self.rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for t in inputs]
                    for _ in range(2)]
        self._do = [torch.empty((self.rows,) + tuple(do.shape[1:]), dtype=do.dtype, device=dev) for _ in range(2)] \
            if self.backward else None
        self.up, self.down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.o_host = torch.empty(tuple(inputs[2].shape), dtype=inputs[2].dtype, pin_memory=True)
        self.grads_host = [torch.empty(tuple(t.shape), dtype=t.dtype, pin_memory=True) for t in inputs] \
            if self.backward else None
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in inputs) + \
            (do.numel() * do.element_size() if self.backward else 0)
        self.d2h_bytes = self.o_host.numel() * self.o_host.element_size() + \
            (sum(t.numel() * t.element_size() for t in self.grads_host) if self.backward else 0)

    def run(self, inputs, do=None):
        """One step.  Returns (o_host, grads_host or None); the host buffers are reused by the next call."""
        if (do is not None) != self.backward:
            raise ValueError("`do` must be given exactly when the pipeline was built with one")
        dev, rows = self.device, self.rows
        compute = torch.cuda.current_stream(dev)
        uploaded = [None, None]      # event: input set s holds the slice
        consumed = [None, None]      # event: the kernels that read input set s are done
        start = torch.cuda.Event()
        start.record(compute)
        self.up.wait_event(start)    # do not start uploading over buffers an earlier step may still read
        self.down.wait_event(start)
        for i in range(self.slices):
            s = i & 1
            lo, hi = i * rows, (i + 1) * rows
            with torch.cuda.stream(self.up):
                if consumed[s] is not None:
                    self.up.wait_event(consumed[s])
                for dst, src in zip(self._in[s], inputs):
                    dst.copy_(src[lo:hi], non_blocking=True)
                if self.backward:
                    self._do[s].copy_(do[lo:hi], non_blocking=True)
                uploaded[s] = torch.cuda.Event()
                uploaded[s].record(self.up)
            compute.wait_event(uploaded[s])
            leaves = [t.detach().requires_grad_(self.backward) for t in self._in[s]]
            o = gdn_joint_call(*leaves, scale=self.scale)
            outs = [o.detach()]
            if self.backward:
                o.backward(self._do[s])
                outs += [t.grad for t in leaves]
            consumed[s] = torch.cuda.Event()
            consumed[s].record(compute)
            for t in outs:
                t.record_stream(self.down)               # keep the allocator from reusing it before the download ran
            with torch.cuda.stream(self.down):
                self.down.wait_event(consumed[s])
                self.o_host[lo:hi].copy_(outs[0], non_blocking=True)
                if self.backward:
                    for hbuf, t in zip(self.grads_host, outs[1:]):
                        hbuf[lo:hi].copy_(t, non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.down)
        compute.wait_event(done)     # the step is complete, in stream order, when the last download is
        return self.o_host, self.grads_host


def gdn_joint_host(q, k, v, k2, q2, g, beta, do=None, *, scale=None, slices=None, device=None):
    """One-shot convenience wrapper around `HostPipeline` (allocates its buffers on every call)."""
    pipe = HostPipeline((q, k, v, k2, q2, g, beta), do, scale=scale, slices=slices, device=device)
    o, grads = pipe.run((q, k, v, k2, q2, g, beta), do)
    torch.cuda.current_stream(pipe.device).synchronize()
    return o, grads
