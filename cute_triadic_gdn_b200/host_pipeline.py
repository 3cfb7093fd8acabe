"""Host-resident entry point: inputs and results live in pinned host memory, transfers overlap the kernels.

The sequences of a batch are independent in the Triadic GDN core (cute_triadic_gdn/ops/gdn_joint.py:45-90 loops over
the batch rows; the kernels here run one CTA chain per (batch row, head)), so the batch is cut into slices and pushed
through a three-stage pipeline on three CUDA streams:

    upload slice i+1   |   forward (+ backward) of slice i   |   download slice i-1

With PCIe carrying both directions at once, a step costs about max(upload, compute, download) instead of their sum.
The results are bitwise those of one `gdn_joint_call` over the whole batch.  A packed row (`cu_seqlens`) is cut the
same way along its documents, which are just as independent: token-balanced ranges of whole documents
(`sharding.document_ranges`), each run with its own re-based offsets.
"""
from __future__ import annotations

import os

import torch

from .joint_torch_ops import gdn_joint_call
from .sharding import document_ranges

_NAMES = ("q", "k", "v", "k2", "q2", "g", "beta")


def bind_host_to_gpu(device_index):
    """Pins the calling process to the CPU cores of the NUMA node its GPU hangs off, so that pinned buffers allocated
    afterwards (first touch) and the copy engine's reads stay on that node.  One rank per GPU calls this before it
    allocates its pinned tensors.  Returns what it found and did: {"bdf", "numa_node", "cpus", "bound"}; a host without
    that information in sysfs (numa_node -1, containers) is left as it is."""
    info = {"bdf": None, "numa_node": None, "cpus": None, "bound": False}
    try:
        pr = torch.cuda.get_device_properties(device_index)
        info["bdf"] = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{info['bdf']}/numa_node") as fh:
            node = int(fh.read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            text = fh.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        info["cpus"] = text
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"] = True
    except (OSError, ValueError, AttributeError, RuntimeError):
        pass
    return info


def _check_host(t, name):
    if t.device.type != "cpu":
        raise ValueError(f"{name} must be a host tensor")
    if not t.is_pinned():
        raise ValueError(f"{name} must be in pinned host memory (tensor.pin_memory())")


class HostPipeline:
    """Reusable buffers and streams for `run`; build once per shape, call every step.

    `inputs` are the seven host tensors (q, k, v, k2, q2, g, beta) in the layouts `gdn_joint_call` takes; `do` is the
    upstream gradient (None: forward only).  Dense rows: `slices` must divide the batch.  Packed row: `cu_seqlens` (host
    or device offsets) and `slices` = number of document ranges (empty ranges are dropped).
    """

    def __init__(self, inputs, do=None, *, scale=None, slices=None, device=None, cu_seqlens=None):
        if len(inputs) != 7:
            raise ValueError("expected (q, k, v, k2, q2, g, beta)")
        for t, n in zip(inputs, _NAMES):
            _check_host(t, n)
        if do is not None:
            _check_host(do, "do")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        B = inputs[0].shape[0]
        if cu_seqlens is None:
            self.slices = B if slices is None else int(slices)
            if self.slices < 1 or B % self.slices:
                raise ValueError(f"slices={self.slices} must divide the batch {B}")
            self.rows = B // self.slices
            # (first, one past last) along the batch axis, offsets on the device (none: dense rows)
            self.parts = [(i * self.rows, (i + 1) * self.rows, None) for i in range(self.slices)]
            self.axis = 0
        else:
            if B != 1:
                raise ValueError("packed rows have batch size 1")
            cu = cu_seqlens.detach().cpu()
            ranges = [r for r in document_ranges(cu, 1 if slices is None else int(slices)) if r.doc_hi > r.doc_lo]
            self.slices = len(ranges)
            self.rows = max(r.tok_hi - r.tok_lo for r in ranges)       # device buffers hold the longest part
            self.parts = [(r.tok_lo, r.tok_hi, (cu[r.doc_lo:r.doc_hi + 1] - cu[r.doc_lo]).to(torch.int32).to(self.device))
                          for r in ranges]
            self.axis = 1
        self.scale = scale
        self.backward = do is not None
        dev = self.device
        # two device-side input sets (upload of slice i+1 overlaps the kernels of slice i)
        shape = (lambda t: (self.rows,) + tuple(t.shape[1:])) if self.axis == 0 else \
            (lambda t: (1, self.rows) + tuple(t.shape[2:]))
        self._in = [[torch.empty(shape(t), dtype=t.dtype, device=dev) for t in inputs] for _ in range(2)]
        self._do = [torch.empty(shape(do), dtype=do.dtype, device=dev) for _ in range(2)] if self.backward else None
        self.up, self.down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.o_host = torch.empty(tuple(inputs[2].shape), dtype=inputs[2].dtype, pin_memory=True)
        self.grads_host = [torch.empty(tuple(t.shape), dtype=t.dtype, pin_memory=True) for t in inputs] \
            if self.backward else None
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in inputs) + \
            (do.numel() * do.element_size() if self.backward else 0)
        self.d2h_bytes = self.o_host.numel() * self.o_host.element_size() + \
            (sum(t.numel() * t.element_size() for t in self.grads_host) if self.backward else 0)

    def run(self, inputs, do=None):
        """One step.  Returns (o_host, grads_host or None), pinned host buffers that the next call reuses.

        The call only ENQUEUES work: when it returns, the downloads into the returned buffers may still be running on the
        pipeline's own stream.  torch's current stream is made to wait for them, so later GPU work is ordered correctly,
        but the CPU must call `wait()` (or synchronise the current stream) before it reads the returned tensors, and
        must be done with them before it calls `run` again."""
        if (do is not None) != self.backward:
            raise ValueError("`do` must be given exactly when the pipeline was built with one")
        dev = self.device
        compute = torch.cuda.current_stream(dev)
        uploaded = [None, None]      # event: input set s holds the slice
        consumed = [None, None]      # event: the kernels that read input set s are done
        start = torch.cuda.Event()
        start.record(compute)
        self.up.wait_event(start)    # do not start uploading over buffers an earlier step may still read
        self.down.wait_event(start)
        for i, (lo, hi, cu_dev) in enumerate(self.parts):
            s = i & 1
            n = hi - lo
            cut = (lambda t: t[lo:hi]) if self.axis == 0 else (lambda t: t[:, lo:hi])        # of a host tensor
            head = (lambda t: t[:n]) if self.axis == 0 else (lambda t: t[:, :n])            # of a device buffer
            with torch.cuda.stream(self.up):
                if consumed[s] is not None:
                    self.up.wait_event(consumed[s])
                for dst, src in zip(self._in[s], inputs):
                    head(dst).copy_(cut(src), non_blocking=True)
                if self.backward:
                    head(self._do[s]).copy_(cut(do), non_blocking=True)
                uploaded[s] = torch.cuda.Event()
                uploaded[s].record(self.up)
            compute.wait_event(uploaded[s])
            leaves = [head(t).detach().requires_grad_(self.backward) for t in self._in[s]]
            o = gdn_joint_call(*leaves, scale=self.scale, cu_seqlens=cu_dev)
            outs = [o.detach()]
            if self.backward:
                o.backward(head(self._do[s]))
                outs += [t.grad for t in leaves]
            consumed[s] = torch.cuda.Event()
            consumed[s].record(compute)
            for t in outs:
                t.record_stream(self.down)               # keep the allocator from reusing it before the download ran
            with torch.cuda.stream(self.down):
                self.down.wait_event(consumed[s])
                cut(self.o_host).copy_(outs[0], non_blocking=True)
                if self.backward:
                    for hbuf, t in zip(self.grads_host, outs[1:]):
                        cut(hbuf).copy_(t, non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.down)
        compute.wait_event(done)     # the step is complete, in stream order, when the last download is
        self._done = done
        return self.o_host, self.grads_host

    def wait(self):
        """Blocks the calling CPU thread until the results of the last `run` are in the host buffers."""
        done = getattr(self, "_done", None)
        if done is not None:
            done.synchronize()


def gdn_joint_host(q, k, v, k2, q2, g, beta, do=None, *, scale=None, slices=None, device=None, cu_seqlens=None):
    """One-shot convenience wrapper around `HostPipeline` (allocates its buffers on every call)."""
    pipe = HostPipeline((q, k, v, k2, q2, g, beta), do, scale=scale, slices=slices, device=device, cu_seqlens=cu_seqlens)
    o, grads = pipe.run((q, k, v, k2, q2, g, beta), do)
    pipe.wait()
    return o, grads
