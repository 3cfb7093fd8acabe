"""Context parallelism: ONE set of long sequences split along the token axis over the ranks of a process group.

Rank r holds tokens [r*T/N, (r+1)*T/N) of every sequence.  The recurrence is serial in the token axis, so rank r needs the
state S after rank r-1's last token (f32, E*64 KB per head and sequence) and, in the backward, rank r-1 needs dL/dS from
rank r.  To keep every GPU busy the heads are cut into `head_groups` groups that travel as a wavefront: rank r works on
group j while rank r+1 works on group j-1, so that a step takes (N - 1 + G) / G segment times instead of N.
The hand-off is a point-to-point send / receive per group and boundary (NCCL over NVLink between GPUs; any backend of
torch.distributed works, the CPU tests use gloo); there is no collective.

The per-segment operator is `chunk_gdn_joint_segment` (state in, state out, differentiable through both); the exchange is
expressed as autograd functions, so `loss.backward()` runs the reverse wavefront by itself.  The reference has no such
path: its sequences live on one GPU (cute_triadic_gdn/ops/gdn_joint.py:252-278).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _RecvState(torch.autograd.Function):
    """Forward: receive the state from the previous rank.  Backward: send its gradient back there."""

    @staticmethod
    def forward(ctx, anchor, shape, dtype, device, src, group, tag):
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, src=src, group=group, tag=tag)
        ctx.src, ctx.group, ctx.tag, ctx.meta = src, group, tag, (shape, dtype, device)
        return buf

    @staticmethod
    def backward(ctx, grad):
        if grad is None:                                   # the segment did not use its incoming state
            shape, dtype, device = ctx.meta
            grad = torch.zeros(shape, dtype=dtype, device=device)
        dist.send(grad.contiguous(), dst=ctx.src, group=ctx.group, tag=ctx.tag)
        return (None,) * 7


class _SendState(torch.autograd.Function):
    """Forward: send the state to the next rank.  Backward: receive its gradient from there.  Returns a scalar zero that the
    caller adds to its output so that the exchange stays in the autograd graph."""

    @staticmethod
    def forward(ctx, state, dst, group, tag):
        dist.send(state.contiguous(), dst=dst, group=group, tag=tag)
        ctx.dst, ctx.group, ctx.tag = dst, group, tag
        ctx.meta = (tuple(state.shape), state.dtype, state.device)
        return state.new_zeros(())

    @staticmethod
    def backward(ctx, _):
        shape, dtype, device = ctx.meta
        grad = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(grad, src=ctx.dst, group=ctx.group, tag=ctx.tag)
        return grad, None, None, None


def head_groups_of(H, groups):
    """Contiguous head ranges [(lo, hi), ...] of near-equal size; at most H groups."""
    groups = max(1, min(int(groups), H))
    cuts = [round(i * H / groups) for i in range(groups + 1)]
    return [(lo, hi) for lo, hi in zip(cuts[:-1], cuts[1:]) if hi > lo]


def context_parallel_joint(q, k, v, k2, q2, g, beta, *, group=None, head_groups=1, scale=None, segment_fn=None,
                           state_dtype=torch.float32):
    """This rank's token slice of every sequence through the Triadic GDN core; returns o for the same slice.

    q, k, v: (B, T_local, H, 128); k2, q2, g: (B, T_local, H, E); beta: (B, T_local, H), with T_local a multiple of 64 and
    rank r of `group` holding the r-th slice.  Differentiable: the backward sends the state gradients the other way.
    `segment_fn(q, k, v, k2, q2, g, beta, state_in, scale) -> (o, state_out)` is the per-segment operator (default: the
    kernels, `chunk_gdn_joint_segment`, whose states are f32; another operator says what its states are with `state_dtype`)."""
    if segment_fn is None:
        from .gdn_joint import chunk_gdn_joint_segment
        segment_fn = lambda *a: chunk_gdn_joint_segment(*a[:7], state_in=a[7], scale=a[8])
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    B, T, H, D = q.shape
    E = k2.shape[-1]
    outs, anchors = [], []
    for j, (lo, hi) in enumerate(head_groups_of(H, head_groups)):
        cut = lambda t: t[:, :, lo:hi].contiguous()
        state_in = None
        if rank > 0:
            state_in = _RecvState.apply(q.new_zeros((), dtype=torch.float32).requires_grad_(torch.is_grad_enabled()),
                                        (B, hi - lo, E, D, D), state_dtype, q.device, to_global(rank - 1), group, j)
        o, state_out = segment_fn(cut(q), cut(k), cut(v), cut(k2), cut(q2), cut(g), cut(beta), state_in, scale)
        if rank + 1 < world:
            anchors.append(_SendState.apply(state_out, to_global(rank + 1), group, j))
        outs.append(o)
    o = torch.cat(outs, dim=2)
    for a in anchors:                  # zero-valued: keeps the sends (and the receives of their gradients) in the graph
        o = o + a.to(o.dtype)
    return o
