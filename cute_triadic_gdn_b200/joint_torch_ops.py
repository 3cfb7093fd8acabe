"""Triadic GDN behind torch.library custom ops, so that torch.compile records one opaque node per call.

Mirrors cute_triadic_gdn/ops/joint_torch_ops.py:8-95 of the reference: one forward op that returns the output and the
tensors the backward needs, one backward op, fake (meta) implementations, autograd registration with a single read of
the saved tensors and without materialising zero gradients for the auxiliary outputs, and `gdn_joint_call`.
The ops live in the namespace `tgdn_b200` so that both packages can be imported into one process.
"""
from __future__ import annotations

import torch
from torch.library import custom_op, register_autograd

from .gdn_joint import (CHUNK, gate_item_floats, _check, _check_device_and_e, _kernel_backward, _kernel_forward, _save_list, _unpack_saved)


@custom_op("tgdn_b200::joint_fwd", mutates_args=(), device_types="cuda")
def joint_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k2: torch.Tensor, q2: torch.Tensor, g: torch.Tensor,
              beta: torch.Tensor, scale: float, chunk_starts: torch.Tensor | None = None,
              token_map: torch.Tensor | None = None) -> list[torch.Tensor]:
    _check(q, k, v, k2, q2, g, beta, packed=token_map is not None)
    _check_device_and_e(q, k2.shape[-1])
    o, gc, AP, Pm, h, W, U = _kernel_forward(q, k, v, k2, q2, g, beta, scale, True, chunk_starts, token_map)
    return [o, gc, AP, Pm, h, W, U]


@joint_fwd.register_fake
def _joint_fwd_fake(q, k, v, k2, q2, g, beta, scale, chunk_starts=None, token_map=None):
    B, T, H, D = q.shape
    E = k2.shape[-1]
    NC = token_map.shape[1] if token_map is not None else T // CHUNK
    return [torch.empty_like(v), g.new_empty(B, NC, H, gate_item_floats(E)), q.new_empty(B, NC, H, 128 * 64),
            q.new_empty(B, NC, H, 64 * 64), q.new_empty(B, NC, H, E, 16, 128, 8), v.new_empty(B, NC, H, CHUNK, 128),
            v.new_empty(B, NC, H, CHUNK, 128)]


@custom_op("tgdn_b200::joint_bwd", mutates_args=(), device_types="cuda")
def joint_bwd(saved: list[torch.Tensor], do: torch.Tensor, scale: float, chunk_starts: torch.Tensor | None = None,
              token_map: torch.Tensor | None = None) -> list[torch.Tensor]:
    q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, _, _ = _unpack_saved(tuple(t.detach() for t in saved) + (None, None))
    return list(_kernel_backward(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, do.contiguous(), scale, chunk_starts,
                                 token_map))


@joint_bwd.register_fake
def _joint_bwd_fake(saved, do, scale, chunk_starts=None, token_map=None):
    q, k, k2, q2, g, beta = saved[:6]
    return [torch.empty_like(q), torch.empty_like(k), torch.empty_like(do), torch.empty_like(k2), torch.empty_like(q2),
            torch.empty_like(g), torch.empty_like(beta)]


def _remember(ctx, inputs, output):
    """Keeps what the backward op reads.  The op returns the output first and its intermediates after it; those are not
    differentiable, and autograd is told not to conjure zero gradients for them (each would be a tensor as large as the
    intermediate itself, on every backward)."""
    *seven, scale, chunk_starts, token_map = inputs
    q, k, _, k2, q2, g, beta = seven
    o, *aux = output
    gc, AP, Pm, h, W, U = aux
    ctx.save_for_backward(*_save_list(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map))
    ctx.scale = scale
    ctx.mark_non_differentiable(*aux)
    ctx.set_materialize_grads(False)


def _differentiate(ctx, grads):
    n_inputs = len(ctx.needs_input_grad)
    do = grads[0]
    if do is None:                                   # the output was not used
        return (None,) * n_inputs
    # ctx.saved_tensors is read exactly once: under activation checkpointing (use_reentrant=False) every read unpacks, and a
    # second one would re-run the forward
    kept = ctx.saved_tensors
    *tensors, chunk_starts, token_map = kept
    seven = joint_bwd(list(tensors), do.contiguous(), ctx.scale, chunk_starts, token_map)
    return (*seven, *([None] * (n_inputs - 7)))


register_autograd("tgdn_b200::joint_fwd", _differentiate, setup_context=_remember)


def gdn_joint_call(q, k, v, k2, q2, g, beta, scale=None, cu_seqlens=None):
    """Triadic GDN for training, as ONE custom-op node (so that torch.compile does not look inside): same arguments and
    packed-row rules as `chunk_gdn_joint`.  Unlike that function this one accepts non-contiguous inputs (it makes them
    contiguous), like the reference's entry of the same name (ops/joint_torch_ops.py:83-95).  sm_100 only,
    E in {1, 2, 4, 8, 12, 16}, head dimension 128."""
    seven = [t.contiguous() for t in (q, k, v, k2, q2, g, beta)]
    if scale is None:
        scale = seven[0].shape[-1] ** -0.5
    chunk_starts = token_map = None
    if cu_seqlens is not None:
        from .joint_packing import prepare_documents
        chunk_starts, token_map = prepare_documents(seven, cu_seqlens)
    return joint_fwd(*seven, float(scale), chunk_starts, token_map)[0]
