"""Triadic GDN behind torch.library custom ops, so that torch.compile records one opaque node per call.

Mirrors cute_triadic_gdn/ops/joint_torch_ops.py:8-95 of the reference: one forward op that returns the output and the
tensors the backward needs, one backward op, fake (meta) implementations, autograd registration with a single read of
the saved tensors and without materialising zero gradients for the auxiliary outputs, and `gdn_joint_call`.
The ops live in the namespace `tgdn_b200` so that both packages can be imported into one process.
"""
from __future__ import annotations

import torch
from torch.library import custom_op, register_autograd

from .gdn_joint import (CHUNK, _check, _check_device_and_e, _kernel_backward, _kernel_forward, _save_list, _unpack_saved)


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
    return [torch.empty_like(v), g.new_empty(B, NC, H, CHUNK, E), q.new_empty(B, NC, H, 128 * 64),
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


def _setup(ctx, inputs, output):
    q, k, v, k2, q2, g, beta, scale, chunk_starts, token_map = inputs
    _, gc, AP, Pm, h, W, U = output
    ctx.save_for_backward(*_save_list(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map))
    ctx.scale = scale
    ctx.mark_non_differentiable(*output[1:])
    # without this autograd materialises a zero gradient for every auxiliary output on each backward
    ctx.set_materialize_grads(False)


def _backward(ctx, grads):
    if grads[0] is None:
        return (None,) * len(ctx.needs_input_grad)
    # one read of saved_tensors: activation checkpointing (use_reentrant=False) unpacks each saved tensor exactly once
    saved = ctx.saved_tensors
    dq, dk, dv, dk2, dq2, dg, db = joint_bwd(list(saved[:-2]), grads[0].contiguous(), ctx.scale, saved[-2], saved[-1])
    return (dq, dk, dv, dk2, dq2, dg, db, None, None, None)[:len(ctx.needs_input_grad)]


register_autograd("tgdn_b200::joint_fwd", _backward, setup_context=_setup)


def gdn_joint_call(q, k, v, k2, q2, g, beta, scale=None, cu_seqlens=None):
    """Traceable Triadic GDN for training; sm_100, E=1/2/4/8/12/16, head dim 128.

    Same inputs and packed-document contract as `chunk_gdn_joint`.  Inputs are made contiguous here; document metadata
    is built on the device; inputs and outputs are not repacked.
    """
    q, k, v, k2, q2, g, beta = (t.contiguous() for t in (q, k, v, k2, q2, g, beta))
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    chunk_starts = token_map = None
    if cu_seqlens is not None:
        from .joint_packing import prepare_documents
        chunk_starts, token_map = prepare_documents((q, k, v, k2, q2, g, beta), cu_seqlens)
    return joint_fwd(q, k, v, k2, q2, g, beta, scale, chunk_starts, token_map)[0]
