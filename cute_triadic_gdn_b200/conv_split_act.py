"""Causal depthwise short convolution whose leading channels get SiLU: `conv_split_act_call`.

Same call, shapes, dtypes and packed-row semantics as the reference's cute_triadic_gdn/ops/conv_split_act.py:194-197
(conv_split_act_call) with its custom ops :143-173 and autograd glue :176-191; the device work is the CUDA library's
tgdn_conv_fwd / tgdn_conv_bwd instead of Triton kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch.library import custom_op, register_autograd

from . import _lib


def _prep(x, weight, cu_seqlens):
    """Argument checks and the layout the kernels need: bf16, unit channel stride, 16-byte aligned rows, and a channel count
    that is a multiple of 8 (a TMA row is a multiple of 16 bytes).  Other channel counts and other weight dtypes, which
    the reference's Triton kernels take as they are (cute_triadic_gdn/ops/conv_split_act.py:133-140), are served through a
    zero-padded copy and a cast; `pad` is the number of channels added."""
    if x.ndim != 3 or weight.ndim != 2 or weight.shape[0] != x.shape[2] or weight.shape[1] != 4:
        raise ValueError("x must be (B, T, C) and weight (C, 4)")
    if x.dtype != torch.bfloat16:
        raise ValueError("x must be bf16")
    if not x.is_cuda or weight.device != x.device:
        raise ValueError("x and weight must be on the same CUDA device")
    pad = (-x.shape[2]) % 8
    weight = weight.to(torch.bfloat16)
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
        weight = torch.nn.functional.pad(weight, (0, 0, 0, pad))
    if x.stride(2) != 1 or x.stride(1) % 8 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    n_docs = 0
    if cu_seqlens is not None:
        if x.shape[0] != 1:
            raise ValueError("cu_seqlens requires a packed row: B=1")
        if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2 or cu_seqlens.device != x.device:
            raise ValueError("cu_seqlens must be a vector of at least two offsets on the input device")
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
        n_docs = cu_seqlens.numel() - 1
    return x, weight.contiguous(), cu_seqlens, n_docs, pad


@custom_op("tgdn_b200::conv_split_act_fwd", mutates_args=(), device_types="cuda")
def conv_split_act_fwd(x: torch.Tensor, weight: torch.Tensor, act_channels: int,
                       cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    x, weight, cu, n_docs, pad = _prep(x, weight, cu_seqlens)
    B, T, C = x.shape
    y = torch.empty((B, T, C), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.tgdn_conv_fwd(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(cu), n_docs, B, T, C,
                                          x.stride(0), x.stride(1), int(act_channels), _lib.stream_of(x)),
                   "tgdn_conv_fwd")
    return y[..., :C - pad].contiguous() if pad else y


@conv_split_act_fwd.register_fake
def _(x, weight, act_channels, cu_seqlens=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@custom_op("tgdn_b200::conv_split_act_bwd", mutates_args=(), device_types="cuda")
def conv_split_act_bwd(x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor, act_channels: int,
                       cu_seqlens: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    wdtype = weight.dtype
    x, weight, cu, n_docs, pad = _prep(x, weight, cu_seqlens)
    if pad:
        dy = torch.nn.functional.pad(dy, (0, pad))
    if dy.stride(2) != 1 or dy.stride(1) % 8 or dy.stride(0) % 8 or dy.data_ptr() % 16:
        dy = dy.contiguous()
    B, T, C = x.shape
    dx = torch.empty((B, T, C), dtype=x.dtype, device=x.device)
    dw = torch.empty_like(weight)
    nbytes = _lib.lib.tgdn_conv_bwd_scratch_bytes(B, T, C)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.tgdn_conv_bwd(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(dy), _lib.ptr(dx), _lib.ptr(dw),
                                          _lib.ptr(cu), n_docs, B, T, C, x.stride(0), x.stride(1), dy.stride(0),
                                          dy.stride(1), int(act_channels), _lib.ptr(scratch), nbytes,
                                          _lib.stream_of(x)), "tgdn_conv_bwd")
    if pad:
        dx, dw = dx[..., :C - pad].contiguous(), dw[:C - pad].contiguous()
    return dx, dw.to(wdtype)


@conv_split_act_bwd.register_fake
def _(x, dy, weight, act_channels, cu_seqlens=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight)


def _remember(ctx, inputs, output):
    """What the backward needs: the input, the taps and (for a packed row) the document offsets."""
    x, weight, act_channels, cu_seqlens = inputs
    keep = [x, weight] + ([] if cu_seqlens is None else [cu_seqlens])
    ctx.save_for_backward(*keep)
    ctx.act_channels = int(act_channels)


def _differentiate(ctx, dy):
    kept = ctx.saved_tensors                      # read once (activation checkpointing unpacks on every read)
    offsets = kept[2] if len(kept) == 3 else None
    dx, dw = conv_split_act_bwd(kept[0], dy, kept[1], ctx.act_channels, offsets)
    return dx, dw, None, None


register_autograd("tgdn_b200::conv_split_act_fwd", _differentiate, setup_context=_remember)


def conv_split_act_call(x, weight, act_channels, cu_seqlens=None):
    """Width-4 causal depthwise convolution over (B, T, C) bf16 `x` with taps `weight` (C, 4); the first `act_channels`
    channels pass through SiLU.  With `cu_seqlens` (offsets of the documents of one packed row, B = 1) the window starts
    afresh at every document.  Same call as the reference's conv_split_act_call (ops/conv_split_act.py:194-197)."""
    return conv_split_act_fwd(x, weight.contiguous(), int(act_channels), cu_seqlens)


# ----------------------------------------------------------------------------------------------------------------------
# The layer glue fused into the convolution (beyond the reference's surface; it describes the glue at
# cute_triadic_gdn/ops/conv_split_act.py:3-5 and leaves it to its caller)
# ----------------------------------------------------------------------------------------------------------------------
def _glue_dims(x, H, E):
    C = x.shape[2]
    if H <= 0 or C != H * (3 * 128 + 2 * E) or E not in (1, 2, 4, 8, 12, 16):
        raise ValueError(f"conv_split_norm: C={C} is not H*(3*128 + 2*E) for H={H}, E={E} (E in 1, 2, 4, 8, 12, 16)")
    if C % 8:
        raise ValueError("conv_split_norm: the channel count must be a multiple of 8")


@custom_op("tgdn_b200::conv_split_norm_fwd", mutates_args=(), device_types="cuda")
def conv_split_norm_fwd(x: torch.Tensor, weight: torch.Tensor, heads: int, slices: int, eps: float,
                        cu_seqlens: Optional[torch.Tensor] = None
                        ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _glue_dims(x, heads, slices)
    x, weight, cu, n_docs, _ = _prep(x, weight, cu_seqlens)
    B, T, C = x.shape
    q, k, v = (torch.empty((B, T, heads, 128), dtype=torch.bfloat16, device=x.device) for _ in range(3))
    k2, q2 = (torch.empty((B, T, heads, slices), dtype=torch.float32, device=x.device) for _ in range(2))
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.tgdn_glue_fwd(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(cu), n_docs, B, T, C, x.stride(0),
                                          x.stride(1), heads, slices, float(eps), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v),
                                          _lib.ptr(k2), _lib.ptr(q2), _lib.stream_of(x)), "tgdn_glue_fwd")
    return q, k, v, k2, q2


@conv_split_norm_fwd.register_fake
def _(x, weight, heads, slices, eps, cu_seqlens=None):
    B, T, _ = x.shape
    qkv = [x.new_empty((B, T, heads, 128)) for _ in range(3)]
    gates = [x.new_empty((B, T, heads, slices), dtype=torch.float32) for _ in range(2)]
    return (*qkv, *gates)


@custom_op("tgdn_b200::conv_split_norm_bwd", mutates_args=(), device_types="cuda")
def conv_split_norm_bwd(x: torch.Tensor, weight: torch.Tensor, dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor,
                        dk2: torch.Tensor, dq2: torch.Tensor, heads: int, slices: int, eps: float,
                        cu_seqlens: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    wdtype = weight.dtype
    x, weight, cu, n_docs, _ = _prep(x, weight, cu_seqlens)
    B, T, C = x.shape
    dq, dk, dv = (t.to(torch.bfloat16).contiguous() for t in (dq, dk, dv))
    dk2, dq2 = (t.to(torch.float32).contiguous() for t in (dk2, dq2))
    dy = torch.empty((B, T, C), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.tgdn_glue_bwd_norm(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(cu), n_docs, B, T, C, x.stride(0),
                                               x.stride(1), heads, slices, float(eps), _lib.ptr(dq), _lib.ptr(dk),
                                               _lib.ptr(dv), _lib.ptr(dk2), _lib.ptr(dq2), _lib.ptr(dy),
                                               _lib.stream_of(x)), "tgdn_glue_bwd_norm")
    dx, dw = conv_split_act_bwd(x, dy, weight, 3 * heads * 128, cu)
    return dx, dw.to(wdtype)


@conv_split_norm_bwd.register_fake
def _(x, weight, dq, dk, dv, dk2, dq2, heads, slices, eps, cu_seqlens=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight)


def _glue_remember(ctx, inputs, output):
    x, weight, heads, slices, eps, cu_seqlens = inputs
    ctx.save_for_backward(*([x, weight] + ([] if cu_seqlens is None else [cu_seqlens])))
    ctx.glue = (int(heads), int(slices), float(eps))


def _glue_differentiate(ctx, dq, dk, dv, dk2, dq2):
    kept = ctx.saved_tensors
    offsets = kept[2] if len(kept) == 3 else None
    heads, slices, eps = ctx.glue
    dx, dw = conv_split_norm_bwd(kept[0], kept[1], dq, dk, dv, dk2, dq2, heads, slices, eps, offsets)
    return dx, dw, None, None, None, None


register_autograd("tgdn_b200::conv_split_norm_fwd", _glue_differentiate, setup_context=_glue_remember)


def conv_split_norm_call(x, weight, heads, slices, cu_seqlens=None, eps=1e-6):
    """The convolution pre-pass with the layer glue fused in: x (B, T, C) bf16 with C = heads*(3*128 + 2*slices) channels
    laid out [q | k | v | k2 | q2] goes straight to what `gdn_joint_call` takes,

        q, k = l2norm(SiLU(conv(x)))  bf16 (B, T, heads, 128)      v = SiLU(conv(x))  bf16 (B, T, heads, 128)
        k2, q2 = l2norm(softplus(conv(x)))  f32 (B, T, heads, slices),     l2norm(s) = s * rsqrt(sum s^2 + eps),

    without the convolution's output ever being written.  Differentiable in x and weight; packed rows as in
    `conv_split_act_call`."""
    return conv_split_norm_fwd(x, weight.contiguous(), int(heads), int(slices), float(eps), cu_seqlens)
