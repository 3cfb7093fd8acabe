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
    if x.ndim != 3 or weight.ndim != 2 or weight.shape[0] != x.shape[2] or weight.shape[1] != 4:
        raise ValueError("x must be (B, T, C) and weight (C, 4)")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ValueError("x and weight must be bf16")
    if not x.is_cuda or weight.device != x.device:
        raise ValueError("x and weight must be on the same CUDA device")
    if x.shape[2] % 8:
        raise ValueError("the channel count must be a multiple of 8")
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
    return x, weight.contiguous(), cu_seqlens, n_docs


@custom_op("tgdn_b200::conv_split_act_fwd", mutates_args=(), device_types="cuda")
def conv_split_act_fwd(x: torch.Tensor, weight: torch.Tensor, act_channels: int,
                       cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
    x, weight, cu, n_docs = _prep(x, weight, cu_seqlens)
    B, T, C = x.shape
    y = torch.empty((B, T, C), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.tgdn_conv_fwd(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(cu), n_docs, B, T, C,
                                          x.stride(0), x.stride(1), int(act_channels), _lib.stream_of(x)),
                   "tgdn_conv_fwd")
    return y


@conv_split_act_fwd.register_fake
def _(x, weight, act_channels, cu_seqlens=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@custom_op("tgdn_b200::conv_split_act_bwd", mutates_args=(), device_types="cuda")
def conv_split_act_bwd(x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor, act_channels: int,
                       cu_seqlens: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    x, weight, cu, n_docs = _prep(x, weight, cu_seqlens)
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
    return dx, dw


@conv_split_act_bwd.register_fake
def _(x, dy, weight, act_channels, cu_seqlens=None):
    return torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(weight)


def _setup(ctx, inputs, output):
    x, weight, act_channels, cu_seqlens = inputs
    ctx.save_for_backward(x, weight, *([cu_seqlens] if cu_seqlens is not None else []))
    ctx.act_channels = act_channels
    ctx.has_cu = cu_seqlens is not None


def _backward(ctx, dy):
    saved = ctx.saved_tensors
    cu_seqlens = saved[2] if ctx.has_cu else None
    dx, dw = conv_split_act_bwd(saved[0], dy, saved[1], ctx.act_channels, cu_seqlens)
    return dx, dw, None, None


register_autograd("tgdn_b200::conv_split_act_fwd", _backward, setup_context=_setup)


def conv_split_act_call(x, weight, act_channels, cu_seqlens=None):
    """x [B, T, C] bf16, weight [C, 4] bf16; channels [0, act_channels) get SiLU, the rest none.  cu_seqlens: document
    boundaries of a packed row (the convolution restarts at each document)."""
    return conv_split_act_fwd(x, weight.contiguous(), int(act_channels), cu_seqlens)
