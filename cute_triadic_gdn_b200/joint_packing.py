"""Packed documents: validation and the device-built chunk metadata.

Mirrors cute_triadic_gdn/ops/joint_packing.py:10-62 (chunk_capacity, the joint_metadata3 op, _validate,
prepare_documents): same checks, same errors, no host read of the offsets.
"""
from __future__ import annotations

import torch
from torch.library import custom_op

from . import _lib

CHUNK = 64
NC_BUCKET = 16


def chunk_capacity(tokens, documents):
    """sum(ceil(len_i / 64)) <= ceil(tokens / 64) + documents - 1, rounded up to a multiple of 16."""
    exact = (tokens + CHUNK - 1) // CHUNK + documents - 1
    return -(-exact // NC_BUCKET) * NC_BUCKET


@custom_op("tgdn_b200::joint_metadata", mutates_args=(), device_types="cuda")
def _metadata(cu_seqlens: torch.Tensor, tokens: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    documents = cu_seqlens.numel() - 1
    capacity = chunk_capacity(tokens, documents)
    dev = cu_seqlens.device
    offsets = torch.empty(documents + 1, dtype=torch.int32, device=dev)
    mapping = torch.empty((3, capacity), dtype=torch.int32, device=dev)
    valid = torch.empty(1, dtype=torch.bool, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.tgdn_metadata(_lib.ptr(cu_seqlens), int(cu_seqlens.dtype == torch.int64), documents,
                                          int(tokens), _lib.ptr(offsets), _lib.ptr(mapping), capacity, _lib.ptr(valid),
                                          _lib.stream_of(cu_seqlens)), "tgdn_metadata")
    return offsets, mapping, valid


@_metadata.register_fake
def _metadata_fake(cu_seqlens, tokens):
    documents = cu_seqlens.numel() - 1
    capacity = chunk_capacity(tokens, documents)
    return (cu_seqlens.new_empty(documents + 1, dtype=torch.int32),
            cu_seqlens.new_empty((3, capacity), dtype=torch.int32),
            cu_seqlens.new_empty(1, dtype=torch.bool))


def _validate(inputs, cu_seqlens):
    q = inputs[0]
    if q.shape[0] != 1 or q.shape[1] <= 0:
        raise ValueError("cu_seqlens requires a nonempty packed row: B=1, T>0")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must be a vector with at least two offsets")
    if cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise ValueError("cu_seqlens must have dtype int32 or int64")
    if cu_seqlens.device != q.device or not cu_seqlens.is_contiguous():
        raise ValueError("cu_seqlens must be contiguous and on the input device")
    if q.shape[1] > 2 ** 31 - 1:
        raise ValueError("packed token offsets must fit int32")


def prepare_documents(inputs, cu_seqlens):
    """Validate the offsets and build (chunk offsets per document, chunk map) on the device; tokens are not copied."""
    _validate(inputs, cu_seqlens)
    q = inputs[0]
    offsets, mapping, valid = _metadata(cu_seqlens, q.shape[1])
    torch._assert_async(valid, "cu_seqlens must start at 0, end at T, and strictly increase")
    return offsets, mapping
