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
    """Entries of the chunk map of a packed row.  N documents over T tokens need at most ceil(T / 64) + N - 1 chunks (every
    document but one can end in a partial chunk); the count is rounded up to the next multiple of 16 so that it takes few
    distinct values from batch to batch.  Same number as the reference's (ops/joint_packing.py:16-20) and tgdn_chunk_capacity."""
    worst = -(-tokens // CHUNK) + documents - 1
    return NC_BUCKET * (-(-worst // NC_BUCKET))


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
def _metadata_shapes(cu_seqlens, tokens):
    n = cu_seqlens.numel() - 1
    like = cu_seqlens.new_empty
    return like(n + 1, dtype=torch.int32), like((3, chunk_capacity(tokens, n)), dtype=torch.int32), like(1, dtype=torch.bool)


def _validate(inputs, cu_seqlens):
    """What can be checked without reading the offsets: a ValueError for the conditions the reference rejects
    (ops/joint_packing.py:38-49).  The values themselves are checked on the device."""
    row = inputs[0]
    if row.shape[0] != 1 or row.shape[1] < 1:
        raise ValueError(f"a packed row has shape (1, T, ...) with T >= 1; got {tuple(row.shape)}")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens: a vector of document offsets, at least [0, T]")
    if cu_seqlens.dtype != torch.int32 and cu_seqlens.dtype != torch.int64:
        raise ValueError(f"cu_seqlens: int32 or int64 offsets, got {cu_seqlens.dtype}")
    if not cu_seqlens.is_contiguous() or cu_seqlens.device != row.device:
        raise ValueError("cu_seqlens: must be contiguous and live on the device of the inputs")
    if row.shape[1] >= 2 ** 31:
        raise ValueError("a packed row is limited to 2^31 - 1 tokens (offsets are 32-bit on the device)")


def prepare_documents(inputs, cu_seqlens):
    """(first chunk of every document, chunk map) of a packed row, built on the device from the offsets; no token is
    copied and nothing is read back.  Offsets that do not start at 0, end at T and strictly increase trip a device-side
    assertion, as in the reference (ops/joint_packing.py:52-62)."""
    _validate(inputs, cu_seqlens)
    offsets, mapping, valid = _metadata(cu_seqlens, inputs[0].shape[1])
    torch._assert_async(valid, "cu_seqlens must start at 0, end at T, and strictly increase")
    return offsets, mapping
