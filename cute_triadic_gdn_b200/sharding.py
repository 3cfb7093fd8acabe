"""Partitioning of the Triadic GDN hot path over GPUs (or over pipeline slices): no exchange step anywhere.

Every kernel is independent per (batch row, head) and per document (the state restarts at every document start,
cute_triadic_gdn/ops/gdn_joint.py:72-73), so the work is cut along those axes and each part is a complete, ordinary
call of `gdn_joint_call`:

  dense rows   contiguous blocks of heads (then batch rows)              -> `head_slice`
  packed rows  contiguous ranges of whole documents, token-balanced      -> `document_ranges`, `shard_documents`

A range of documents is a contiguous range of tokens, so slicing the token axis of a `(1, T, ...)` tensor gives a
contiguous view: nothing is copied, and the offsets are re-based to start at zero.
"""
from __future__ import annotations

from typing import NamedTuple, Sequence

import torch


def head_slice(heads: int, world: int, rank: int) -> slice:
    """Rank `rank` of `world` gets heads [rank*H/world, (rank+1)*H/world); `world` must divide `heads`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if heads % world:
        raise ValueError(f"{heads} heads are not divisible over {world} parts")
    per = heads // world
    return slice(rank * per, (rank + 1) * per)


class DocumentRange(NamedTuple):
    doc_lo: int      # first document of the part
    doc_hi: int      # one past its last document (doc_lo == doc_hi: the part is empty)
    tok_lo: int      # first token
    tok_hi: int      # one past the last token


def _offsets(cu_seqlens) -> list[int]:
    cu = cu_seqlens.detach().cpu().tolist() if isinstance(cu_seqlens, torch.Tensor) else [int(c) for c in cu_seqlens]
    if len(cu) < 2 or cu[0] != 0 or any(b <= a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must be strictly increasing and start at 0")
    return cu


def document_ranges(cu_seqlens, parts: int) -> list[DocumentRange]:
    """Cut the documents into `parts` contiguous ranges whose token counts are as even as whole documents allow.

    The k-th cut is the document boundary nearest to k*T/parts (ties go to the earlier boundary); cuts never move
    backwards, so with fewer documents than parts some ranges are empty.  Deterministic, host-side, O(N + parts).
    """
    if parts < 1:
        raise ValueError("parts must be positive")
    cu = _offsets(cu_seqlens)
    total, n_docs = cu[-1], len(cu) - 1
    cuts, j = [0], 0
    for k in range(1, parts):
        target = k * total / parts
        while j < n_docs and abs(cu[j + 1] - target) < abs(cu[j] - target):
            j += 1
        cuts.append(j)
    cuts.append(n_docs)
    return [DocumentRange(a, b, cu[a], cu[b]) for a, b in zip(cuts, cuts[1:])]


def shard_documents(inputs: Sequence[torch.Tensor], cu_seqlens: torch.Tensor, parts: int, index: int):
    """Part `index` of `parts` of a packed problem: (views of the inputs on its tokens, its re-based offsets, its range).

    `inputs` are `(1, T, ...)` tensors sharing the token axis; the views are contiguous.  An empty part returns views of
    length zero and `None` for the offsets: there is nothing to call the kernels with.
    """
    rng = document_ranges(cu_seqlens, parts)[index]
    views = [t[:, rng.tok_lo:rng.tok_hi] for t in inputs]
    if rng.doc_lo == rng.doc_hi:
        return views, None, rng
    cu = cu_seqlens[rng.doc_lo:rng.doc_hi + 1] - cu_seqlens[rng.doc_lo]
    return views, cu.contiguous(), rng
