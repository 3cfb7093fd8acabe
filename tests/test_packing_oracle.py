"""The CPU restatement of the packed-document metadata, pinned by what the reference's own pack_documents
(cute_triadic_gdn/ops/joint_packing.py:65-90) makes of the same offsets.

tests/golden/packing_cases.npz stores, per offsets vector, the reference's `restore` (token -> position in the row that
pads every document to whole chunks) and `chunk_starts` (padded chunk begins a document).  Position // 64 is the chunk a
token lands in, so the two arrays fix every chunk's first token and number of valid rows and every document's first
chunk: exactly the chunk map the device kernel must build (cute_triadic_gdn/kernels/sm90_joint_packed.py:64-99).
"""
import os

import numpy as np
import pytest

from helpers import GOLDEN
from oracle import packing_oracle

Z = np.load(os.path.join(GOLDEN, "packing_cases.npz"))
N_CASES = sum(1 for k in Z.files if k.startswith("cu_"))


@pytest.mark.parametrize("i", range(N_CASES))
def test_chunk_map_matches_reference_packing(i):
    cu, restore, flags = Z[f"cu_{i}"], Z[f"restore_{i}"], Z[f"chunk_starts_{i}"]
    T, n = int(cu[-1]), len(cu) - 1
    offsets, start, rows, order, ok = packing_oracle.metadata(cu.tolist(), T)
    assert ok
    chunk_of = restore // 64
    used = int(chunk_of.max()) + 1
    assert offsets[-1] == used                                     # chunks in use
    # every chunk: first token and valid rows as the reference's padding implies
    for c in range(used):
        toks = np.nonzero(chunk_of == c)[0]
        assert start[c] == toks[0] and rows[c] == len(toks)
        assert (np.diff(toks) == 1).all() and (restore[toks] % 64 == np.arange(len(toks))).all()
    assert (rows[used:] == 0).all() and (start[used:] == T).all()  # unused capacity: no rows, first token = T
    # every document: its first chunk is where the reference raises its reset flag
    assert np.nonzero(flags[:used])[0].tolist() == offsets[:-1].tolist()
    # capacity: the reference's padded row rounded up to the bucket of 16 chunks
    assert len(start) == packing_oracle.chunk_capacity(T, n) and len(start) >= len(flags) and len(start) % 16 == 0
    # longest-first order: a permutation of the documents, chunk counts non-increasing, ties in document order
    counts = np.diff(offsets)
    assert sorted(order.tolist()) == list(range(n))
    key = [(-counts[d], d) for d in order]
    assert key == sorted(key)


@pytest.mark.parametrize("cu,T", [([0, 70, 60, 640], 640), ([1, 70, 640], 640), ([0, 70, 600], 640), ([0, 70, 70, 640], 640)])
def test_bad_offsets_are_flagged(cu, T):
    assert not packing_oracle.metadata(cu, T)[4]
