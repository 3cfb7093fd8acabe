"""CPU restatement of the packed-document metadata.  TEST INFRASTRUCTURE ONLY.

Follows cute_triadic_gdn/kernels/sm90_joint_packed.py:64-99 (metadata_kernel) and
cute_triadic_gdn/ops/joint_packing.py:16-20 (chunk_capacity): per document the index of its first 64-token chunk,
per chunk its first token and its number of valid rows, and the documents ordered longest first (ties in document order).
Parity pinned: the reference's device kernel needs a GPU and its DSL, but its host statement of the same chunking,
pack_documents (cute_triadic_gdn/ops/joint_packing.py:65-90), runs anywhere; what it makes of the packed cases is stored
in tests/golden/packing_cases.npz (written by tests/golden/make_golden.py) and tests/test_packing_oracle.py holds this
restatement to it.
"""
import numpy as np


def chunk_capacity(tokens, documents):
    exact = (tokens + 63) // 64 + documents - 1
    return -(-exact // 16) * 16


def metadata(cu, tokens):
    cu = [int(c) for c in cu]
    n = len(cu) - 1
    cap = chunk_capacity(tokens, n)
    valid = cu[0] == 0 and cu[-1] == tokens and all(b > a for a, b in zip(cu, cu[1:]))
    counts = [(b - a + 63) // 64 for a, b in zip(cu, cu[1:])]
    offsets = np.zeros(n + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    start = np.full(cap, tokens, dtype=np.int32)
    rows = np.zeros(cap, dtype=np.int32)
    for d in range(n):
        for s in range(counts[d]):
            start[offsets[d] + s] = cu[d] + 64 * s
            rows[offsets[d] + s] = min(64, cu[d + 1] - cu[d] - 64 * s)
    order = sorted(range(n), key=lambda d: (-counts[d], d))
    return offsets, start, rows, np.asarray(order, dtype=np.int32), valid
