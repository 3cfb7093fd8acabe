"""Seeded random shapes and document layouts against the fp32 oracle: odd head counts, single-chunk rows, one-token
documents, documents that end one token past a chunk boundary, every supported slice count."""
import random

import pytest
import torch

from cute_triadic_gdn_b200 import _lib, gdn_joint_call
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu

TOL_O, TOL_G = 1e-2, 2e-2          # relative L2 against the fp32 run of the reference's torch path


def _cases():
    rnd = random.Random(20240607)
    out = []
    for i in range(14):
        E = rnd.choice([1, 2, 4, 8, 12, 16])
        H = rnd.choice([1, 2, 3, 5])
        if i % 2 == 0:                                    # dense
            out.append((rnd.choice([1, 2, 3]), 64 * rnd.choice([1, 2, 3, 5]), H, E, None))
        else:                                             # packed: a few documents with awkward lengths
            lens = [rnd.choice([1, 2, 63, 64, 65, 100, 129, 200]) for _ in range(rnd.choice([1, 2, 4, 6]))]
            cu = [0]
            for n in lens:
                cu.append(cu[-1] + n)
            out.append((1, cu[-1], H, E, cu))
    return out


@pytest.mark.parametrize("B,T,H,E,docs", _cases())
def test_random_shape_matches_oracle(B, T, H, E, docs):
    inputs = orc.make_inputs(B, T, H, E, seed=1000 * E + T + H, dist="baseline")
    do = orc.make_grad_output((B, T, H, 128), 11)
    cu = torch.tensor(docs, dtype=torch.int32) if docs else None
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, inputs, do, cu_seqlens=cu, dtype=torch.float32)
    leaves = [t.detach().clone().cuda().requires_grad_(True) for t in inputs]
    o = gdn_joint_call(*leaves, cu_seqlens=None if cu is None else cu.cuda())
    o.backward(do.cuda())
    assert _lib.device_status() == 0
    assert orc.rel_l2(o.detach().float().cpu(), o_ref) < TOL_O
    for name, t, ref in zip(("dq", "dk", "dv", "dk2", "dq2", "dg", "dbeta"), leaves, g_ref):
        err = orc.rel_l2(t.grad.float().cpu(), ref)
        assert err < TOL_G, f"{name}: {err:.3e}"
