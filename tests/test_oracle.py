"""The CPU oracle against outputs of the reference itself (tests/golden) and against the token-by-token definition."""
import os

import numpy as np
import pytest
import torch

from oracle import triadic_oracle as orc
from helpers import GRADS, bf16, conv_files, core_files, load_core


@pytest.mark.parametrize("path", core_files(), ids=os.path.basename)
def test_chunk_oracle_matches_reference_outputs(path):
    ins, do, cu, ref = load_core(path)
    o, grads = orc.reference_with_grads(orc.chunk_reference, ins, do, cu_seqlens=cu, dtype=torch.float32)
    assert orc.rel_l2(o, ref["o"]) < 2e-5
    for n, gr in zip(GRADS, grads):
        assert orc.rel_l2(gr, ref["d" + n]) < 2e-4, n


@pytest.mark.parametrize("path", [p for p in core_files() if "e2" in p or "e8" in p], ids=os.path.basename)
def test_definition_matches_reference_outputs(path):
    ins, do, cu, ref = load_core(path)
    o, grads = orc.reference_with_grads(orc.sequential_reference, ins, do, cu_seqlens=cu, dtype=torch.float64)
    assert orc.rel_l2(o, ref["o"]) < 2e-5
    for n, gr in zip(GRADS, grads):
        assert orc.rel_l2(gr, ref["d" + n]) < 2e-4, n


@pytest.mark.parametrize("path", conv_files(), ids=os.path.basename)
def test_conv_oracle_matches_reference_kernels(path):
    z = np.load(path)
    x, w, dy = bf16(z["x"]), bf16(z["w"]), bf16(z["dy"])
    cu = torch.from_numpy(z["cu_seqlens"]) if "cu_seqlens" in z.files else None
    act = int(z["act"])
    y32 = orc.conv_reference(x, w, act, cu, rounded=False)
    dx, dw = orc.conv_reference_backward(x, w, act, dy, cu)
    ry, rdx = bf16(z["ref_y"]).float(), bf16(z["ref_dx"]).float()
    # The fixture was produced by the Triton interpreter, whose f32 -> bf16 store truncates (the compiled kernel
    # rounds to nearest even, which is what the oracle does): compare with the truncation of the oracle's f32 value.
    trunc = (y32.view(torch.int32) & -65536).view(torch.float32)
    assert ((trunc - ry).abs() <= 2 ** -7 * ry.abs() + 1e-30).all()
    assert (trunc == ry).float().mean() > 0.98
    assert orc.rel_l2(y32, ry) < 5e-3
    assert orc.rel_l2(dx.float(), rdx) < 5e-3
    assert orc.rel_l2(dw.float(), torch.from_numpy(z["ref_dw_f32"])) < 5e-3


def test_lognormal_documents_cover_the_row():
    cu = orc.lognormal_documents(131072, seed=3)
    assert cu[0] == 0 and cu[-1] == 131072 and (cu[1:] > cu[:-1]).all()
