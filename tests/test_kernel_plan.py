"""oracle/kernel_plan.py, the torch model of the CUDA kernels' dataflow that the stage-level GPU tests compare with.

Rounding off, float64: the model's explicit backward formulas must agree with autograd through the oracle's chunkwise
restatement to round-off.  Rounding on (a bf16 rounding wherever the kernels store or stage a tensor in bf16), float32:
the model must stay inside the parity tolerance of the hot path (o 1e-2, every gradient 2e-2 relative L2), on both input
distributions, which is what makes the rounding plan admissible.
"""
import pytest
import torch

from helpers import GRADS
from oracle import triadic_oracle as orc
from oracle.kernel_plan import run_plan


def _case(B, T, H, E, dist, seed=1):
    ins = orc.make_inputs(B, T, H, E, seed, dist)
    do = orc.make_grad_output((B, T, H, 128), 7)
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, ins, do, dtype=torch.float64)
    return ins, do, o_ref, g_ref


@pytest.mark.parametrize("B,T,H,E,dist", [(1, 192, 2, 4, "baseline"), (1, 128, 1, 1, "baseline"), (1, 128, 1, 8, "mild"),
                                          (1, 128, 1, 12, "baseline")])
def test_backward_formulas_match_autograd(B, T, H, E, dist):
    ins, do, o_ref, g_ref = _case(B, T, H, E, dist)
    o, grads, _ = run_plan(*ins, do, rounding=False, dtype=torch.float64)
    assert orc.rel_l2(o, o_ref) < 1e-12
    for n, a, b in zip(GRADS, grads, g_ref):
        assert orc.rel_l2(a, b) < 1e-10, n


@pytest.mark.parametrize("B,T,H,E,dist", [(1, 512, 2, 8, "baseline"), (1, 512, 2, 8, "mild"), (1, 256, 1, 16, "baseline"),
                                          (1, 256, 2, 1, "mild"), (1, 256, 1, 12, "mild")])
def test_rounding_plan_is_inside_the_tolerance(B, T, H, E, dist):
    ins, do, o_ref, g_ref = _case(B, T, H, E, dist)
    o, grads, _ = run_plan(*ins, do, rounding=True, dtype=torch.float32)
    assert orc.rel_l2(o, o_ref) < 1e-2
    for n, a, b in zip(GRADS, grads, g_ref):
        assert orc.rel_l2(a, b) < 2e-2, n


def test_document_resets():
    """`reset` marks chunks that start a document: the model must equal the oracle run on the packed row."""
    ins = orc.make_inputs(1, 256, 1, 4, 5, "mild")
    do = orc.make_grad_output((1, 256, 1, 128), 7)
    cu = torch.tensor([0, 128, 256], dtype=torch.int32)
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, ins, do, cu_seqlens=cu, dtype=torch.float64)
    o, grads, _ = run_plan(*ins, do, reset=[True, False, True, False], rounding=False, dtype=torch.float64)
    assert orc.rel_l2(o, o_ref) < 1e-12
    for n, a, b in zip(GRADS, grads, g_ref):
        assert orc.rel_l2(a, b) < 1e-10, n
