"""End-to-end parity of the kernels with the CPU oracle: forward output and the gradients of all seven inputs.

Cases and structure follow the reference's tests/test_joint.py:46-67 (E in 1/2/4/8/12/16, batch rows and packed
documents, custom-op call bitwise equal to the direct call); tolerances are the tighter ones of the build target:
o within 1e-2 and every gradient within 2e-2 relative L2 of an fp32 evaluation of the reference math.
"""
import os

import pytest
import torch

from cute_triadic_gdn_b200 import _lib, chunk_gdn_joint, gdn_joint_call
from oracle import triadic_oracle as orc
from helpers import GRADS, core_files, load_core

pytestmark = pytest.mark.gpu
TOL_O, TOL_G = 1e-2, 2e-2

CASES = [(2, 256, 4, 1, None), (2, 256, 4, 2, None), (2, 256, 4, 4, None), (2, 256, 4, 8, None),
         (2, 256, 4, 12, None), (2, 256, 4, 16, None),
         (1, 640, 4, 8, [0, 70, 133, 400, 640]), (1, 320, 4, 2, [0, 64, 65, 320]), (1, 512, 4, 4, [0, 512]),
         (1, 3000, 8, 16, [0, 17, 900, 901, 1500, 2999, 3000])]


def run(fn, inputs, do, cu):
    leaves = [t.detach().clone().cuda().requires_grad_(True) for t in inputs]
    o = fn(*leaves, cu_seqlens=None if cu is None else cu.cuda())
    o.backward(do.cuda())
    return o.detach(), [t.grad for t in leaves]


def compare(o, grads, o_ref, g_ref):
    assert orc.rel_l2(o.float().cpu(), o_ref) < TOL_O, f"forward {orc.rel_l2(o.float().cpu(), o_ref):.3e}"
    for name, a, b in zip(GRADS, grads, g_ref):
        err = orc.rel_l2(a.float().cpu(), b)
        assert err < TOL_G, f"grad {name}: {err:.3e}"


@pytest.mark.parametrize("dist", ["mild", "baseline"])
@pytest.mark.parametrize("B,T,H,E,docs", CASES)
def test_against_oracle(B, T, H, E, docs, dist):
    inputs = orc.make_inputs(B, T, H, E, seed=E * 1000 + T, dist=dist)
    do = orc.make_grad_output((B, T, H, 128), 7)
    cu = torch.tensor(docs, dtype=torch.int32) if docs else None
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, inputs, do, cu_seqlens=cu, dtype=torch.float32)
    o_ker, g_ker = run(chunk_gdn_joint, inputs, do, cu)
    assert _lib.device_status() == 0
    compare(o_ker, g_ker, o_ref, g_ref)
    o_op, g_op = run(gdn_joint_call, inputs, do, cu)
    assert torch.equal(o_op, o_ker), "custom-op call differs from the direct call"
    for name, a, b in zip(GRADS, g_op, g_ker):
        assert torch.equal(a, b), f"custom-op grad {name} differs from the direct call"


@pytest.mark.parametrize("path", core_files(), ids=os.path.basename)
def test_against_reference_outputs(path):
    """The stored outputs of the reference's own torch path (fp32)."""
    inputs, do, cu, ref = load_core(path)
    o, grads = run(chunk_gdn_joint, inputs, do, cu)
    assert _lib.device_status() == 0
    compare(o, grads, ref["o"], [ref["d" + n] for n in GRADS])


@pytest.mark.parametrize("docs", [None, [0, 100, 101, 384]])
def test_recomputed_masks_are_bitwise_identical(docs, monkeypatch):
    T = 384
    inputs = orc.make_inputs(1, T, 2, 4, seed=5)
    do = orc.make_grad_output((1, T, 2, 128), 7)
    cu = torch.tensor(docs, dtype=torch.int32) if docs else None
    monkeypatch.setenv("GJ_SAVE_MASKS", "1")
    o1, g1 = run(gdn_joint_call, inputs, do, cu)
    monkeypatch.setenv("GJ_SAVE_MASKS", "0")
    o0, g0 = run(gdn_joint_call, inputs, do, cu)
    assert torch.equal(o1, o0)
    for a, b in zip(g1, g0):
        assert torch.equal(a, b)


def test_inference_path_and_argument_checks():
    inputs = [t.cuda() for t in orc.make_inputs(1, 128, 2, 2, seed=9)]
    with torch.no_grad():
        o = chunk_gdn_joint(*inputs)
    o2 = gdn_joint_call(*inputs)
    assert torch.equal(o, o2)
    with pytest.raises(AssertionError):
        chunk_gdn_joint(inputs[0][:, :100], *[t[:, :100] for t in inputs[1:]])          # T % 64
    with pytest.raises(AssertionError):
        chunk_gdn_joint(inputs[0].float(), *inputs[1:])                                  # dtype
    with pytest.raises(NotImplementedError):
        chunk_gdn_joint(*inputs, reference=True)
    bad = [t.cuda() for t in orc.make_inputs(1, 128, 2, 3, seed=9)]
    with pytest.raises(ValueError):
        chunk_gdn_joint(*bad)                                                            # E = 3
    with pytest.raises(ValueError):
        gdn_joint_call(*[t.repeat(2, *([1] * (t.ndim - 1))) for t in inputs],
                       cu_seqlens=torch.tensor([0, 128], dtype=torch.int32, device="cuda"))   # packed needs B = 1


@pytest.mark.parametrize("E", [2, 8])
def test_steep_decay_takes_the_direct_mask_gradient_path(E):
    """Gates of -6 .. -10 per token: a 16-row block decays by far more than 2^-100, which switches the matrix-gradient
    kernel from its factorised decay tables to one exponential per (t, s, e); the results must still match the oracle."""
    B, T, H = 1, 256, 2
    inputs = list(orc.make_inputs(B, T, H, E, seed=900 + E, dist="mild"))
    gen = torch.Generator().manual_seed(17)
    inputs[5] = -(6.0 + 4.0 * torch.rand(B, T, H, E, generator=gen))
    do = orc.make_grad_output((B, T, H, 128), 7)
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, inputs, do, dtype=torch.float32)
    o_ker, g_ker = run(chunk_gdn_joint, inputs, do, None)
    assert _lib.device_status() == 0
    compare(o_ker, g_ker, o_ref, g_ref)


@pytest.mark.parametrize("E", [2, 8])
def test_log_gates_above_zero_follow_the_recurrence(E):
    """The contract, as in the reference, is g <= 0 (the log of a decay).  A gate above zero makes the chunk-local cumulative
    gate rise from one row to the next; the kernels must then leave their factorised decay tables (which would clamp such
    a factor at one without a word) and evaluate exp(gc_t - gc_s) as it is, like the reference's kernels, which gives the
    token-by-token recurrence S_e <- exp(g_te) S_e itself.  (The reference's torch path clamps that factor in its masks,
    cute_triadic_gdn/ops/gdn_joint.py:54, and so leaves the recurrence for such inputs; the definition is the yardstick here.)"""
    B, T, H = 1, 128, 2
    inputs = list(orc.make_inputs(B, T, H, E, seed=950 + E, dist="mild"))
    g = inputs[5].clone()
    g[:, 16] = 0.4                                              # the case of a single raised gate at a block boundary
    g[:, 37, :, 0] = 0.25
    inputs[5] = g
    do = orc.make_grad_output((B, T, H, 128), 7)
    o_ref, g_ref = orc.reference_with_grads(orc.sequential_reference, inputs, do, dtype=torch.float64)
    o_ker, g_ker = run(chunk_gdn_joint, inputs, do, None)
    assert _lib.device_status() == 0
    compare(o_ker, g_ker, o_ref.float(), [x.float() for x in g_ref])
