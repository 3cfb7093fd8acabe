"""Activation checkpointing around the custom ops.

torch.utils.checkpoint(use_reentrant=False) re-runs the forward inside the backward and unpacks every saved tensor exactly
once; the reference documents the contract its autograd glue keeps for that (cute_triadic_gdn/ops/joint_torch_ops.py:67-72:
one read of ctx.saved_tensors, no materialised zero gradients for the auxiliary outputs).  The same must hold here: the
checkpointed call gives bitwise the gradients of the plain call, with GJ_SAVE_MASKS on and off, dense and packed."""
import pytest
import torch
from torch.utils.checkpoint import checkpoint

from cute_triadic_gdn_b200 import _lib, conv_split_act_call, gdn_joint_call
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


def _grads(fn, inputs, do, cu):
    leaves = [t.detach().clone().requires_grad_(True) for t in inputs]
    o = fn(*leaves, cu)
    o.backward(do)
    return o.detach(), [t.grad for t in leaves]


@pytest.mark.parametrize("save_masks", ["1", "0"])
@pytest.mark.parametrize("packed", [False, True])
def test_checkpointed_call_equals_plain_call(monkeypatch, save_masks, packed):
    monkeypatch.setenv("GJ_SAVE_MASKS", save_masks)
    B, T, H, E = (1, 320, 2, 8) if packed else (2, 256, 2, 8)
    ins = [t.cuda() for t in orc.make_inputs(B, T, H, E, seed=55, dist="mild")]
    do = orc.make_grad_output((B, T, H, 128), 7).cuda()
    cu = torch.tensor([0, 64, 65, 320], dtype=torch.int32, device="cuda") if packed else None
    plain = lambda *a: gdn_joint_call(*a[:7], cu_seqlens=a[7])
    ckpt = lambda *a: checkpoint(lambda *b: gdn_joint_call(*b, cu_seqlens=a[7]), *a[:7], use_reentrant=False)
    o_p, g_p = _grads(plain, ins, do, cu)
    o_c, g_c = _grads(ckpt, ins, do, cu)
    assert _lib.device_status() == 0
    assert torch.equal(o_p, o_c)
    for a, b in zip(g_p, g_c):
        assert torch.equal(a, b)


def test_checkpointed_conv_equals_plain_call():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(1, 300, 256, generator=g).to(torch.bfloat16).cuda()
    w = (0.5 * torch.randn(256, 4, generator=g)).to(torch.bfloat16).cuda()
    dy = torch.randn(1, 300, 256, generator=g).to(torch.bfloat16).cuda()
    cu = torch.tensor([0, 100, 300], dtype=torch.int32, device="cuda")

    def grads(fn):
        xl, wl = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = fn(xl, wl)
        y.backward(dy)
        return y.detach(), xl.grad, wl.grad

    a = grads(lambda xl, wl: conv_split_act_call(xl, wl, 128, cu))
    b = grads(lambda xl, wl: checkpoint(lambda p, q: conv_split_act_call(p, q, 128, cu), xl, wl, use_reentrant=False))
    for u, v in zip(a, b):
        assert torch.equal(u, v)
