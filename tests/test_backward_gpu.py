"""Backward kernels on the device, stage by stage against the torch model of the kernels' dataflow."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib
from cute_triadic_gdn_b200 import gdn_joint as gj
from oracle import kernel_plan as plan
from oracle import triadic_oracle as orc
from plan_helpers import decode_items, state_to_matrix

pytestmark = pytest.mark.gpu


def _gpu(ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("E", [1, 2, 4, 8, 12, 16])
@pytest.mark.parametrize("dist", ["baseline", "mild"])
def test_reverse_recurrence_dense(E, dist):
    B, T, H = 2, 256, 2
    ins = orc.make_inputs(B, T, H, E, seed=200 + E, dist=dist)
    do = orc.make_grad_output((B, T, H, 128), 7)
    scale = 128 ** -0.5
    q, k, v, k2, q2, g, beta = _gpu(ins)
    o, gc, AP, Pm, h, W, U = gj._kernel_forward(q, k, v, k2, q2, g, beta, scale, True)
    dog = do.cuda()
    dV, dU, ds, dkg, dr = gj._run_reverse(q, k, dog, k2, q2, beta, gc, AP, Pm, U, scale)
    assert _lib.device_status() == 0
    _, grads, st = plan.run_plan(*ins, do, rounding=True)
    rv, sg = st["rev"], st["sg"]
    NC = T // 64
    conv = lambda t: t.cpu().float().permute(0, 2, 1, 3, 4).reshape(B * H, NC, 64, 128)
    assert orc.rel_l2(conv(dU), rv["dU"]) < 8e-3
    assert orc.rel_l2(dV.cpu().float(), grads[2]) < 8e-3
    # the gradient state is stored only for the slices whose chunk decay is at least 2^-24
    keep = (gj.chunk_gates(gc, E)[:, :, :, 63, :] * 1.4426950408889634 >= plan.DD_MIN_LOG2_DECAY).cpu()           # (B, NC, H, E)
    keep = keep.permute(0, 2, 1, 3).reshape(B * H, NC, E)
    dsm = decode_items(ds.cpu().float(), state_to_matrix)                                     # (B*H, NC, E, 128, 128)
    if keep.any():
        assert orc.rel_l2(dsm[keep], rv["ds"][keep]) < 1e-2
    if dist == "baseline":
        assert not keep.any()                               # decay of 64 tokens of -softplus(N(0,1)): never kept
    drs = dr.cpu().sum(3).permute(0, 2, 1, 3, 4).reshape(B * H, NC, 64, E)
    assert orc.rel_l2(drs, rv["dr"]) < 1e-2
    # value-block images [token / 8][key row][token % 8] -> (key row, token), summed over the blocks, transposed
    img = dkg.cpu().float().permute(0, 1, 2, 3, 5, 4, 6).reshape(B, NC, H, -1, 128, 64).sum(3).transpose(-1, -2)
    dkg_sum = img.permute(0, 2, 1, 3, 4).reshape(B * H, NC, 64, 128)
    assert orc.rel_l2(dkg_sum, sg["dKg"]) < 1e-2


@pytest.mark.parametrize("E", [1, 2, 4, 8, 12, 16])
@pytest.mark.parametrize("dist", ["baseline", "mild"])
def test_state_grads_dense(E, dist):
    B, T, H = 1, 256, 2
    ins = orc.make_inputs(B, T, H, E, seed=300 + E, dist=dist)
    do = orc.make_grad_output((B, T, H, 128), 7)
    scale = 128 ** -0.5
    q, k, v, k2, q2, g, beta = _gpu(ins)
    dog = do.cuda()
    o, gc, AP, Pm, h, W, U = gj._kernel_forward(q, k, v, k2, q2, g, beta, scale, True)
    dV, dU, ds, dkg, dr = gj._run_reverse(q, k, dog, k2, q2, beta, gc, AP, Pm, U, scale)
    dkq, da, dc, dd = gj._run_state_grads(q, k, dog, dV, h, ds, dkg, k2, q2, gc, scale)
    assert _lib.device_status() == 0
    _, _, st = plan.run_plan(*ins, do, rounding=True)
    sg = st["sg"]
    NC = T // 64
    ch = lambda t: t.cpu().permute(0, 2, 1, 3, 4).reshape(B * H, NC, *t.shape[3:])
    # dkq is a bf16 image [column / 8][row][column % 8] per (batch, chunk, head): back to [row][column]
    dkq = dkq.float().permute(0, 1, 2, 4, 3, 5).reshape(B, NC, H, 128, 128)
    assert orc.rel_l2(ch(dkq)[:, :, :64], sg["dK"]) < 1e-2
    assert orc.rel_l2(ch(dkq)[:, :, 64:], sg["dQ"]) < 1e-2
    assert orc.rel_l2(ch(da), sg["da"]) < 1e-2
    assert orc.rel_l2(ch(dc), sg["dc"]) < 1e-2
    ddk = dd.cpu().permute(0, 2, 1, 3).reshape(B * H, NC, E)
    if dist == "baseline":
        assert (ddk == 0).all() and (sg["dd"] == 0).all()   # every chunk decay is below the threshold: no trace is taken
    else:
        assert orc.rel_l2(ddk, sg["dd"]) < 1e-2
