"""Masks and forward recurrence on the device, stage by stage against the torch model of the kernels' dataflow and
end to end against the CPU oracle."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib
from cute_triadic_gdn_b200.gdn_joint import _kernel_forward, chunk_gates
from oracle import kernel_plan as plan
from oracle import triadic_oracle as orc
from plan_helpers import decode_items, image_to_matrix, state_to_matrix

pytestmark = pytest.mark.gpu


def _gpu(ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("E", [1, 2, 4, 8, 12, 16])
@pytest.mark.parametrize("dist", ["baseline", "mild"])
def test_forward_stages_dense(E, dist):
    B, T, H = 2, 256, 2
    ins = orc.make_inputs(B, T, H, E, seed=100 + E, dist=dist)
    do = orc.make_grad_output((B, T, H, 128), 7)
    scale = 128 ** -0.5
    o, gc, AP, Pm, h, W, U = _kernel_forward(*_gpu(ins), scale, True)
    assert _lib.device_status() == 0
    _, _, st = plan.run_plan(*ins, do, rounding=True)
    mk, fw = st["masks"], st["fwd"]
    # masks
    gcc = chunk_gates(gc, E).cpu()                                                 # (B, NC, H, 64, E)
    gcp = gcc.permute(0, 2, 1, 3, 4).reshape(B * H, T // 64, 64, E)
    assert orc.rel_l2(gcp, mk["gc"]) < 1e-5
    # the gate factors behind gc: a = k2 exp(gc), r = k2 exp(gL - gc), c = scale q2 exp(gc), then d = exp(gL) padded to 16
    per_chunk = lambda x: x.reshape(B, T // 64, 64, H, E).permute(0, 1, 3, 2, 4)
    k2c, q2c = per_chunk(ins[3]), per_chunk(ins[4])
    fac = gc.cpu()[..., 64 * E:256 * E].unflatten(-1, (3, 64, E))
    assert orc.rel_l2(fac[..., 0, :, :], k2c * gcc.exp()) < 1e-5
    assert orc.rel_l2(fac[..., 1, :, :], k2c * (gcc[..., 63:64, :] - gcc).exp()) < 1e-5
    assert orc.rel_l2(fac[..., 2, :, :], scale * q2c * gcc.exp()) < 1e-5
    dpad = gc.cpu()[..., 256 * E:]
    assert dpad.shape[-1] == 16 and orc.rel_l2(dpad[..., :E], gcc[..., 63, :].exp()) < 1e-5 and not dpad[..., E:].any()
    A = decode_items(AP.cpu().float(), lambda x: image_to_matrix(x, 128, 64, 128, 2048))
    assert orc.rel_l2(A[:, :, :64], mk["A"]) < 4e-3
    assert orc.rel_l2(A[:, :, 64:], mk["PA"]) < 4e-3
    Pmm = decode_items(Pm.cpu().float(), lambda x: image_to_matrix(x, 64, 64, 128, 1024))
    assert orc.rel_l2(Pmm, mk["Pm"]) < 4e-3
    # forward recurrence
    conv = lambda t: t.cpu().float().permute(0, 2, 1, 3, 4).reshape(B * H, T // 64, 64, 128)
    assert orc.rel_l2(conv(W), fw["W"]) < 6e-3
    assert orc.rel_l2(conv(U), fw["U"]) < 6e-3
    hm = decode_items(h.cpu().float(), state_to_matrix)
    assert orc.rel_l2(hm, fw["h"]) < 8e-3
    o_ref = orc.chunk_reference(*ins, dtype=torch.float32)
    assert orc.rel_l2(o.cpu().float(), o_ref) < 1e-2
