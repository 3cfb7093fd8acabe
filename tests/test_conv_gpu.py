"""conv_split_act on the device against the CPU oracle and the stored outputs of the reference's kernels."""
import numpy as np
import pytest
import torch

from cute_triadic_gdn_b200 import _lib, conv_split_act_call
from oracle import triadic_oracle as orc
from helpers import bf16, conv_files

pytestmark = pytest.mark.gpu


def _run(x, w, act, dy, cu):
    xg = x.cuda().requires_grad_(True)
    wg = w.cuda().requires_grad_(True)
    y = conv_split_act_call(xg, wg, act, None if cu is None else cu.cuda())
    y.backward(dy.cuda())
    assert _lib.device_status() == 0
    return y.detach().cpu(), xg.grad.cpu(), wg.grad.cpu()


def _check(x, w, act, dy, cu):
    y, dx, dw = _run(x, w, act, dy, cu)
    y32 = orc.conv_reference(x, w, act, cu, rounded=False)
    ry = y32.to(torch.bfloat16)
    # bit-exact up to f32 summation order: allow one bf16 step where the f32 value sits on a rounding boundary
    step = 2.0 ** -7 * ry.float().abs() + 1e-30
    assert ((y.float() - ry.float()).abs() <= step).all()
    assert (y == ry).float().mean() > 0.995
    rdx, rdw = orc.conv_reference_backward(x, w, act, dy, cu)
    assert orc.rel_l2(dx.float(), rdx.float()) < 4e-3
    assert orc.rel_l2(dw.float(), rdw.float()) < 8e-3


@pytest.mark.parametrize("path", conv_files())
def test_conv_golden(path):
    z = np.load(path)
    cu = torch.from_numpy(z["cu_seqlens"]) if "cu_seqlens" in z.files else None
    _check(bf16(z["x"]), bf16(z["w"]), int(z["act"]), bf16(z["dy"]), cu)


@pytest.mark.parametrize("B,T,C,act,docs", [
    (2, 513, 264, 200, None),
    (1, 1, 8, 8, None),
    (1, 1000, 1032, 520, [0, 1, 2, 5, 300, 301, 999, 1000]),
    (3, 64, 1024, 0, None),
    (1, 700, 128, 128, [0, 700]),
])
def test_conv_shapes(B, T, C, act, docs):
    g = torch.Generator().manual_seed(T + C)
    x = torch.randn(B, T, C, generator=g).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, generator=g)).to(torch.bfloat16)
    dy = torch.randn(B, T, C, generator=g).to(torch.bfloat16)
    cu = None if docs is None else torch.tensor(docs, dtype=torch.int32)
    _check(x, w, act, dy, cu)


def test_conv_at_the_channel_count_of_the_triadic_layer():
    """C = 32 * (3 * 128 + 2 * 12) = 13056 channels with SiLU on the first 12288, packed documents, a few hundred tokens."""
    C, act, T = 13056, 12288, 300
    g = torch.Generator().manual_seed(C)
    x = torch.randn(1, T, C, generator=g).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, generator=g)).to(torch.bfloat16)
    dy = torch.randn(1, T, C, generator=g).to(torch.bfloat16)
    _check(x, w, act, dy, torch.tensor([0, 1, 70, 71, 200, 300], dtype=torch.int32))


def test_conv_strided_input_and_linearity():
    g = torch.Generator().manual_seed(3)
    big = torch.randn(2, 300, 512, generator=g).to(torch.bfloat16).cuda()
    x = big[:, :, 128:384]                               # channel slice: row stride 512, 16-byte aligned
    w = (0.5 * torch.randn(256, 4, generator=g)).to(torch.bfloat16).cuda()
    y = conv_split_act_call(x, w, 0)
    y2 = conv_split_act_call(x.contiguous(), w, 0)
    assert torch.equal(y, y2)
    # without activation the map is linear in the weights: conv(x, 2w) == 2 conv(x, w) exactly in bf16
    assert torch.equal(conv_split_act_call(x, (2 * w.float()).to(torch.bfloat16), 0).float(), 2 * y.float())
