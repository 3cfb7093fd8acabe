"""The convolution with the layer glue fused in (`conv_split_norm_call`) against its f32 oracle: outputs to bf16 rounding,
gradients of x and weight against autograd through the oracle, packed documents, odd head counts (a channel tile that
straddles q | k), and the composition with the core."""
import pytest
import torch
import torch.nn.functional as F

from cute_triadic_gdn_b200 import _lib, conv_split_act_call, conv_split_norm_call, gdn_joint_call
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


def make(B, T, H, E, seed):
    gen = torch.Generator().manual_seed(seed)
    C = H * (3 * 128 + 2 * E)
    x = torch.randn(B, T, C, generator=gen).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, generator=gen)).to(torch.bfloat16)
    grads = [torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16) for _ in range(3)] + \
            [torch.randn(B, T, H, E, generator=gen) for _ in range(2)]
    return x, w, grads


@pytest.mark.parametrize("B,T,H,E,docs", [
    (2, 96, 2, 8, None),
    (1, 200, 3, 12, [0, 1, 5, 70, 133, 200]),       # odd head count: a 256-channel tile holds a q head and a k head
    (1, 131, 1, 4, [0, 64, 131]),
    (2, 40, 4, 16, None),
    (1, 77, 4, 1, [0, 3, 77]),
    (1, 64, 4, 2, None),
])
def test_fused_glue_against_oracle(B, T, H, E, docs):
    x, w, grads = make(B, T, H, E, 5 + E)
    cu = torch.tensor(docs, dtype=torch.int32) if docs else None
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    outs = conv_split_norm_call(xg, wg, H, E, None if cu is None else cu.cuda())
    torch.autograd.backward(outs, [g.cuda() for g in grads])
    assert _lib.device_status() == 0
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    refs = orc.glue_reference(xr, wr, H, E, cu)
    torch.autograd.backward(refs, [g.float() for g in grads])
    for name, a, r in zip(("q", "k", "v", "k2", "q2"), outs, refs):
        assert a.shape == r.shape and a.dtype == (torch.float32 if name in ("k2", "q2") else torch.bfloat16), name
        assert orc.rel_l2(a.detach().float().cpu(), r.detach()) < (1e-5 if name in ("k2", "q2") else 4e-3), name
    # the backward rounds the gradient of the convolution's output to bf16 once and recomputes SiLU' at the bf16-rounded
    # pre-activation, like the plain convolution's backward (tolerances of tests/test_conv_gpu.py, doubled for the extra pass)
    assert orc.rel_l2(xg.grad.float().cpu(), xr.grad) < 8e-3
    assert orc.rel_l2(wg.grad.float().cpu(), wr.grad) < 1.6e-2


def test_fused_glue_equals_the_unfused_pipeline_and_feeds_the_core():
    """The unfused pipeline (convolution, bf16 y, split, torch norms) and the fused call agree to the rounding of y."""
    T, H, E = 512, 2, 8
    x, w, _ = make(1, T, H, E, 11)
    cu = torch.tensor([0, 100, 320, 512], dtype=torch.int32).cuda()
    xd, wd = x.cuda(), w.cuda()
    with torch.no_grad():
        q, k, v, k2, q2 = conv_split_norm_call(xd, wd, H, E, cu)
        y = conv_split_act_call(xd, wd, 3 * H * 128, cu)
        yq, yk, yv, yk2, yq2 = y.split([H * 128, H * 128, H * 128, H * E, H * E], dim=-1)
        l2 = lambda t: t * torch.rsqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        uq, uk = (l2(t.float().view(1, T, H, 128)).to(torch.bfloat16) for t in (yq, yk))
        uk2, uq2 = (l2(F.softplus(t.float()).view(1, T, H, E)) for t in (yk2, yq2))
        for a, r in ((q, uq), (k, uk), (v, yv.view(1, T, H, 128)), (k2, uk2), (q2, uq2)):
            assert orc.rel_l2(a.float(), r.float()) < 6e-3
        g = -F.softplus(torch.randn(1, T, H, E, device="cuda"))
        beta = torch.sigmoid(torch.randn(1, T, H, device="cuda"))
        o = gdn_joint_call(q, k, v, k2, q2, g, beta, cu_seqlens=cu)
        o_u = gdn_joint_call(uq, uk, yv.reshape(1, T, H, 128).contiguous(), uk2, uq2, g, beta, cu_seqlens=cu)
    assert _lib.device_status() == 0
    assert orc.rel_l2(o.float(), o_u.float()) < 1.5e-2


def test_fused_glue_argument_checks():
    x, w, _ = make(1, 64, 2, 8, 3)
    with pytest.raises(ValueError):
        conv_split_norm_call(x.cuda(), w.cuda(), 2, 4)              # C does not match H, E
    with pytest.raises(ValueError):
        conv_split_norm_call(x.cuda(), w.cuda(), 2, 8, torch.tensor([0, 64], dtype=torch.int32))   # offsets on the host
