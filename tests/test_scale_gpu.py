"""Larger configurations and size-independent properties of the kernels.

Shapes follow the benchmark configurations at reduced size (the CPU oracle has to finish in seconds): packed lognormal
documents with E=16, the convolution pre-pass feeding the core with E=12 and eight equal documents, and a long dense row.
Properties that hold at any size: a (batch row, head) slice computed alone is bitwise equal to the same slice of the full
problem; a packed row of whole-chunk documents is bitwise equal to the same documents as batch rows."""
import pytest
import torch
import torch.nn.functional as F

from cute_triadic_gdn_b200 import _lib, chunk_gdn_joint, conv_split_act_call, gdn_joint_call
from oracle import triadic_oracle as orc
from helpers import GRADS

pytestmark = pytest.mark.gpu


def run(fn, inputs, do, cu):
    leaves = [t.detach().clone().cuda().requires_grad_(True) for t in inputs]
    o = fn(*leaves, cu_seqlens=None if cu is None else cu.cuda())
    o.backward(do.cuda())
    return o.detach(), [t.grad for t in leaves]


def test_packed_lognormal_documents_e16():
    T, H, E = 12288, 2, 16
    cu = orc.lognormal_documents(T, seed=11, median=700.0)
    ins = orc.make_inputs(1, T, H, E, seed=21)
    do = orc.make_grad_output((1, T, H, 128), 22)
    o, grads = run(gdn_joint_call, ins, do, cu)
    assert _lib.device_status() == 0
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, ins, do, cu_seqlens=cu, dtype=torch.float32)
    assert orc.rel_l2(o.float().cpu(), o_ref) < 1e-2
    for n, a, b in zip(GRADS, grads, g_ref):
        assert orc.rel_l2(a.float().cpu(), b) < 2e-2, n


def test_conv_prepass_feeds_core_e12():
    """x -> conv_split_act -> split [q|k|v|k2|q2] -> l2-normalise -> core, eight equal documents; gradients reach x and w."""
    T, H, E = 2048, 2, 12
    C, act = H * (3 * 128 + 2 * E), 3 * H * 128
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(1, T, C, generator=gen).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, generator=gen)).to(torch.bfloat16)
    g = -F.softplus(torch.randn(1, T, H, E, generator=gen))
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen))
    do = orc.make_grad_output((1, T, H, 128), 23)
    cu = torch.arange(0, T + 1, T // 8, dtype=torch.int32)

    def split(y):
        q, k, v, k2, q2 = y.split([H * 128, H * 128, H * 128, H * E, H * E], dim=-1)
        n = lambda t, d: t.float().view(1, T, H, d)
        l2 = lambda t: t * torch.rsqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        return (l2(n(q, 128)).to(torch.bfloat16), l2(n(k, 128)).to(torch.bfloat16), n(v, 128).to(torch.bfloat16),
                l2(n(k2, E)), l2(n(q2, E)))

    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    gg, bg = g.cuda().requires_grad_(True), beta.cuda().requires_grad_(True)
    y = conv_split_act_call(xg, wg, act, cu.cuda())
    q, k, v, k2, q2 = split(y)
    o = gdn_joint_call(q.contiguous(), k.contiguous(), v.contiguous(), k2.contiguous(), q2.contiguous(), gg, bg,
                       cu_seqlens=cu.cuda())
    o.backward(do.cuda())
    assert _lib.device_status() == 0
    # oracle: the same glue on the CPU around the conv and core oracles, differentiated by autograd up to the output of the
    # convolution (the casts to bf16 pass gradients through), then the convolution's own backward oracle
    y_ref = orc.conv_reference(x, w, act, cu)
    yl = y_ref.float().requires_grad_(True)
    gl, bl = g.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    qr, kr, vr, k2r, q2r = split(yl)
    o_ref = orc.chunk_reference(qr, kr, vr, k2r, q2r, gl, bl, cu_seqlens=cu, dtype=torch.float32)
    assert orc.rel_l2(o.float().cpu(), o_ref.detach()) < 1.5e-2
    o_ref.backward(do.float())
    dx_ref, dw_ref = orc.conv_reference_backward(x, w, act, yl.grad.to(torch.bfloat16), cu)
    assert orc.rel_l2(gg.grad.cpu(), gl.grad) < 2e-2
    assert orc.rel_l2(bg.grad.cpu(), bl.grad) < 2e-2
    assert orc.rel_l2(xg.grad.float().cpu(), dx_ref.float()) < 2e-2
    assert orc.rel_l2(wg.grad.float().cpu(), dw_ref.float()) < 2e-2


def test_long_dense_row_slice_against_oracle_and_slice_independence():
    B, T, H, E = 2, 8192, 4, 8
    ins = orc.make_inputs(B, T, H, E, seed=31)
    do = orc.make_grad_output((B, T, H, 128), 32)
    o, grads = run(gdn_joint_call, ins, do, None)
    b, h = 1, 3
    sl = [t[b:b + 1, :, h:h + 1].contiguous() for t in ins]
    dsl = do[b:b + 1, :, h:h + 1].contiguous()
    o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, sl, dsl, dtype=torch.float32)
    assert orc.rel_l2(o[b:b + 1, :, h:h + 1].float().cpu(), o_ref) < 1e-2
    for n, a, r in zip(GRADS, grads, g_ref):
        assert orc.rel_l2(a[b:b + 1, :, h:h + 1].float().cpu(), r) < 2e-2, n
    # the slice computed on its own is bitwise the slice of the full problem
    o1, g1 = run(gdn_joint_call, sl, dsl, None)
    assert torch.equal(o1, o[b:b + 1, :, h:h + 1])
    for a, full in zip(g1, grads):
        assert torch.equal(a, full[b:b + 1, :, h:h + 1])
    assert _lib.device_status() == 0


@pytest.mark.parametrize("E", [2, 8, 16])
def test_packed_whole_chunk_documents_equal_batch_rows(E):
    N, T0, H = 3, 192, 2
    ins = orc.make_inputs(N, T0, H, E, seed=41 + E)
    do = orc.make_grad_output((N, T0, H, 128), 42)
    o_d, g_d = run(chunk_gdn_joint, ins, do, None)
    packed = [t.reshape(1, N * T0, *t.shape[2:]).contiguous() for t in ins]
    cu = torch.arange(0, N * T0 + 1, T0, dtype=torch.int32)
    o_p, g_p = run(chunk_gdn_joint, packed, do.reshape(1, N * T0, H, 128), cu)
    assert torch.equal(o_p.view_as(o_d), o_d)
    for a, b in zip(g_p, g_d):
        assert torch.equal(a.view_as(b), b)
