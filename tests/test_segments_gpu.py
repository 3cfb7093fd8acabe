"""Sequences processed in segments chained by their recurrent state, forward AND backward, on one GPU.

`chunk_gdn_joint_segment` hands the f32 state out of a segment and into the next, and the gradient of the state the other
way (tgdn_fwd_state, tgdn_bwd_recurrent_state).  Both travel in f32, which is what the unsplit kernels carry across a
chunk boundary in registers: outputs and all seven gradients of the chained run must be BITWISE those of the unsplit run."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib, gdn_joint_call
from cute_triadic_gdn_b200.gdn_joint import chunk_gdn_joint_segment
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,dist", [(1, "mild"), (4, "baseline"), (8, "mild"), (8, "baseline"), (12, "mild"), (16, "mild")])
def test_chained_segments_equal_the_unsplit_run(E, dist):
    B, T, H = 2, 384, 2
    ins = orc.make_inputs(B, T, H, E, seed=40 + E, dist=dist)
    do = orc.make_grad_output((B, T, H, 128), 41).cuda()
    whole = [t.cuda().requires_grad_(True) for t in ins]
    o_ref = gdn_joint_call(*whole)
    o_ref.backward(do)
    cuts = [0, 128, 192, 384]                      # three segments of different lengths
    leaves = [t.cuda().requires_grad_(True) for t in ins]
    state, outs = None, []
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        o, state = chunk_gdn_joint_segment(*[t[:, lo:hi].contiguous() for t in leaves], state_in=state)
        outs.append(o)
    o = torch.cat(outs, 1)
    o.backward(do)                                 # the last state_out is unused: its gradient arrives as None
    assert _lib.device_status() == 0
    assert torch.equal(o, o_ref)
    for name, a, b in zip("q k v k2 q2 g beta".split(), leaves, whole):
        assert torch.equal(a.grad, b.grad), name


def test_gradient_reaches_the_initial_state_and_leaves_the_final_one():
    """dL/d(state_in) against autograd through the f64 token-by-token definition on a short sequence."""
    B, T, H, E = 1, 64, 1, 2
    ins = orc.make_inputs(B, T, H, E, seed=9, dist="mild")
    gen = torch.Generator().manual_seed(10)
    s0 = 0.1 * torch.randn(B, H, E, 128, 128, generator=gen)
    do = orc.make_grad_output((B, T, H, 128), 11)
    ds_out = 0.01 * torch.randn(B, H, E, 128, 128, generator=gen)
    leaves = [t.cuda().requires_grad_(True) for t in ins]
    s_in = s0.cuda().requires_grad_(True)
    o, s_out = chunk_gdn_joint_segment(*leaves, state_in=s_in)
    torch.autograd.backward([o, s_out], [do.cuda(), ds_out.cuda()])
    assert _lib.device_status() == 0
    # the definition, f64
    q, k, v, k2, q2, g, beta = (t.double().requires_grad_(True) for t in ins)
    S = s0.double().requires_grad_(True)
    S0 = S
    rows = []
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        kap = k2[:, t, :, :, None] * k[:, t, :, None, :]
        pred = torch.einsum('bhed,bhedv->bhv', kap, S)
        S = S + beta[:, t, :, None, None, None] * kap[..., None] * (v[:, t] - pred)[:, :, None, None, :]
        rows.append(torch.einsum('bhed,bhedv->bhv', q2[:, t, :, :, None] * q[:, t, :, None, :], S) * 128 ** -0.5)
    o_ref = torch.stack(rows, 1)
    torch.autograd.backward([o_ref, S], [do.double(), ds_out.double()])
    assert orc.rel_l2(o.float().cpu(), o_ref.detach().float()) < 1e-2
    assert orc.rel_l2(s_out.detach().cpu().double(), S.detach()) < 1e-2
    assert orc.rel_l2(s_in.grad.cpu().double(), S0.grad) < 2e-2
    for name, a, b in zip("q k v k2 q2 g beta".split(), leaves, (q, k, v, k2, q2, g, beta)):
        assert orc.rel_l2(a.grad.float().cpu(), b.grad.float()) < 2e-2, name


@pytest.mark.parametrize("E", [4, 8, 16])
def test_checkpointed_backward_is_bitwise_and_saves_memory(E):
    """`checkpoint_tokens`: the backward recomputes each segment from the state at its start; same bits, less memory."""
    from cute_triadic_gdn_b200 import chunk_gdn_joint
    B, T, H = 2, 1024, 4
    ins = orc.make_inputs(B, T, H, E, seed=60 + E, dist="mild")
    do = orc.make_grad_output((B, T, H, 128), 61).cuda()

    def run(**kw):
        leaves = [t.cuda().requires_grad_(True) for t in ins]
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        o = chunk_gdn_joint(*leaves, **kw)
        held = torch.cuda.memory_allocated() - base           # what the forward keeps for the backward (plus o)
        o.backward(do)
        return o.detach(), [t.grad for t in leaves], held

    o_ref, g_ref, held_ref = run()
    o_ck, g_ck, held_ck = run(checkpoint_tokens=256)
    assert _lib.device_status() == 0
    assert torch.equal(o_ck, o_ref)
    for a, b in zip(g_ck, g_ref):
        assert torch.equal(a, b)
    assert held_ck < 0.6 * held_ref, (held_ck, held_ref)
    with pytest.raises(ValueError):
        chunk_gdn_joint(*[t.cuda().requires_grad_(True) for t in ins], checkpoint_tokens=100)
