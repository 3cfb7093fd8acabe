"""The torch.library registrations: fake (meta) kernels on the CPU, one graph node per call under torch.compile on a GPU.

Reference contract: cute_triadic_gdn/ops/joint_torch_ops.py:8-95 (one forward node, one backward node, fakes that depend
only on the input shapes), cute_triadic_gdn/ops/joint_packing.py:10-62 (metadata sizes depend only on T and N)."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import cute_triadic_gdn_b200  # noqa: F401  (registers the ops)
from cute_triadic_gdn_b200.joint_packing import chunk_capacity


def _fake_inputs(B, T, H, E):
    dev = "cuda"
    q = torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=dev)
    k2 = torch.empty(B, T, H, E, device=dev)
    return [q, torch.empty_like(q), torch.empty_like(q), k2, torch.empty_like(k2), torch.empty_like(k2),
            torch.empty(B, T, H, device=dev)]


@pytest.mark.parametrize("E", [1, 8, 16])
def test_fake_kernels_give_the_real_shapes_dense(E):
    B, T, H, NC = 2, 256, 4, 4
    with FakeTensorMode():
        ins = _fake_inputs(B, T, H, E)
        o, gc, AP, Pm, h, W, U = torch.ops.tgdn_b200.joint_fwd(*ins, 128 ** -0.5, None, None)
        assert o.shape == (B, T, H, 128) and o.dtype == torch.bfloat16 and o.device.type == "cuda"
        assert gc.shape == (B, NC, H, 256 * E + 16) and gc.dtype == torch.float32
        assert AP.numel() == B * NC * H * 128 * 64 and Pm.numel() == B * NC * H * 64 * 64
        assert h.shape == (B, NC, H, E, 16, 128, 8) and W.shape == U.shape == (B, NC, H, 64, 128)
        saved = list(ins[:2]) + list(ins[3:]) + [gc, AP, Pm, h, W, U]
        grads = torch.ops.tgdn_b200.joint_bwd(saved, torch.empty_like(o), 128 ** -0.5, None, None)
        assert [g.shape for g in grads] == [t.shape for t in ins]
        assert [g.dtype for g in grads] == [t.dtype for t in ins]


def test_fake_kernels_packed_sizes_depend_only_on_tokens_and_documents():
    T, H, E, N = 1000, 2, 4, 5
    cap = chunk_capacity(T, N)
    with FakeTensorMode():
        cu = torch.empty(N + 1, dtype=torch.int32, device="cuda")
        offsets, mapping, valid = torch.ops.tgdn_b200.joint_metadata(cu, T)
        assert offsets.shape == (N + 1,) and mapping.shape == (3, cap) and valid.shape == (1,)
        ins = _fake_inputs(1, T, H, E)
        o, gc, AP, Pm, h, W, U = torch.ops.tgdn_b200.joint_fwd(*ins, 0.1, offsets, mapping)
        assert o.shape == (1, T, H, 128) and gc.shape == (1, cap, H, 256 * E + 16) and h.shape[1] == cap


def test_fake_conv():
    with FakeTensorMode():
        x = torch.empty(2, 512, 256, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(256, 4, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.tgdn_b200.conv_split_act_fwd(x, w, 128, None)
        assert y.shape == x.shape and y.dtype == torch.bfloat16
        dx, dw = torch.ops.tgdn_b200.conv_split_act_bwd(x, torch.empty_like(x), w, 128, None)
        assert dx.shape == x.shape and dw.shape == w.shape


@pytest.mark.gpu
def test_one_node_per_call_under_torch_compile():
    """fullgraph tracing must succeed (no graph break) and see exactly one forward node; results equal eager bitwise."""
    from cute_triadic_gdn_b200 import conv_split_act_call, gdn_joint_call
    from oracle import triadic_oracle as orc
    seen = []

    def backend(gm, example_inputs):
        seen.append([str(n.target) for n in gm.graph.nodes if n.op == "call_function"])
        return gm.forward

    ins = [t.cuda() for t in orc.make_inputs(2, 256, 2, 8, seed=1)]
    fn = torch.compile(lambda *a: gdn_joint_call(*a), backend=backend, fullgraph=True)
    with torch.no_grad():
        out = fn(*ins)
        ref = gdn_joint_call(*ins)
    assert torch.equal(out, ref)
    calls = [t for t in seen[0] if "tgdn_b200" in t]
    assert len(calls) == 1 and "joint_fwd" in calls[0]

    seen.clear()
    x = torch.randn(1, 512, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(256, 4, device="cuda").to(torch.bfloat16)
    cfn = torch.compile(lambda a, b: conv_split_act_call(a, b, 128), backend=backend, fullgraph=True)
    with torch.no_grad():
        assert torch.equal(cfn(x, w), conv_split_act_call(x, w, 128))
    calls = [t for t in seen[0] if "tgdn_b200" in t]
    assert len(calls) == 1 and "conv_split_act_fwd" in calls[0]


@pytest.mark.gpu
def test_compiled_training_step_matches_eager():
    """Forward + backward through torch.compile (aot_eager: the autograd registration is traced too)."""
    from cute_triadic_gdn_b200 import gdn_joint_call
    from oracle import triadic_oracle as orc
    ins = orc.make_inputs(1, 256, 2, 4, seed=2)
    do = orc.make_grad_output((1, 256, 2, 128), 3).cuda()

    def step(fn):
        leaves = [t.cuda().requires_grad_(True) for t in ins]
        o = fn(*leaves)
        o.backward(do)
        return [o.detach()] + [t.grad for t in leaves]

    eager = step(gdn_joint_call)
    compiled = step(torch.compile(gdn_joint_call, backend="aot_eager", fullgraph=True))
    for a, b in zip(compiled, eager):
        assert torch.equal(a, b)
