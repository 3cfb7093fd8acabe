"""Host-resident pipeline: same bits as one device-resident call over the whole batch."""
import pytest
import torch

from cute_triadic_gdn_b200 import HostPipeline, _lib, gdn_joint_call, gdn_joint_host
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


def _direct(ins, do):
    leaves = [t.cuda().requires_grad_(True) for t in ins]
    o = gdn_joint_call(*leaves)
    o.backward(do.cuda())
    return [o.detach().cpu()] + [t.grad.cpu() for t in leaves]


@pytest.mark.parametrize("B,T,H,E,slices", [(4, 512, 2, 8, 4), (4, 256, 4, 4, 2), (3, 256, 2, 16, 3), (2, 256, 2, 1, 1)])
def test_pipeline_matches_direct_call(B, T, H, E, slices):
    ins = [t.pin_memory() for t in orc.make_inputs(B, T, H, E, seed=50 + E)]
    do = orc.make_grad_output((B, T, H, 128), 9).pin_memory()
    ref = _direct(ins, do)
    pipe = HostPipeline(ins, do, slices=slices)
    for _ in range(3):                                  # buffers are reused from step to step
        o, grads = pipe.run(ins, do)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        for a, b in zip([o] + grads, ref):
            assert torch.equal(a, b)
    assert pipe.h2d_bytes == sum(t.numel() * t.element_size() for t in ins) + do.numel() * do.element_size()


def test_forward_only_and_argument_checks():
    ins = [t.pin_memory() for t in orc.make_inputs(2, 256, 2, 8, seed=3)]
    o, grads = gdn_joint_host(*ins, slices=2)
    assert grads is None
    ref = gdn_joint_call(*[t.cuda() for t in ins]).cpu()
    assert torch.equal(o, ref)
    with pytest.raises(ValueError):
        HostPipeline(ins, slices=3)                     # does not divide the batch
    with pytest.raises(ValueError):
        HostPipeline([t.clone() for t in ins])          # pageable, not pinned
    with pytest.raises(ValueError):
        HostPipeline([t.cuda() for t in ins])           # not host tensors


def test_packed_row_is_cut_along_documents():
    T, H, E = 1536, 2, 8
    cu = torch.tensor([0, 100, 612, 613, 1000, 1536], dtype=torch.int32)
    ins = [t.pin_memory() for t in orc.make_inputs(1, T, H, E, seed=77)]
    do = orc.make_grad_output((1, T, H, 128), 5).pin_memory()
    leaves = [t.cuda().requires_grad_(True) for t in ins]
    o = gdn_joint_call(*leaves, cu_seqlens=cu.cuda())
    o.backward(do.cuda())
    ref = [o.detach().cpu()] + [t.grad.cpu() for t in leaves]
    pipe = HostPipeline(ins, do, slices=3, cu_seqlens=cu)
    assert 1 <= pipe.slices <= 3
    for _ in range(2):
        oh, grads = pipe.run(ins, do)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        for a, b in zip([oh] + grads, ref):
            assert torch.equal(a, b)
