"""Packed-document metadata on the device, integer-exact against the CPU restatement."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib
from cute_triadic_gdn_b200.joint_packing import _metadata, chunk_capacity
from oracle import packing_oracle
from oracle.triadic_oracle import lognormal_documents

pytestmark = pytest.mark.gpu

CASES = [([0, 70, 133, 400, 640], 640), ([0, 64, 65, 320], 320), ([0, 512], 512),
         ([0, 17, 900, 901, 1500, 2999, 3000], 3000), ([0, 1], 1), ([0, 1, 2, 3, 4], 4)]


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("cu,T", CASES + [(lognormal_documents(131072, 5).tolist(), 131072)])
def test_metadata_exact(cu, T, dtype):
    dev = torch.tensor(cu, dtype=dtype, device="cuda")
    offsets, mapping, valid = _metadata(dev, T)
    o, start, rows, order, ok = packing_oracle.metadata(cu, T)
    n = len(cu) - 1
    assert mapping.shape == (3, chunk_capacity(T, n))
    assert bool(valid.item()) and ok
    assert offsets.cpu().tolist() == o.tolist()
    assert mapping[0].cpu().tolist() == start.tolist()
    assert mapping[1].cpu().tolist() == rows.tolist()
    assert mapping[2, :n].cpu().tolist() == order.tolist()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("cu,T", [([0, 70, 60, 640], 640), ([1, 70, 640], 640), ([0, 70, 600], 640), ([0, 70, 70, 640], 640)])
def test_bad_offsets_are_flagged_not_followed(cu, T):
    dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    canary = torch.full((3, chunk_capacity(T, len(cu) - 1) + 64), -7, dtype=torch.int32, device="cuda")
    _, _, valid = _metadata(dev, T)
    assert not bool(valid.item())
    assert (canary == -7).all()
