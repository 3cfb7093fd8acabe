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


@pytest.mark.parametrize("cu,T", [([0, 70, 60, 640], 640), ([1, 70, 640], 640), ([0, 70, 600], 640), ([0, 70, 70, 640], 640),
                                  ([0, 100000, 640], 640), ([0, -5, 640], 640)])
def test_bad_offsets_are_flagged_not_followed(cu, T):
    """Offsets that do not start at 0, end at T and strictly increase: the kernel must say so and must not write outside
    the buffers it was given.  The buffers are carved out of larger ones filled with a marker, and the library is called
    through its C ABI directly, so every byte around them can be checked."""
    import ctypes
    n = len(cu) - 1
    cap = chunk_capacity(T, n)
    dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    PAD = 256
    big_map = torch.full((PAD + 3 * cap + PAD,), -7, dtype=torch.int32, device="cuda")
    big_off = torch.full((PAD + n + 1 + PAD,), -7, dtype=torch.int32, device="cuda")
    big_val = torch.full((PAD + 16 + PAD,), 0x55, dtype=torch.uint8, device="cuda")
    mapping, offsets, valid = big_map[PAD:PAD + 3 * cap], big_off[PAD:PAD + n + 1], big_val[PAD:PAD + 1]
    rc = _lib.lib.tgdn_metadata(ctypes.c_void_p(dev.data_ptr()), 0, n, T, ctypes.c_void_p(offsets.data_ptr()),
                                ctypes.c_void_p(mapping.data_ptr()), cap, ctypes.c_void_p(valid.data_ptr()),
                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert valid.item() == 0
    assert (big_map[:PAD] == -7).all() and (big_map[PAD + 3 * cap:] == -7).all()
    assert (big_off[:PAD] == -7).all() and (big_off[PAD + n + 1:] == -7).all()
    assert (big_val[:PAD] == 0x55).all() and (big_val[PAD + 1:] == 0x55).all()
    # entries the kernel did write (documents it could still place) never point outside the row
    start, rows = mapping[:cap], mapping[cap:2 * cap]
    wrote = rows != -7
    assert ((rows[wrote] >= 0) & (rows[wrote] <= 64)).all()
    assert ((start[wrote] >= 0) & (start[wrote] + rows[wrote] <= T) | (rows[wrote] == 0)).all()
    assert _lib.device_status() == 0
