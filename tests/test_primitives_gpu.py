"""tcgen05 / TMA building blocks on the device: one product per operand-layout pair, and a tensor-map tile load."""
import ctypes

import numpy as np
import pytest
import torch

from cute_triadic_gdn_b200 import _lib

pytestmark = pytest.mark.gpu
NAMES = ["sw128-K", "sw128-MN", "plain-K", "plain-MN"]


def _run(M, N, K, la, lb, seed=0):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(K, N, generator=g).to(torch.bfloat16).cuda()
    D = torch.full((128, N), float("nan"), device="cuda")
    _lib.check(_lib.lib.tgdn_selftest_mma(_lib.ptr(A), _lib.ptr(B), _lib.ptr(D), M, N, K, la, lb, _lib.stream_of(A)),
               "selftest_mma")
    assert _lib.device_status() == 0
    return A, B, D


@pytest.mark.parametrize("la", range(4))
@pytest.mark.parametrize("lb", range(4))
@pytest.mark.parametrize("N,K", [(64, 128), (128, 64), (32, 64), (16, 256)])
def test_mma_layouts(la, lb, N, K):
    A, B, D = _run(128, N, K, la, lb, seed=la * 4 + lb)
    ref = A.float() @ B.float()
    err = (D - ref).abs().max().item()
    assert err < 1e-2 * ref.abs().max().item(), f"A {NAMES[la]} B {NAMES[lb]}: max err {err}"


def test_m64_rows_live_in_documented_lanes():
    """Where a 64-row product leaves its rows in tensor memory (reported, and pinned to what the kernels assume)."""
    A, B, D = _run(64, 32, 64, 0, 0, seed=5)
    ref = (A.float() @ B.float())
    base = torch.zeros(128, 32, device="cuda")
    base[:64] = ref
    extra = (D - base).cpu()
    refc = ref.cpu()
    lanes = {}
    for lane in range(128):
        if extra[lane].abs().max() < 1e-3:
            continue
        d = (refc - extra[lane][None]).abs().amax(1)
        lanes[lane] = int(d.argmin()) if d.min() < 1e-2 else -1
    print("M=64 lane -> row:", lanes)
    assert len(lanes) == 64


def test_tma_tile_and_bulk_copy():
    B, T, H = 2, 200, 3
    x = torch.randn(B, T, H, 128).to(torch.bfloat16).cuda()
    bulk = torch.arange(4096, dtype=torch.uint8).cuda()
    out = torch.zeros(8192 + 4096, dtype=torch.uint8, device="cuda")
    col0, head, tok0, batch = 64, 1, 150, 1      # rows 150..213: the last 14 lie past T and must read as zero
    _lib.check(_lib.lib.tgdn_selftest_tma(_lib.ptr(x), B, T, H, col0, head, tok0, batch, _lib.ptr(bulk), 4096,
                                          _lib.ptr(out), _lib.stream_of(x)), "selftest_tma")
    assert _lib.device_status() == 0
    img = out[:8192].cpu().numpy().view(np.uint16)
    want = np.zeros(4096, dtype=np.uint16)
    xs = x.cpu().view(torch.int16).numpy().view(np.uint16)
    for r in range(64):
        for c in range(64):
            off = r * 128 + ((((c >> 3) ^ r) & 7) << 4) + ((c & 7) << 1)
            want[off // 2] = xs[batch, tok0 + r, head, col0 + c] if tok0 + r < T else 0
    assert (img == want).all()
    assert (out[8192:].cpu() == bulk.cpu()).all()
