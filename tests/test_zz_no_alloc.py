"""tgdn_conv_bwd_static: the convolution backward for hosts that are not allowed to allocate device memory.

Such a host (a server with a fixed, externally owned arena, or a thread on which cudaMalloc is off limits) cannot hand
the library the scratch buffer that tgdn_conv_bwd asks for; the static variant keeps its weight-gradient partials in an
array built into the library.  The test drives both entry points through the C ABI on the same inputs, twice in a row
with different sizes (the array keeps the first call's contents), and expects identical results; it also checks that a
problem too large for the array is refused with its own error code.  Collected last on purpose.
"""
import ctypes

import pytest
import torch

from cute_triadic_gdn_b200 import _lib

pytestmark = pytest.mark.gpu
STATIC_BYTES = 8 << 20


def _both(B, T, C, act, docs, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, C, generator=g).to(torch.bfloat16).cuda()
    w = (0.5 * torch.randn(C, 4, generator=g)).to(torch.bfloat16).cuda()
    dy = torch.randn(B, T, C, generator=g).to(torch.bfloat16).cuda()
    cu = None if docs is None else torch.tensor(docs, dtype=torch.int32, device="cuda")
    n_docs = 0 if docs is None else len(docs) - 1
    L, p = _lib.lib, _lib.ptr
    nbytes = L.tgdn_conv_bwd_scratch_bytes(B, T, C)
    assert nbytes <= STATIC_BYTES
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
    dx_b, dw_b = torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
    stream = _lib.stream_of(x)
    _lib.check(L.tgdn_conv_bwd(p(x), p(w), p(dy), p(dx_a), p(dw_a), p(cu), n_docs, B, T, C, x.stride(0), x.stride(1),
                               dy.stride(0), dy.stride(1), act, p(scratch), nbytes, stream), "tgdn_conv_bwd")
    _lib.check(L.tgdn_conv_bwd_static(p(x), p(w), p(dy), p(dx_b), p(dw_b), p(cu), n_docs, B, T, C, x.stride(0), x.stride(1),
                                      dy.stride(0), dy.stride(1), act, stream), "tgdn_conv_bwd_static")
    torch.cuda.synchronize()
    return dx_a, dw_a, dx_b, dw_b


def test_static_scratch_variant_matches_two_calls_in_a_row():
    # first a larger problem, then a smaller one that reuses (part of) the array with the first call's leftovers in it
    for (B, T, C, act, docs, seed) in [(2, 1500, 520, 264, None, 1), (1, 300, 64, 64, [0, 1, 130, 300], 2)]:
        dx_a, dw_a, dx_b, dw_b = _both(B, T, C, act, docs, seed)
        assert torch.equal(dx_a, dx_b)            # same kernels, same summation order: bit-identical
        assert torch.equal(dw_a, dw_b)
        assert torch.isfinite(dw_b.float()).all()
    assert _lib.device_status() == 0


def test_static_scratch_variant_allocates_nothing_after_its_first_call():
    """The point of the entry: once the first call on the device has loaded the library's module and looked the array up,
    a call leaves the amount of free device memory exactly as it found it (the caller's own tensors are made before)."""
    g = torch.Generator().manual_seed(5)
    B, T, C, act = 1, 700, 256, 128
    x = torch.randn(B, T, C, generator=g).to(torch.bfloat16).cuda()
    w = (0.5 * torch.randn(C, 4, generator=g)).to(torch.bfloat16).cuda()
    dy = torch.randn(B, T, C, generator=g).to(torch.bfloat16).cuda()
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    L, p = _lib.lib, _lib.ptr
    stream = _lib.stream_of(x)
    call = lambda: L.tgdn_conv_bwd_static(p(x), p(w), p(dy), p(dx), p(dw), None, 0, B, T, C, x.stride(0), x.stride(1),
                                          dy.stride(0), dy.stride(1), act, stream)
    assert call() == 0                                        # warm-up: module load and address lookup
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert _lib.device_status() == 0


def test_static_scratch_variant_refuses_oversized_problems():
    L = _lib.lib
    fake = ctypes.c_void_p(4096)
    B, T, C = 48, 4096, 13056                      # needs 60 MB of partials: more than the built-in array
    assert L.tgdn_conv_bwd_scratch_bytes(B, T, C) > STATIC_BYTES
    rc = L.tgdn_conv_bwd_static(fake, fake, fake, fake, fake, None, 0, B, T, C, T * C, C, T * C, C, 0, None)
    assert rc == -7
    assert b"static" in L.tgdn_error_string(rc)
