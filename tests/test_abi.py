"""The C ABI without a GPU: the library builds, loads and exports what include/tgdn.h declares; argument checks that
run before any launch return the documented codes."""
import ctypes

import pytest

from cute_triadic_gdn_b200 import _lib
from oracle.packing_oracle import chunk_capacity


def test_every_declared_symbol_is_exported_and_bound():
    declared = _lib.declared_symbols()
    assert declared, "no declarations found in include/tgdn.h"
    for name in declared:
        assert hasattr(_lib.lib, name), f"{name} is declared but not exported"
    assert sorted(_lib.SIGNATURES) == declared


def test_gate_item_size_matches_the_host_side():
    from cute_triadic_gdn_b200.gdn_joint import gate_item_floats
    for E in (1, 2, 4, 8, 12, 16):
        assert _lib.lib.tgdn_gate_item_floats(E) == gate_item_floats(E) == 256 * E + 16


def test_chunk_gates_is_a_view_of_the_first_block():
    import torch
    from cute_triadic_gdn_b200.gdn_joint import chunk_gates, gate_item_floats
    E = 4
    gc = torch.arange(2 * 3 * 5 * gate_item_floats(E), dtype=torch.float32).reshape(2, 3, 5, gate_item_floats(E))
    view = chunk_gates(gc, E)
    assert view.shape == (2, 3, 5, 64, E)
    assert view.data_ptr() == gc.data_ptr()
    assert torch.equal(view[1, 2, 4, 63], gc[1, 2, 4, 63 * E:64 * E])


def test_version_and_error_strings():
    assert _lib.lib.tgdn_abi_version() >= 101
    assert _lib.lib.tgdn_error_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5, -6, -1002, -77):
        assert len(_lib.lib.tgdn_error_string(code)) > 3


@pytest.mark.parametrize("T,N", [(64, 1), (640, 4), (3000, 6), (131072, 57), (1, 1), (65, 2)])
def test_chunk_capacity_matches_reference_formula(T, N):
    assert _lib.lib.tgdn_chunk_capacity(T, N) == chunk_capacity(T, N)


def _conv_scratch(B, T, C):
    """One f32 weight-gradient partial of C x 4 per CTA along the token axis: four waves of the 2 x 148 resident CTAs of the
    backward, in runs of at least eight 32-token tiles."""
    n_tiles, columns = (T + 31) // 32, (C + 255) // 256 * B
    g = max(1, min(n_tiles // 8, 4 * 2 * 148 // columns))
    tpg = (n_tiles + g - 1) // g
    groups = (n_tiles + tpg - 1) // tpg
    return B * groups * C * 4 * 4


def test_null_and_shape_arguments_are_rejected_before_launch():
    L = _lib.lib
    null = ctypes.c_void_p(None)
    fake = ctypes.c_void_p(4096)
    assert L.tgdn_conv_fwd(null, null, null, null, 0, 1, 64, 64, 0, 64, 0, null) == -2
    assert L.tgdn_conv_fwd(fake, fake, fake, null, 0, 1, 64, 63, 0, 63, 0, null) == -1       # C % 8
    assert L.tgdn_conv_fwd(ctypes.c_void_p(4098), fake, fake, null, 0, 1, 64, 64, 0, 64, 0, null) == -3
    assert L.tgdn_conv_bwd(fake, fake, fake, fake, fake, null, 0, 1, 64, 64, 0, 64, 0, 64, 0, null, 0, null) == -5
    assert L.tgdn_conv_bwd_scratch_bytes(1, 300, 64) == _conv_scratch(1, 300, 64)
    assert L.tgdn_conv_bwd_scratch_bytes(1, 32768, 13056) == _conv_scratch(1, 32768, 13056)
    assert L.tgdn_metadata(null, 0, 1, 64, null, null, 16, null, null) == -2
    assert L.tgdn_metadata(fake, 0, 3, 640, fake, fake, 8, fake, null) == -1                  # capacity too small
    assert L.tgdn_selftest_mma(fake, fake, fake, 96, 64, 64, 0, 0, null) == -1
