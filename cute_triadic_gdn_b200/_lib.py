"""ctypes binding of libtgdn_b200.so (the C ABI declared in include/tgdn.h).

The library is the only implementation of the hot path: there is no fallback.  If the shared object is missing it is
built once with nvcc (cute_triadic_gdn_b200/build.py); if that is impossible the import fails loudly.
"""
from __future__ import annotations

import ctypes
import os
import re

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libtgdn_b200.so")
HEADERS = [os.path.join(_PKG, "..", "include", n) for n in ("tgdn.h", "tgdn_selftest.h")]

_c = ctypes
_P, _I, _L, _F = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float

# name -> (restype, argtypes); kept in the order of include/tgdn.h
SIGNATURES = {
    "tgdn_error_string": (_c.c_char_p, [_I]),
    "tgdn_abi_version": (_I, []),
    "tgdn_device_status": (_I, [_P]),
    "tgdn_conv_fwd": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _I, _P]),
    "tgdn_conv_bwd_scratch_bytes": (_L, [_I, _I, _I]),
    "tgdn_conv_bwd": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _I, _P, _L, _P]),
    "tgdn_conv_bwd_static": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _I, _P]),
    "tgdn_chunk_capacity": (_I, [_I, _I]),
    "tgdn_metadata": (_I, [_P, _I, _I, _I, _P, _P, _I, _P, _P]),
    "tgdn_gate_item_floats": (_I, [_I]),
    "tgdn_masks": (_I, [_P, _P, _P, _P, _P, _P, _F, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "tgdn_fwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "tgdn_fwd_state": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "tgdn_glue_fwd": (_I, [_P, _P, _P, _I, _I, _I, _I, _L, _L, _I, _I, _F, _P, _P, _P, _P, _P, _P]),
    "tgdn_glue_bwd_norm": (_I, [_P, _P, _P, _I, _I, _I, _I, _L, _L, _I, _I, _F, _P, _P, _P, _P, _P, _P, _P]),
    "tgdn_decode_step": (_I, [_P] * 7 + [_F, _I, _I, _I, _P, _P, _P]),
    "tgdn_bwd_recurrent": (_I, [_P] * 10 + [_F, _P, _P] + [_I] * 6 + [_P] * 6),
    "tgdn_bwd_recurrent_state": (_I, [_P] * 10 + [_F, _P, _P] + [_I] * 6 + [_P] * 8),
    "tgdn_bwd_state_grads": (_I, [_P] * 10 + [_F, _P] + [_I] * 5 + [_P] * 5),
    "tgdn_bwd_matrix": (_I, [_P] * 16 + [_F, _P] + [_I] * 5 + [_P] * 7),
    "tgdn_selftest_mma": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "tgdn_selftest_tma": (_I, [_P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "tgdn_selftest_wait": (_I, [_c.c_longlong, _P, _P]),
}


class TgdnError(RuntimeError):
    """A call into libtgdn_b200 returned a non-zero code."""


def declared_symbols():
    """Names of the functions declared in include/tgdn.h and include/tgdn_selftest.h."""
    text = ""
    for path in HEADERS:
        with open(path) as fh:
            text += re.sub(r"/\*.*?\*/", "", fh.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(tgdn_[a-z0-9_]+)\s*\(", text)))


def _load():
    """Builds the library when a source changed since it was linked (a no-op otherwise) and binds the signatures.  Several
    ranks may import the package at once: the build is serialised by a file lock and the library is moved into place
    atomically (build.py), so nobody can load a half-written file.  A library that is out of date and cannot be rebuilt
    is NOT loaded silently: its signatures may no longer match include/tgdn.h."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_tgdn_build", os.path.join(_PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        mod.build()
    except Exception as exc:
        if not os.path.exists(LIB_PATH):
            raise
        if not mod.up_to_date():
            raise RuntimeError("libtgdn_b200.so is older than its sources and could not be rebuilt "
                               f"({type(exc).__name__}: {exc}); refusing to bind a stale library") from exc
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(code, what):
    if code != 0:
        raise TgdnError(f"{what}: {lib.tgdn_error_string(code).decode()} (code {code})")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t):
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def device_status():
    """Blocking read-and-clear of the device status word (0 = every kernel ran to completion normally)."""
    out = ctypes.c_int(0)
    check(lib.tgdn_device_status(ctypes.byref(out)), "tgdn_device_status")
    return out.value
