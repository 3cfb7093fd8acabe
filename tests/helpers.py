"""Shared helpers of the test-suite: golden fixtures and comparisons."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GRADS = "q k v k2 q2 g beta".split()


def bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16)


def load_core(path):
    z = np.load(path)
    ins = [bf16(z["q"]), bf16(z["k"]), bf16(z["v"])] + [torch.from_numpy(z[n]) for n in ("k2", "q2", "g", "beta")]
    do = bf16(z["do"])
    cu = torch.from_numpy(z["cu_seqlens"]) if "cu_seqlens" in z.files else None
    ref = {"o": torch.from_numpy(z["ref_o"])}
    for n in GRADS:
        ref["d" + n] = torch.from_numpy(z["ref_d" + n])
    return ins, do, cu, ref


def core_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "core_*.npz")))


def conv_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "conv_*.npz")))
