"""Generate the golden fixtures in this directory from the reference package itself.

Run once, on a machine where the reference checkout is available:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

It imports the reference's differentiable torch path (`cute_triadic_gdn.ops.gdn_joint._JointTorch`,
`cute_triadic_gdn.ops.joint_packing.pack_documents`) and, for the convolution, the reference's Triton
kernels executed by the Triton interpreter on the CPU, and stores inputs and outputs of small seeded cases
as compressed .npz files.  The tests compare the CPU oracle (oracle/triadic_oracle.py) with these files, so the
reference is not needed when the tests run.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle.triadic_oracle import make_grad_output, make_inputs  # noqa: E402

# (name, B, T, H, E, dist, docs)
CORE_CASES = [
    ("dense_e1", 1, 128, 2, 1, "baseline", None),
    ("dense_e2", 1, 64, 1, 2, "baseline", None),
    ("dense_e4", 2, 128, 1, 4, "baseline", None),
    ("dense_e8", 1, 128, 1, 8, "baseline", None),
    ("dense_e12", 1, 64, 1, 12, "mild", None),
    ("dense_e16", 1, 128, 1, 16, "mild", None),
    ("packed_e2", 1, 200, 1, 2, "baseline", [0, 64, 65, 200]),
    ("packed_e8", 1, 230, 1, 8, "mild", [0, 70, 133, 230]),
]


def bits(t):
    return t.view(torch.int16).numpy()


def core_case(ref_joint, ref_pack, name, B, T, H, E, dist, docs):
    ins = make_inputs(B, T, H, E, seed=1000 * E + T, dist=dist)
    do = make_grad_output((B, T, H, 128), seed=7)
    # fp32 copies of the bf16-rounded tensors: the reference's torch path upcasts anyway; this keeps o and the
    # gradients in fp32 instead of rounding them to bf16 at the end
    leaves = [t.float().clone().requires_grad_(True) for t in ins]
    cu = None if docs is None else torch.tensor(docs, dtype=torch.int32)
    if cu is None:
        o = ref_joint.apply(*leaves, 128 ** -0.5, None)
    else:
        packed, chunk_starts, restore = ref_pack(tuple(leaves), cu)
        o = ref_joint.apply(*packed, 128 ** -0.5, chunk_starts).index_select(1, restore)
    o.backward(do.float())
    out = {"o": o.detach().numpy()}
    for n, t in zip("q k v k2 q2 g beta".split(), leaves):
        out["d" + n] = t.grad.numpy()
    inp = {"q": bits(ins[0]), "k": bits(ins[1]), "v": bits(ins[2]), "k2": ins[3].numpy(), "q2": ins[4].numpy(),
           "g": ins[5].numpy(), "beta": ins[6].numpy(), "do": bits(do)}
    if docs is not None:
        inp["cu_seqlens"] = np.asarray(docs, dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, f"core_{name}.npz"), **inp, **{"ref_" + k: v for k, v in out.items()})
    print("wrote", name, {k: float(np.abs(v).max()) for k, v in out.items()})


def conv_case(mod, name, B, T, C, act, docs, seed):
    import triton
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, C, generator=gen).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, generator=gen)).to(torch.bfloat16)
    dy = torch.randn(B, T, C, generator=gen).to(torch.bfloat16)
    cu = None if docs is None else torch.tensor(docs, dtype=torch.int32)
    fwd, bwd = mod._fwd_kernel.fn.fn, mod._bwd_kernel.fn.fn      # the jitted functions under heuristics + autotune
    Bq, Tq, D, W, BW, NB, NT, chunk_indices = mod._layout(x, w, cu)
    BD = 32

    def forward(act_ch):
        y = torch.empty_like(x)
        fwd[(triton.cdiv(D, BD), NT, B)](
            x, y, w, cu, chunk_indices, B, T, x.stride(0), x.stride(1), x.stride(2),
            D=D, W=W, BT=64, BW=BW, BD=BD, NB=NB, ACT_CH=act_ch, IS_VARLEN=cu is not None)
        return y

    y = forward(act)
    pre = forward(0) if act > 0 else None
    dx = torch.empty_like(x)
    dw = torch.empty(B * NT, D, W, dtype=torch.float32)
    bwd[(triton.cdiv(D, BD), NT, B)](
        x, pre, w, dy, dx, dw, cu, chunk_indices, B, T, x.stride(0), x.stride(1), x.stride(2),
        dx.stride(0), dx.stride(1), dx.stride(2), dy.stride(0), dy.stride(1), dy.stride(2),
        D=D, W=W, BT=64, BW=BW, BD=BD, NB=NB, ACT_CH=act, IS_VARLEN=cu is not None)
    dwsum = dw.sum(0).to(w.dtype)
    d = {"x": bits(x), "w": bits(w), "dy": bits(dy), "act": np.int32(act),
         "ref_y": bits(y), "ref_dx": bits(dx), "ref_dw": bits(dwsum), "ref_dw_f32": dw.sum(0).numpy()}
    if docs is not None:
        d["cu_seqlens"] = np.asarray(docs, dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, f"conv_{name}.npz"), **d)
    print("wrote conv", name)


# packed rows whose chunking the reference's pack_documents pins: (cu_seqlens, T)
PACKING_CASES = [([0, 70, 133, 400, 640], 640), ([0, 64, 65, 320], 320), ([0, 512], 512),
                 ([0, 17, 900, 901, 1500, 2999, 3000], 3000), ([0, 1], 1), ([0, 1, 2, 3, 4], 4),
                 ([0, 63, 127, 128, 192, 1000], 1000)]


def packing_cases(ref_pack):
    """What the reference's pack_documents makes of each offsets vector: `restore` (token -> position in the padded
    row) and `chunk_starts` (padded chunk begins a document).  Together they fix every chunk's first token and valid rows,
    and every document's first chunk, which is what the device metadata must reproduce."""
    out = {}
    for i, (cu, T) in enumerate(PACKING_CASES):
        x = torch.zeros(1, T, 1, 1)
        _, chunk_starts, restore = ref_pack((x,), torch.tensor(cu, dtype=torch.int32))
        out[f"cu_{i}"] = np.asarray(cu, dtype=np.int64)
        out[f"restore_{i}"] = restore.numpy().astype(np.int64)
        out[f"chunk_starts_{i}"] = chunk_starts.numpy().reshape(-1)
    np.savez_compressed(os.path.join(HERE, "packing_cases.npz"), **out)
    print("wrote packing_cases", len(PACKING_CASES))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    sys.path.insert(0, sys.argv[1])
    from cute_triadic_gdn.ops import gdn_joint, joint_packing
    torch.manual_seed(0)
    packing_cases(joint_packing.pack_documents)
    if "--packing-only" in sys.argv:
        return
    for case in CORE_CASES:
        core_case(gdn_joint._JointTorch, joint_packing.pack_documents, *case)
    try:
        from cute_triadic_gdn.ops import conv_split_act as mod
        conv_case(mod, "dense", 2, 100, 96, 64, None, 11)
        conv_case(mod, "packed", 1, 150, 80, 48, [0, 1, 3, 70, 150], 12)
        conv_case(mod, "noact", 1, 70, 40, 0, None, 13)
    except Exception as exc:   # the Triton interpreter is optional; the core fixtures do not depend on it
        print("conv fixtures not generated:", repr(exc))


if __name__ == "__main__":
    main()
