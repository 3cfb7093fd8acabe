"""CPU oracle for the Triadic Gated DeltaNet hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch on the CPU, what the reference package computes on this path.  It is
imported by the tests, by the smoke check and by the CPU-baseline leg of the benchmark, and by nothing
else: the product path (the CUDA library) never falls back to it.

Two independent restatements of the core are given, and the tests check them against each other and
against stored outputs of the reference itself (tests/golden):

  * `sequential_reference`  the token-by-token definition of the recurrence
        S_e <- exp(g_te) S_e ;  S <- S + beta_t kappa_t (v_t - S^T kappa_t)^T ;  o_t = S^T (q2_t (x) q_t) scale
    (reference: README.md:36-42, cute_triadic_gdn/ops/gdn_joint.py:1-8);
  * `chunk_reference`       the chunkwise form with 64-token chunks that the reference's torch path
    evaluates (reference: cute_triadic_gdn/ops/gdn_joint.py:36-39 cumsum, :45-60 masks, :63-90 forward,
    :93-115 autograd wrapper; packed rows: cute_triadic_gdn/ops/joint_packing.py:65-90).

Both are differentiable through autograd and accept a `dtype` (float32 reproduces the reference's
arithmetic, float64 gives a tighter yardstick).  `conv_reference` restates the width-4 causal depthwise
convolution with SiLU on the leading channels (reference: cute_triadic_gdn/ops/conv_split_act.py:20-55 forward,
:58-107 backward; bf16 output rounding :55, SiLU' evaluated on the bf16-rounded pre-activation :158-159, :96-99).

Parity status: the core restatements are pinned by tests/golden/*.npz, generated from the reference's own
`_JointTorch` / `pack_documents` by tests/golden/make_golden.py.  The convolution has no test and no torch
path in the reference; it is pinned against the reference's Triton kernels run through the Triton
interpreter on the CPU (same generator script).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CHUNK = 64


# ----------------------------------------------------------------------------------------------------
# seeded inputs
# ----------------------------------------------------------------------------------------------------
def l2norm(t: torch.Tensor) -> torch.Tensor:
    """t * rsqrt(sum(t^2) + 1e-6) over the last axis (reference fixture: tests/test_joint.py:16-18)."""
    tf = t.float()
    return (tf * torch.rsqrt((tf * tf).sum(-1, keepdim=True) + 1e-6)).to(t.dtype)


def make_inputs(B, T, H, E, seed, dist="baseline"):
    """Seeded inputs, generated on the CPU so that every machine sees the same bits.

    dist="baseline": q, k = l2norm(N(0,1)) bf16; v = N(0,1) bf16; k2, q2 = l2norm(N(0,1)) over E, f32;
    g = -softplus(N(0,1)); beta = sigmoid(N(0,1)).  Draw order q, k, v, k2, q2, g, beta.
    dist="mild": the distribution of the reference's own test fixture (tests/test_joint.py:21-31):
    v = 0.5 N(0,1), k2, q2 = l2norm(softplus(N(0,1))), g = -softplus(N(0,1)+3) * U(0,1)[H,E] * 0.2.
    """
    gen = torch.Generator().manual_seed(int(seed))
    r = lambda *s: torch.randn(*s, generator=gen)
    q = l2norm(r(B, T, H, 128)).to(torch.bfloat16)
    k = l2norm(r(B, T, H, 128)).to(torch.bfloat16)
    if dist == "baseline":
        v = r(B, T, H, 128).to(torch.bfloat16)
        k2 = l2norm(r(B, T, H, E))
        q2 = l2norm(r(B, T, H, E))
        g = -F.softplus(r(B, T, H, E))
    elif dist == "mild":
        v = (0.5 * r(B, T, H, 128)).to(torch.bfloat16)
        k2 = l2norm(F.softplus(r(B, T, H, E)))
        q2 = l2norm(F.softplus(r(B, T, H, E)))
        g = -F.softplus(r(B, T, H, E) + 3.0) * torch.rand(H, E, generator=gen) * 0.2
    else:
        raise ValueError(dist)
    beta = torch.sigmoid(r(B, T, H))
    return [t.contiguous() for t in (q, k, v, k2, q2, g.float(), beta)]


def make_grad_output(shape, seed):
    """Upstream gradient dO = N(0,1) rounded to bf16."""
    gen = torch.Generator().manual_seed(int(seed))
    return torch.randn(*shape, generator=gen).to(torch.bfloat16)


def lognormal_documents(T, seed, median=2048.0, sigma=1.0):
    """Document lengths max(1, round(lognormal(ln median, sigma))) drawn until they cover T; the last one
    is truncated.  Returns the int32 prefix sums (cu_seqlens)."""
    import numpy as np
    rng = np.random.default_rng(int(seed))
    cu = [0]
    while cu[-1] < T:
        n = max(1, int(round(float(rng.lognormal(math.log(median), sigma)))))
        cu.append(min(T, cu[-1] + n))
    return torch.tensor(cu, dtype=torch.int32)


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b|| / ||b|| (reference: tests/test_joint.py:42-43)."""
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


# ----------------------------------------------------------------------------------------------------
# the recurrence, token by token (the definition)
# ----------------------------------------------------------------------------------------------------
def _documents(T, cu_seqlens):
    if cu_seqlens is None:
        return [(0, T)]
    cu = [int(c) for c in cu_seqlens.tolist()]
    if cu[0] != 0 or cu[-1] != T or any(b <= a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must start at 0, end at T, and strictly increase")
    return list(zip(cu[:-1], cu[1:]))


def sequential_reference(q, k, v, k2, q2, g, beta, scale=None, cu_seqlens=None, dtype=torch.float64):
    """o (B,T,H,128) in `dtype`, one token at a time; the state restarts at every document start."""
    B, T, H, D = q.shape
    E = k2.shape[-1]
    scale = D ** -0.5 if scale is None else scale
    q, k, v, k2, q2, g, beta = (t.to(dtype) for t in (q, k, v, k2, q2, g, beta))
    rows = []
    for (lo, hi) in _documents(T, cu_seqlens):
        S = torch.zeros(B, H, E, D, v.shape[-1], dtype=dtype)
        for t in range(lo, hi):
            S = S * g[:, t].exp()[..., None, None]
            kap = k2[:, t, :, :, None] * k[:, t, :, None, :]                    # (B,H,E,D)
            pred = torch.einsum('bhed,bhedv->bhv', kap, S)
            S = S + beta[:, t, :, None, None, None] * kap[..., None] * (v[:, t] - pred)[:, :, None, None, :]
            qk = q2[:, t, :, :, None] * q[:, t, :, None, :]
            rows.append(torch.einsum('bhed,bhedv->bhv', qk, S) * scale)
    return torch.stack(rows, 1)


# ----------------------------------------------------------------------------------------------------
# the chunkwise form
# ----------------------------------------------------------------------------------------------------
def chunk_cumsum(g):
    """Inclusive cumulative sum of the log gate inside every 64-token chunk: (B,T,H,E) -> (B,NC,H,64,E)."""
    B, T, H, E = g.shape
    return g.view(B, T // CHUNK, CHUNK, H, E).cumsum(2).transpose(2, 3)


def _chunks(t):
    B, T, H, X = t.shape
    return t.view(B, T // CHUNK, CHUNK, H, X).transpose(2, 3)                   # (B,NC,H,64,X)


def chunk_masks(k, k2, q2, gc, beta):
    """The UT transform A = (I + strict_lower(beta_t <k_t,k_s> M_ts))^-1 and the decay masks
    M_ts = sum_e k2_te k2_se exp(gc_te - gc_se), Mp_ts = sum_e q2_te k2_se exp(gc_te - gc_se).
    All arguments chunked: k (B,NC,H,64,128), k2/q2/gc (B,NC,H,64,E), beta (B,NC,H,64)."""
    decay = (gc[..., :, None, :] - gc[..., None, :, :]).clamp(max=0.0).exp()    # (…,t,s,E)
    M = (k2[..., :, None, :] * k2[..., None, :, :] * decay).sum(-1)
    Mp = (q2[..., :, None, :] * k2[..., None, :, :] * decay).sum(-1)
    gram = k @ k.transpose(-1, -2)
    eye = torch.eye(CHUNK, dtype=k.dtype)
    A = torch.linalg.inv(eye + (beta[..., None] * gram * M).tril(-1))
    return A, M, Mp


def _chunk_document(q, k, v, k2, q2, g, beta, scale):
    """One batch of whole-chunk sequences starting from a zero state."""
    B, T, H, D = q.shape
    E = k2.shape[-1]
    gc = chunk_cumsum(g)
    qc, kc, vc, k2c, q2c = (_chunks(t) for t in (q, k, v, k2, q2))
    bc = beta.view(B, T // CHUNK, CHUNK, H).transpose(2, 3)
    A, _, Mp = chunk_masks(kc, k2c, q2c, gc, bc)
    S = torch.zeros(B, H, E, D, v.shape[-1], dtype=q.dtype)
    out = []
    for n in range(T // CHUNK):
        K, Q, V = kc[:, n], qc[:, n], vc[:, n]                                  # (B,H,64,·)
        gcn, gl = gc[:, n], gc[:, n, :, -1]                                     # (B,H,64,E), (B,H,E)
        a = k2c[:, n] * gcn.exp()
        c = q2c[:, n] * gcn.exp()
        r = k2c[:, n] * (gl[:, :, None] - gcn).exp()
        KS = torch.einsum('bhtd,bhedv->bhtev', K, S)
        QS = torch.einsum('bhtd,bhedv->bhtev', Q, S)
        W = V - torch.einsum('bhte,bhtev->bhtv', a, KS)
        U = A[:, n] @ (bc[:, n, :, :, None] * W)
        intra = ((Q @ K.transpose(-1, -2)) * Mp[:, n]).tril(0) @ U
        out.append(scale * (torch.einsum('bhte,bhtev->bhtv', c, QS) + intra))
        S = gl.exp()[..., None, None] * S + torch.einsum('bhte,bhtd,bhtv->bhedv', r, K, U)
    return torch.stack(out, 1).transpose(2, 3).reshape(B, T, H, v.shape[-1])    # (B,NC,H,64,V) -> (B,T,H,V)


def chunk_reference(q, k, v, k2, q2, g, beta, scale=None, cu_seqlens=None, dtype=torch.float32):
    """o (B,T,H,128) in `dtype` by the chunkwise form.  Packed rows: every document is padded with zero
    tokens to whole chunks and evaluated from a zero state (zero k2, q2, beta rows change nothing)."""
    B, T, H, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    ins = [t.to(dtype) for t in (q, k, v, k2, q2, g, beta)]
    if cu_seqlens is None:
        if T % CHUNK:
            raise ValueError("T must be a multiple of 64 without cu_seqlens")
        return _chunk_document(*ins, scale)
    if B != 1:
        raise ValueError("cu_seqlens requires a packed row, B=1")
    outs = []
    for (lo, hi) in _documents(T, cu_seqlens):
        pad = (-(hi - lo)) % CHUNK
        doc = [F.pad(t[:, lo:hi], (0, 0) * (t.ndim - 2) + (0, pad)) for t in ins]
        outs.append(_chunk_document(*doc, scale)[:, :hi - lo])
    return torch.cat(outs, 1)


def reference_with_grads(fn, inputs, do, scale=None, cu_seqlens=None, dtype=torch.float32):
    """Run `fn` (one of the two restatements) and differentiate: returns o and the seven gradients, in `dtype`."""
    leaves = [t.detach().to(dtype).requires_grad_(True) for t in inputs]
    o = fn(*leaves, scale=scale, cu_seqlens=cu_seqlens, dtype=dtype)
    grads = torch.autograd.grad(o, leaves, do.to(dtype))
    return o.detach(), [x.detach() for x in grads]


# ----------------------------------------------------------------------------------------------------
# the convolution pre-pass
# ----------------------------------------------------------------------------------------------------
def _silu_grad(y):
    s = torch.sigmoid(y)
    return s * (1 + y * (1 - s))


def conv_reference(x, weight, act_channels, cu_seqlens=None, rounded=True):
    """y (B,T,C) bf16: y[t,c] = sum_w x[t-3+w,c] weight[c,w] in f32, SiLU on channels < act_channels, one
    rounding to bf16 (round to nearest even, as the reference's store asks); the window restarts at every
    document start.  rounded=False returns the f32 values before that rounding."""
    B, T, C = x.shape
    W = weight.shape[1]
    xf, wf = x.float(), weight.float()
    y = torch.empty(B, T, C, dtype=torch.float32)
    for (lo, hi) in _documents(T, cu_seqlens):
        seg = F.pad(xf[:, lo:hi].transpose(1, 2), (W - 1, 0))
        y[:, lo:hi] = F.conv1d(seg, wf[:, None, :], groups=C).transpose(1, 2)
    if act_channels > 0:
        y[..., :act_channels] = F.silu(y[..., :act_channels])
    return y.to(x.dtype) if rounded else y


def conv_reference_backward(x, weight, act_channels, dy, cu_seqlens=None):
    """(dx bf16, dw in weight's dtype).  The SiLU derivative is taken at the bf16-rounded pre-activation, as the
    reference recomputes it with a second forward launch; dw is accumulated in f32 and rounded once."""
    B, T, C = x.shape
    W = weight.shape[1]
    xf, wf = x.float(), weight.float()
    dyf = dy.float().clone()
    if act_channels > 0:
        pre = conv_reference(x, weight, 0, cu_seqlens).float()
        dyf[..., :act_channels] *= _silu_grad(pre[..., :act_channels])
    dx = torch.zeros(B, T, C, dtype=torch.float32)
    dw = torch.zeros(C, W, dtype=torch.float32)
    for (lo, hi) in _documents(T, cu_seqlens):
        n = hi - lo
        for w in range(W):                      # y[t] += x[t-3+w] weight[w]
            sh = W - 1 - w
            if sh >= n:
                continue
            dx[:, lo:hi - sh] += dyf[:, lo + sh:hi] * wf[:, w]
            dw[:, w] += (dyf[:, lo + sh:hi] * xf[:, lo:hi - sh]).sum((0, 1))
    return dx.to(x.dtype), dw.to(weight.dtype)


def glue_reference(x, weight, heads, slices, cu_seqlens=None, eps=1e-6):
    """The layer glue the reference describes around its convolution (cute_triadic_gdn/ops/conv_split_act.py:3-5: "q, k, v
    (SiLU) and its second key and query (no activation, softplus afterwards)"), in f32 and differentiable in x and weight
    (pass float tensors that require grad): channels [q | k | v | k2 | q2] -> q, k = l2norm(SiLU(conv)), v = SiLU(conv) as
    (B, T, heads, 128); k2, q2 = l2norm(softplus(conv)) as (B, T, heads, slices); l2norm(s) = s * rsqrt(sum s^2 + eps).
    Nothing is rounded."""
    B, T, C = x.shape
    W = weight.shape[1]
    xf, wf = x.float(), weight.float()
    rows = []
    for (lo, hi) in _documents(T, cu_seqlens):
        seg = F.pad(xf[:, lo:hi].transpose(1, 2), (W - 1, 0))
        rows.append(F.conv1d(seg, wf[:, None, :], groups=C).transpose(1, 2))
    y = torch.cat(rows, 1)
    hd = heads * 128
    q, k, v, k2, q2 = y.split([hd, hd, hd, heads * slices, heads * slices], dim=-1)
    l2 = lambda t: t * torch.rsqrt((t * t).sum(-1, keepdim=True) + eps)
    q, k, v = (F.silu(t).view(B, T, heads, 128) for t in (q, k, v))
    k2, q2 = (F.softplus(t).view(B, T, heads, slices) for t in (k2, q2))
    return l2(q), l2(k), v, l2(k2), l2(q2)
