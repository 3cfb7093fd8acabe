"""A torch model of the CUDA kernels' dataflow.  TEST INFRASTRUCTURE ONLY.

The CUDA library evaluates the chunkwise Triadic GDN (reference math: cute_triadic_gdn/ops/gdn_joint.py:45-90)
in five kernels: masks, forward recurrence, reverse recurrence, state gradients and the per-chunk matrix
gradients.  This file evaluates the same stages with explicit formulas for the backward pass (no autograd), with
an optional bf16 rounding at every place where the kernels store or stage a tensor in bf16.  The tests use it
  * with rounding off and float64: to check the backward formulas against autograd of the oracle;
  * with rounding on: to check that the rounding plan stays inside the parity tolerance, and to localise a
    mismatch of the GPU path to one stage by comparing intermediates.
Tensors are chunked and batched over (batch x head): K, Q, V, dO are (N, NC, 64, 128); k2, q2, g are
(N, NC, 64, E); beta is (N, NC, 64).  `reset[n]` marks chunks that start a document (state restarts).
"""
from __future__ import annotations

import torch

CHUNK = 64


def _rd(on):
    if on:
        return lambda t: t.to(torch.bfloat16).to(t.dtype)
    return lambda t: t


def to_chunks(t):
    """(B,T,H,X) or (B,T,H) -> (B*H, NC, 64, X) / (B*H, NC, 64)."""
    if t.ndim == 3:
        B, T, H = t.shape
        return t.view(B, T // CHUNK, CHUNK, H).permute(0, 3, 1, 2).reshape(B * H, T // CHUNK, CHUNK)
    B, T, H, X = t.shape
    return t.view(B, T // CHUNK, CHUNK, H, X).permute(0, 3, 1, 2, 4).reshape(B * H, T // CHUNK, CHUNK, X)


def from_chunks(t, B, H):
    """inverse of to_chunks"""
    if t.ndim == 3:
        N, NC, C = t.shape
        return t.view(B, H, NC, C).permute(0, 2, 3, 1).reshape(B, NC * C, H)
    N, NC, C, X = t.shape
    return t.view(B, H, NC, C, X).permute(0, 2, 3, 1, 4).reshape(B, NC * C, H, X)


def gates(k2, q2, gc, scale):
    gl = gc[..., -1:, :]
    eg, egr = gc.exp(), (gl - gc).exp()
    return dict(a=k2 * eg, c=scale * q2 * eg, r=k2 * egr, d=gl[..., 0, :].exp(), eg=eg, egr=egr)


def masks_stage(K, Q, k2, q2, g, beta, scale, rounding):
    rd = _rd(rounding)
    gc = g.cumsum(-2)
    decay = (gc[..., :, None, :] - gc[..., None, :, :]).clamp(max=0.0).exp()
    M = (k2[..., :, None, :] * k2[..., None, :, :] * decay).sum(-1)
    Mp = (q2[..., :, None, :] * k2[..., None, :, :] * decay).sum(-1)
    Pkk = K @ K.transpose(-1, -2)
    Pqk = Q @ K.transpose(-1, -2)
    eye = torch.eye(CHUNK, dtype=K.dtype)
    A = torch.linalg.inv(eye + (beta[..., None] * Pkk * M).tril(-1))
    Pm = scale * (Pqk * Mp).tril(0)
    PA = rd(Pm) @ rd(A)                      # the kernel multiplies the two bf16 images it is about to store
    return dict(gc=gc, A=rd(A), Pm=rd(Pm), PA=rd(PA), M=M, Mp=Mp, decay=decay, Pkk=Pkk, Pqk=Pqk)


def forward_stage(K, Q, V, k2, q2, beta, scale, mk, reset, rounding):
    rd = _rd(rounding)
    N, NC, C, D = K.shape
    E = k2.shape[-1]
    gt = gates(k2, q2, mk["gc"], scale)
    S = torch.zeros(N, E, D, D, dtype=K.dtype)
    o, Ws, Us, hs = [], [], [], []
    for n in range(NC):
        if reset is not None:
            S = torch.where(reset[n], torch.zeros_like(S), S) if isinstance(reset[n], torch.Tensor) else (S * 0 if reset[n] else S)
        Sb = rd(S)
        hs.append(Sb)
        R = torch.einsum('ntd,nedv->netv', K[:, n], Sb)
        Rq = torch.einsum('ntd,nedv->netv', Q[:, n], Sb)
        W = V[:, n] - torch.einsum('nte,netv->ntv', gt["a"][:, n], R)
        bW = rd(beta[:, n, :, None] * W)
        U = mk["A"][:, n] @ bW
        Oi = mk["PA"][:, n] @ bW
        o.append(rd(torch.einsum('nte,netv->ntv', gt["c"][:, n], Rq) + Oi))
        # r_e*U is a product of two bf16 values rounded once (the kernel scales the packed row of U it stores)
        Vn = rd(rd(gt["r"][:, n]).transpose(1, 2)[..., None] * rd(U)[:, None])   # (N,E,64,V)
        S = gt["d"][:, n][..., None, None] * S + torch.einsum('ntd,netv->nedv', K[:, n], Vn)
        Ws.append(rd(W))
        Us.append(rd(U))
    st = lambda x: torch.stack(x, 1)
    return dict(o=st(o), W=st(Ws), U=st(Us), h=st(hs), gates=gt)


def reverse_stage(K, Q, dO, beta, mk, fw, reset, rounding):
    rd = _rd(rounding)
    N, NC, C, D = K.shape
    gt = fw["gates"]
    E = gt["a"].shape[-1]
    G = torch.zeros(N, E, D, D, dtype=K.dtype)
    dU_, dV_, ds_, dr_ = [None] * NC, [None] * NC, [None] * NC, [None] * NC
    for n in reversed(range(NC)):
        Gb = rd(G)
        ds_[n] = Gb
        KG = torch.einsum('ntd,nedv->netv', K[:, n], Gb)
        dU = torch.einsum('nte,netv->ntv', gt["r"][:, n], KG) + mk["Pm"][:, n].transpose(-1, -2) @ dO[:, n]
        dr_[n] = torch.einsum('ntv,netv->nte', fw["U"][:, n], KG)
        dUb = rd(dU)
        dU_[n] = dUb
        Z = mk["A"][:, n].transpose(-1, -2) @ dUb
        dW = beta[:, n, :, None] * Z
        dV_[n] = rd(dW)
        # bf16 factors times the bf16 rows that are stored (dV) or were loaded (dO), rounded once
        X1 = rd(-rd(gt["a"][:, n]).transpose(1, 2)[..., None] * rd(dW)[:, None])
        X2 = rd(rd(gt["c"][:, n]).transpose(1, 2)[..., None] * dO[:, n][:, None])
        G = gt["d"][:, n][..., None, None] * G + torch.einsum('ntd,netv->nedv', K[:, n], X1) \
            + torch.einsum('ntd,netv->nedv', Q[:, n], X2)
        if reset is not None and bool(reset[n]):
            G = G * 0                                   # nothing flows into the previous document
    st = lambda x: torch.stack(x, 1)
    return dict(dU=st(dU_), dV=st(dV_), ds=st(ds_), dr=st(dr_))


DD_MIN_LOG2_DECAY = -24.0       # below this log2 of the chunk decay, exp(gL) * <h, G> is taken as zero (see the kernels)


def value_block(E):
    """Value columns one CTA of the reverse recurrence owns."""
    return 16 if E > 8 else 32


def state_grad_stage(K, Q, dO, fw, rv, mk, rounding):
    rd = _rd(rounding)
    gt = fw["gates"]
    a, c, r = (gt[x].transpose(2, 3)[..., None] for x in "acr")                 # (N,NC,E,64,1)
    h, G = fw["h"], rv["ds"]                                                    # (N,NC,E,D,V)
    dW, U = rv["dV"], fw["U"]
    E = h.shape[2]
    # P_e = [dW ; dO] h_e^T on the tensor core (bf16 operands, f32 result); the gate-weighted sum over the slices and the
    # row sums against K and Q are taken from it in f32.
    P = torch.einsum('nctv,ncedv->ncetd', dW, h)
    Pq = torch.einsum('nctv,ncedv->ncetd', dO, h)
    # The part of dK that contracts the gradient state is formed in the reverse recurrence, per block of value columns,
    # from r_e*U rounded to bf16, and leaves it rounded to bf16; the blocks are then added up in f32.
    Vn = rd(rd(r) * U[:, :, None])             # U is the stored bf16 tensor; r_e enters as bf16 too
    VC = value_block(E)
    dKg = 0
    for j in range(128 // VC):
        sl = slice(j * VC, (j + 1) * VC)
        dKg = dKg + rd(torch.einsum('ncetv,ncedv->nctd', Vn[..., sl], G[..., sl]))
    # the state parts of dK and dQ are handed to the matrix kernel as bf16
    dK = rd((-a * P).sum(2) + dKg)
    dQ = rd((c * Pq).sum(2))
    da = -torch.einsum('nctd,ncetd->ncte', K, P)
    dc = torch.einsum('nctd,ncetd->ncte', Q, Pq)
    dd = (h * G).sum((-1, -2))                                                  # (N,NC,E)
    if rounding:                                                                # slices whose chunk decay cannot matter are skipped
        gl = mk["gc"][..., -1, :]
        dd = torch.where(gl * 1.4426950408889634 >= DD_MIN_LOG2_DECAY, dd, torch.zeros_like(dd))
    return dict(dK=dK, dQ=dQ, da=da, dc=dc, dd=dd, dKg=dKg)


def matrix_stage(K, Q, dO, k2, q2, beta, scale, mk, fw, rv, sg, rounding):
    rd = _rd(rounding)
    gt = fw["gates"]
    T = lambda x: x.transpose(-1, -2)
    A, M, Mp, decay, Pkk, Pqk = mk["A"], mk["M"], mk["Mp"], mk["decay"], mk["Pkk"], mk["Pqk"]
    dPm = dO @ T(fw["U"])
    dAp = rv["dU"] @ T(fw["W"])
    X = scale * (Mp * dPm).tril(0)
    dmp = scale * (Pqk * dPm).tril(0)
    dbeta = (dAp * A).sum(-2)
    dA = rd(dAp * beta[..., None, :])
    Y = rd(T(A) @ dA)
    dL = -(Y @ T(A)).tril(-1)
    dbeta = dbeta + (dL * Pkk * M).sum(-1)
    dPkk = beta[..., None] * dL * M
    dm = beta[..., None] * dL * Pkk
    Xb, Zb = rd(X), rd(dPkk + T(dPkk))
    dQ = rd(Xb @ K + sg["dQ"])
    dK = rd(T(Xb) @ Q + Zb @ K + sg["dK"])
    # mask gradients
    r1 = torch.einsum('ncts,nctse,ncse->ncte', dmp, decay, k2)
    c1 = torch.einsum('ncts,nctse,ncte->ncse', dmp, decay, q2)
    r2 = torch.einsum('ncts,nctse,ncse->ncte', dm, decay, k2)
    c2 = torch.einsum('ncts,nctse,ncte->ncse', dm, decay, k2)
    da, dc, dr = sg["da"], sg["dc"], rv["dr"]
    dk2 = da * gt["eg"] + dr * gt["egr"] + c1 + r2 + c2
    dq2 = dc * scale * gt["eg"] + r1
    dgc = da * gt["a"] + dc * gt["c"] - dr * gt["r"] + q2 * r1 + k2 * (r2 - c1 - c2)
    last = (dr * gt["r"]).sum(-2) + sg["dd"] * gt["d"]
    dgc = torch.cat([dgc[..., :-1, :], dgc[..., -1:, :] + last[..., None, :]], -2)
    dg = dgc.flip(-2).cumsum(-2).flip(-2)
    return dict(dq=dQ, dk=dK, dk2=dk2, dq2=dq2, dg=dg, dbeta=dbeta)


def run_plan(q, k, v, k2, q2, g, beta, do, scale=None, reset=None, rounding=True, dtype=torch.float32):
    """Forward and backward of dense (B,T,H,·) inputs; returns o, the seven gradients and the stage outputs."""
    B, T, H, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    K, Q, V, dO, k2c, q2c, gch, bc = (to_chunks(t.to(dtype)) for t in (k, q, v, do, k2, q2, g, beta))
    mk = masks_stage(K, Q, k2c, q2c, gch, bc, scale, rounding)
    fw = forward_stage(K, Q, V, k2c, q2c, bc, scale, mk, reset, rounding)
    rv = reverse_stage(K, Q, dO, bc, mk, fw, reset, rounding)
    sg = state_grad_stage(K, Q, dO, fw, rv, mk, rounding)
    mt = matrix_stage(K, Q, dO, k2c, q2c, bc, scale, mk, fw, rv, sg, rounding)
    back = lambda t: from_chunks(t, B, H)
    grads = [back(mt["dq"]), back(mt["dk"]), back(rv["dV"]), back(mt["dk2"]), back(mt["dq2"]), back(mt["dg"]),
             back(mt["dbeta"])]
    return back(fw["o"]), grads, dict(masks=mk, fwd=fw, rev=rv, sg=sg, mat=mt)
