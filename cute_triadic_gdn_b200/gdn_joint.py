"""Triadic Gated DeltaNet: `chunk_gdn_joint`, the plain autograd entry, and the kernel pipeline behind it.

Mirrors the operator layer of the reference, cute_triadic_gdn/ops/gdn_joint.py: `_check` (:235-249), the forward
pipeline `_cute_forward` (:144-164), the autograd function `_JointCute` (:201-232), the GJ_SAVE_MASKS switch
(:167-198) and `chunk_gdn_joint` (:252-278).  The device work is the C ABI of libtgdn_b200 (include/tgdn.h); this file
only checks arguments, allocates outputs with torch and enqueues the kernels on torch's current stream.

    S_e <- exp(g_te) S_e ;  S <- S + beta_t kappa_t (v_t - S^T kappa_t)^T ;  o_t = S^T (q2_t (x) q_t) * scale

Inputs (contiguous, one CUDA device): q, k, v (B,T,H,128) bf16; k2, q2, g (B,T,H,E) f32; beta (B,T,H) f32;
E in {1,2,4,8,12,16}.  Without cu_seqlens T % 64 == 0; with cu_seqlens B = 1 and the state restarts at every document.
"""
from __future__ import annotations

import os

import torch

from . import _lib

CHUNK = 64
HEAD_DIM = 128
SUPPORTED_E = (1, 2, 4, 8, 12, 16)


def _check(q, k, v, k2, q2, g, beta, packed=False):
    """Shapes, dtypes, contiguity and device of the seven inputs; an AssertionError names the first thing that is off (the
    reference raises the same error class for the same conditions: ops/gdn_joint.py:235-249)."""
    tensors = dict(q=q, k=k, v=v, k2=k2, q2=q2, g=g, beta=beta)
    assert q.ndim == 4, f"q: expected (B, T, H, 128), got {tuple(q.shape)}"
    B, T, H, D = q.shape
    assert D == HEAD_DIM, f"q: the head dimension must be {HEAD_DIM}, got {D}"
    for name in ("k", "v"):
        assert tuple(tensors[name].shape) == (B, T, H, HEAD_DIM), \
            f"{name}: expected {(B, T, H, HEAD_DIM)} like q, got {tuple(tensors[name].shape)}"
    assert T >= 1, "the sequence is empty"
    assert packed or T % CHUNK == 0, f"T = {T}: rows without cu_seqlens must hold whole chunks of {CHUNK} tokens"
    E = k2.shape[-1] if k2.ndim == 4 else 0
    assert E >= 1, f"k2: expected (B, T, H, E) with E >= 1, got {tuple(k2.shape)}"
    for name in ("k2", "q2", "g"):
        assert tuple(tensors[name].shape) == (B, T, H, E), \
            f"{name}: expected {(B, T, H, E)}, got {tuple(tensors[name].shape)}"
    assert tuple(beta.shape) == (B, T, H), f"beta: expected {(B, T, H)} (one write strength per head), got {tuple(beta.shape)}"
    for name, t in tensors.items():
        want = torch.bfloat16 if name in ("q", "k", "v") else torch.float32
        assert t.dtype == want, f"{name}: dtype {t.dtype}, expected {want}"
        assert t.is_cuda and t.device == q.device, f"{name}: every input must live on q's CUDA device"
        assert t.is_contiguous(), f"{name}: not contiguous"


def _check_device_and_e(q, E):
    if torch.cuda.get_device_capability(q.device)[0] != 10 or E not in SUPPORTED_E:
        raise ValueError("the Triadic GDN kernels require an sm_100 device and E=1/2/4/8/12/16")


def _save_masks():
    """GJ_SAVE_MASKS=1 (default) keeps the chunk operators of the forward for the backward; GJ_SAVE_MASKS=0 drops them
    and lets the backward recompute them with the same kernel (bitwise identical), trading one extra launch for
    24 KiB per (chunk, head) of saved memory.  Read at forward time, like the reference (ops/gdn_joint.py:167-173)."""
    return os.environ.get("GJ_SAVE_MASKS", "1") == "1"


def _dims(q, k2, token_map):
    B, T, H, _ = q.shape
    E = k2.shape[-1]
    NC = token_map.shape[1] if token_map is not None else T // CHUNK
    return B, T, H, E, NC


def gate_item_floats(E):
    """Floats per (batch row, chunk, head) of the gate tensor: gc, a, r, c as 64 x E blocks, then d padded to 16 (include/tgdn.h)."""
    return 4 * CHUNK * E + 16


def chunk_gates(gc, E):
    """The cumulative log gate (B, NC, H, 64, E) as a view of the gate tensor that tgdn_masks writes."""
    return gc[..., :CHUNK * E].unflatten(-1, (CHUNK, E))


def _run_masks(q, k, k2, q2, g, beta, scale, token_map, gc=None):
    """(gc, AP, Pm) of every chunk.  gc holds the cumulative log gate and the gate factors, AP = [A; Pm A] operand image,
    Pm image; see include/tgdn.h."""
    B, T, H, E, NC = _dims(q, k2, token_map)
    dev = q.device
    gc_out = torch.empty((B, NC, H, gate_item_floats(E)), dtype=torch.float32, device=dev)
    AP = torch.empty((B, NC, H, 128 * 64), dtype=torch.bfloat16, device=dev)
    Pm = torch.empty((B, NC, H, 64 * 64), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.tgdn_masks(_lib.ptr(q), _lib.ptr(k), _lib.ptr(k2), _lib.ptr(q2), _lib.ptr(g), _lib.ptr(beta),
                                       float(scale), _lib.ptr(token_map), B, T, H, E, NC, _lib.ptr(gc_out), _lib.ptr(AP),
                                       _lib.ptr(Pm), _lib.stream_of(q)), "tgdn_masks")
    return gc_out, AP, Pm


def _run_forward(q, k, v, k2, q2, beta, gc, AP, scale, save, chunk_starts=None, token_map=None, state_in=None,
                 state_out=None):
    """Forward recurrence: (o, h, W, U); h, W, U are None unless save.  state_in / state_out: optional f32
    (sequences, H, E, 128, 128) tensors holding the recurrent state before the first and after the last token."""
    B, T, H, E, NC = _dims(q, k2, token_map)
    dev = q.device
    o = torch.empty_like(v)
    if token_map is not None:
        o.zero_()  # rows of a packed row are all covered by documents; kept defined even for a rejected chunk map
    h = W = U = None
    if save:
        h = torch.empty((B, NC, H, E, 16, 128, 8), dtype=torch.bfloat16, device=dev)
        W = torch.empty((B, NC, H, CHUNK, 128), dtype=torch.bfloat16, device=dev)
        U = torch.empty((B, NC, H, CHUNK, 128), dtype=torch.bfloat16, device=dev)
    n_docs = chunk_starts.numel() - 1 if chunk_starts is not None else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.tgdn_fwd_state(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(k2), _lib.ptr(q2), _lib.ptr(beta),
                                           _lib.ptr(gc), _lib.ptr(AP), float(scale), _lib.ptr(chunk_starts),
                                           _lib.ptr(token_map), n_docs, B, T, H, E, NC, _lib.ptr(o), _lib.ptr(W),
                                           _lib.ptr(U), _lib.ptr(h), _lib.ptr(state_in), _lib.ptr(state_out),
                                           _lib.stream_of(q)), "tgdn_fwd_state")
    return o, h, W, U


def _kernel_forward(q, k, v, k2, q2, g, beta, scale, save, chunk_starts=None, token_map=None):
    """masks -> forward recurrence.  Returns (o, gc, AP, Pm, h, W, U); h, W, U are None unless save."""
    gc, AP, Pm = _run_masks(q, k, k2, q2, g, beta, scale, token_map)
    o, h, W, U = _run_forward(q, k, v, k2, q2, beta, gc, AP, scale, save, chunk_starts, token_map)
    return o, gc, AP, Pm, h, W, U


def _value_block(E):
    """Width of the value-axis block one CTA of the recurrences owns (fixed by the library per E)."""
    return 16 if E > 8 else 32


def _run_reverse(q, k, do, k2, q2, beta, gc, AP, Pm, U, scale, chunk_starts=None, token_map=None, grad_state_in=None,
                 grad_state_out=None):
    """Reverse recurrence: (dV, dU, ds, dkg, dr).  ds is written only for slices whose chunk decay matters to dg.
    grad_state_in / grad_state_out: optional f32 (sequences, H, E, 128, 128) tensors, dL/dS after the last and before the
    first token (the hand-off between segments of one sequence)."""
    B, T, H, E, NC = _dims(q, k2, token_map)
    dev = q.device
    NV = 128 // _value_block(E)
    alloc = torch.zeros if token_map is not None else torch.empty     # unused map entries stay defined
    dV = torch.zeros_like(do) if token_map is not None else torch.empty_like(do)
    dU = torch.empty((B, NC, H, CHUNK, 128), dtype=torch.bfloat16, device=dev)
    ds = torch.empty((B, NC, H, E, 16, 128, 8), dtype=torch.bfloat16, device=dev)
    dkg = alloc((B, NC, H, NV, 8, 128, 8), dtype=torch.bfloat16, device=dev)   # image [token / 8][key row][token % 8] per value block
    dr = torch.empty((B, NC, H, NV, CHUNK, E), dtype=torch.float32, device=dev)
    n_docs = chunk_starts.numel() - 1 if chunk_starts is not None else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.tgdn_bwd_recurrent_state(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(do), _lib.ptr(k2), _lib.ptr(q2), _lib.ptr(beta), _lib.ptr(gc),
            _lib.ptr(AP), _lib.ptr(Pm), _lib.ptr(U), float(scale), _lib.ptr(chunk_starts), _lib.ptr(token_map), n_docs,
            B, T, H, E, NC, _lib.ptr(dV), _lib.ptr(dU), _lib.ptr(ds), _lib.ptr(dkg), _lib.ptr(dr),
            _lib.ptr(grad_state_in), _lib.ptr(grad_state_out), _lib.stream_of(q)), "tgdn_bwd_recurrent_state")
    return dV, dU, ds, dkg, dr


def _run_state_grads(q, k, do, dV, h, ds, dkg, k2, q2, gc, scale, token_map=None):
    """State gradients: (dkq, da, dc, dd)."""
    B, T, H, E, NC = _dims(q, k2, token_map)
    dev = q.device
    alloc = torch.zeros if token_map is not None else torch.empty     # unused map entries stay defined
    dkq = alloc((B, NC, H, 16, 128, 8), dtype=torch.bfloat16, device=dev)    # image [column / 8][row][column % 8]
    da = alloc((B, NC, H, CHUNK, E), dtype=torch.float32, device=dev)
    dc = alloc((B, NC, H, CHUNK, E), dtype=torch.float32, device=dev)
    dd = alloc((B, NC, H, E), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.tgdn_bwd_state_grads(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(do), _lib.ptr(dV), _lib.ptr(h), _lib.ptr(ds), _lib.ptr(dkg), _lib.ptr(k2),
            _lib.ptr(q2), _lib.ptr(gc), float(scale), _lib.ptr(token_map), B, T, H, E, NC, _lib.ptr(dkq), _lib.ptr(da),
            _lib.ptr(dc), _lib.ptr(dd), _lib.stream_of(q)), "tgdn_bwd_state_grads")
    return dkq, da, dc, dd


def _run_matrix(q, k, do, dU, W, U, AP, k2, q2, beta, gc, dkq, da, dc, dd, dr, scale, token_map=None):
    """Matrix gradients, mask gradients and final assembly: (dq, dk, dk2, dq2, dg, dbeta)."""
    B, T, H, E, NC = _dims(q, k2, token_map)
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dk2, dq2, dg, db = torch.empty_like(k2), torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(beta)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib.tgdn_bwd_matrix(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(do), _lib.ptr(dU), _lib.ptr(W), _lib.ptr(U), _lib.ptr(AP), _lib.ptr(k2),
            _lib.ptr(q2), _lib.ptr(beta), _lib.ptr(gc), _lib.ptr(dkq), _lib.ptr(da), _lib.ptr(dc), _lib.ptr(dd),
            _lib.ptr(dr), float(scale), _lib.ptr(token_map), B, T, H, E, NC, _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dk2),
            _lib.ptr(dq2), _lib.ptr(dg), _lib.ptr(db), _lib.stream_of(q)), "tgdn_bwd_matrix")
    return dq, dk, dk2, dq2, dg, db


def _kernel_backward(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, do, scale, chunk_starts=None, token_map=None,
                     grad_state_in=None, grad_state_out=None):
    """reverse recurrence -> state gradients -> matrix gradients.  Returns (dq, dk, dv, dk2, dq2, dg, dbeta)."""
    if AP is None:      # GJ_SAVE_MASKS=0: the forward's own kernel again, bitwise identical
        _, AP, Pm = _run_masks(q, k, k2, q2, g, beta, scale, token_map)
    dV, dU, ds, dkg, dr = _run_reverse(q, k, do, k2, q2, beta, gc, AP, Pm, U, scale, chunk_starts, token_map,
                                       grad_state_in, grad_state_out)
    dkq, da, dc, dd = _run_state_grads(q, k, do, dV, h, ds, dkg, k2, q2, gc, scale, token_map)
    del ds, dkg
    dq, dk, dk2, dq2, dg, db = _run_matrix(q, k, do, dU, W, U, AP, k2, q2, beta, gc, dkq, da, dc, dd, dr, scale,
                                           token_map)
    return dq, dk, dV, dk2, dq2, dg, db


def _save_list(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map):
    """Tensors kept for the backward: 14 with the chunk operators, 12 without (GJ_SAVE_MASKS=0)."""
    if _save_masks():
        return (q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map)
    return (q, k, k2, q2, g, beta, gc, h, W, U, chunk_starts, token_map)


def _unpack_saved(saved):
    if len(saved) == 14:
        return saved
    q, k, k2, q2, g, beta, gc, h, W, U, chunk_starts, token_map = saved
    return (q, k, k2, q2, g, beta, gc, None, None, h, W, U, chunk_starts, token_map)


class _JointKernels(torch.autograd.Function):
    """The kernel pipeline as a plain autograd function (reference: ops/gdn_joint.py:201-232, _JointCute)."""

    @staticmethod
    def forward(ctx, q, k, v, k2, q2, g, beta, scale, chunk_starts=None, token_map=None):
        o, gc, AP, Pm, h, W, U = _kernel_forward(q, k, v, k2, q2, g, beta, scale, True, chunk_starts, token_map)
        ctx.save_for_backward(*_save_list(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map))
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, chunk_starts, token_map = _unpack_saved(ctx.saved_tensors)
        grads = _kernel_backward(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, do.contiguous(), ctx.scale,
                                 chunk_starts, token_map)
        return (*(gr if need else None for gr, need in zip(grads, ctx.needs_input_grad)),
                *([None] * (len(ctx.needs_input_grad) - 7)))


class _JointKernelsState(torch.autograd.Function):
    """The kernel pipeline on ONE SEGMENT of longer sequences: the recurrent state comes in and goes out, and so does its
    gradient in the backward (f32 (B, H, E, 128, 128) each).  Dense rows only.  No counterpart in the reference, whose
    sequences always start from a zero state inside one call."""

    @staticmethod
    def forward(ctx, q, k, v, k2, q2, g, beta, state_in, scale):
        B, T, H, _ = q.shape
        E = k2.shape[-1]
        gc, AP, Pm = _run_masks(q, k, k2, q2, g, beta, scale, None)
        state_out = torch.empty((B, H, E, 128, 128), dtype=torch.float32, device=q.device)
        o, h, W, U = _run_forward(q, k, v, k2, q2, beta, gc, AP, scale, True, None, None,
                                  None if state_in is None else state_in.contiguous(), state_out)
        ctx.save_for_backward(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U)
        ctx.scale = scale
        ctx.has_state = state_in is not None
        ctx.set_materialize_grads(False)              # an unused state_out arrives as None, not as a tensor of zeros
        return o, state_out

    @staticmethod
    def backward(ctx, do, dstate_out):
        q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U = ctx.saved_tensors
        B, T, H, _ = q.shape
        E = k2.shape[-1]
        dstate_in = torch.empty((B, H, E, 128, 128), dtype=torch.float32, device=q.device) if ctx.has_state else None
        g_in = None if dstate_out is None else dstate_out.to(torch.float32).contiguous()
        do = torch.zeros((B, T, H, 128), dtype=torch.bfloat16, device=q.device) if do is None else do.contiguous()
        grads = _kernel_backward(q, k, k2, q2, g, beta, gc, AP, Pm, h, W, U, do, ctx.scale, None, None, g_in, dstate_in)
        return (*grads, dstate_in, None)


class _JointKernelsCheckpointed(torch.autograd.Function):
    """Backward state recomputation: the forward keeps only the inputs and the f32 state at every segment boundary
    (E*64 KB per head, sequence and segment) instead of the per-chunk tensors (h: E*32 KB per head and CHUNK of 64 tokens,
    W, U, the chunk operators); the backward walks the segments from the last to the first, runs each segment's forward
    again with everything saved, then its backward, and hands the gradient of the state to the segment before.  Results
    are bitwise those of the plain function; the price is one more masks + forward pass.  Dense rows only."""

    @staticmethod
    def forward(ctx, q, k, v, k2, q2, g, beta, scale, seg_tokens):
        B, T, H, _ = q.shape
        E = k2.shape[-1]
        cuts = list(range(0, T, seg_tokens)) + [T]
        states, outs, state = [], [], None
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            part = [t[:, lo:hi].contiguous() for t in (q, k, v, k2, q2, g, beta)]
            states.append(state)
            gc, AP, _ = _run_masks(part[0], part[1], part[3], part[4], part[5], part[6], scale, None)
            nxt = torch.empty((B, H, E, 128, 128), dtype=torch.float32, device=q.device) if hi < T else None
            outs.append(_run_forward(part[0], part[1], part[2], part[3], part[4], part[6], gc, AP, scale, False, None, None,
                                     state, nxt)[0])
            state = nxt
        ctx.save_for_backward(q, k, v, k2, q2, g, beta, *[s for s in states if s is not None])
        ctx.scale, ctx.cuts = scale, cuts
        return torch.cat(outs, 1)

    @staticmethod
    def backward(ctx, do):
        q, k, v, k2, q2, g, beta, *bounds = ctx.saved_tensors
        states = [None] + list(bounds)
        B, T, H, _ = q.shape
        E = k2.shape[-1]
        grads = [torch.empty_like(t) for t in (q, k, v, k2, q2, g, beta)]
        g_state = None
        for i in reversed(range(len(ctx.cuts) - 1)):
            lo, hi = ctx.cuts[i], ctx.cuts[i + 1]
            pq, pk, pv, pk2, pq2, pg, pb = (t[:, lo:hi].contiguous() for t in (q, k, v, k2, q2, g, beta))
            gc, AP, Pm = _run_masks(pq, pk, pk2, pq2, pg, pb, ctx.scale, None)
            _, h, W, U = _run_forward(pq, pk, pv, pk2, pq2, pb, gc, AP, ctx.scale, True, None, None, states[i], None)
            g_prev = torch.empty((B, H, E, 128, 128), dtype=torch.float32, device=q.device) if i > 0 else None
            part = _kernel_backward(pq, pk, pk2, pq2, pg, pb, gc, AP, Pm, h, W, U, do[:, lo:hi].contiguous(), ctx.scale,
                                    None, None, g_state, g_prev)
            for dst, src in zip(grads, part):
                dst[:, lo:hi] = src
            g_state = g_prev
        return (*grads, None, None)


def chunk_gdn_joint_segment(q, k, v, k2, q2, g, beta, state_in=None, scale=None):
    """One segment of longer sequences, differentiable through the state: returns (o, state_out).  `state_in` (None:
    zero) and `state_out` are f32 (B, H, E, 128, 128), S_e as [key row][value column]; gradients flow into `state_in`
    and out of `state_out`, so that segments chained by their states (on one GPU or, with the states sent between
    ranks, on several: `context_parallel.py`) give the outputs and gradients of the unsplit sequences.  T must be a
    multiple of 64; dense rows only."""
    _check(q, k, v, k2, q2, g, beta, packed=False)
    _check_device_and_e(q, k2.shape[-1])
    B, T, H, _ = q.shape
    E = k2.shape[-1]
    if state_in is not None and (tuple(state_in.shape) != (B, H, E, 128, 128) or state_in.dtype != torch.float32
                                 or state_in.device != q.device):
        raise ValueError(f"state_in must be an f32 tensor of shape {(B, H, E, 128, 128)} on the inputs' device")
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _JointKernelsState.apply(q, k, v, k2, q2, g, beta, state_in, float(scale))


def chunk_gdn_joint(q, k, v, k2, q2, g, beta, scale=None, cu_seqlens=None, reference=False, *, initial_state=None,
                    output_final_state=False, checkpoint_tokens=None):
    """Triadic GDN with autograd for all seven tensor inputs, on the sm_100a kernels.

    Inference that continues a sequence (no counterpart in the reference, whose forward always starts from zero):
    `initial_state` is an f32 (sequences, H, E, 128, 128) tensor, sequences = batch rows or documents, holding S_e as
    [key row][value column]; with `output_final_state=True` the call returns (o, final_state) in the same form.  Both are
    forward-only: they are rejected when a gradient is required.

    With cu_seqlens the inputs are one packed row (1, T, ...): contiguous int32/int64 CUDA offsets that start at 0,
    end at T and strictly increase; document lengths are arbitrary and the state resets at every document start.
    `checkpoint_tokens=S` (training, dense rows): backward state recomputation.  Only the inputs and the f32 state every
    S tokens are kept; the backward recomputes each segment's forward before differentiating it (bitwise the same results,
    one more forward pass, the per-chunk saved tensors of one segment at a time instead of the whole sequence).
    `reference=True` asked the reference package for its torch pipeline; this package ships kernels only (its CPU
    restatement of that pipeline lives with the tests), so the flag is rejected instead of silently running something else.
    """
    if reference:
        raise NotImplementedError("reference=True: this package has no torch fallback; the CPU oracle used by the "
                                  "tests is oracle/triadic_oracle.py")
    _check(q, k, v, k2, q2, g, beta, packed=cu_seqlens is not None)
    _check_device_and_e(q, k2.shape[-1])
    chunk_starts = token_map = None
    if cu_seqlens is not None:
        from .joint_packing import prepare_documents
        chunk_starts, token_map = prepare_documents((q, k, v, k2, q2, g, beta), cu_seqlens)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, k2, q2, g, beta))
    if initial_state is not None or output_final_state:
        if needs_grad:
            raise ValueError("initial_state / output_final_state are forward-only: run them under torch.no_grad()")
        B, T, H, _ = q.shape
        E = k2.shape[-1]
        n_seq = B if cu_seqlens is None else cu_seqlens.numel() - 1
        shape = (n_seq, H, E, 128, 128)
        if initial_state is not None:
            if tuple(initial_state.shape) != shape or initial_state.dtype != torch.float32 or initial_state.device != q.device:
                raise ValueError(f"initial_state must be an f32 tensor of shape {shape} on the inputs' device")
            initial_state = initial_state.contiguous()
        final = torch.empty(shape, dtype=torch.float32, device=q.device) if output_final_state else None
        gc, AP, _ = _run_masks(q, k, k2, q2, g, beta, float(scale), token_map)
        o = _run_forward(q, k, v, k2, q2, beta, gc, AP, float(scale), False, chunk_starts, token_map, initial_state, final)[0]
        return (o, final) if output_final_state else o
    if needs_grad and checkpoint_tokens is not None:
        if cu_seqlens is not None:
            raise ValueError("checkpoint_tokens: dense rows only (a packed row is already cut at its documents)")
        seg = int(checkpoint_tokens)
        if seg <= 0 or seg % CHUNK:
            raise ValueError(f"checkpoint_tokens must be a positive multiple of {CHUNK}")
        if seg < q.shape[1]:
            return _JointKernelsCheckpointed.apply(q, k, v, k2, q2, g, beta, float(scale), seg)
    if needs_grad:
        return _JointKernels.apply(q, k, v, k2, q2, g, beta, float(scale), chunk_starts, token_map)
    return _kernel_forward(q, k, v, k2, q2, g, beta, float(scale), False, chunk_starts, token_map)[0]


def gdn_joint_decode(q, k, v, k2, q2, g, beta, state, scale=None):
    """One token per sequence on a resident state (decode).  No counterpart in the reference.

    q, k, v: bf16 (B, 1, H, 128) or (B, H, 128); k2, q2, g: f32 (B, 1, H, E) or (B, H, E); beta: f32 (B, 1, H) or (B, H);
    `state`: contiguous f32 (B, H, E, 128, 128), the form `chunk_gdn_joint(..., output_final_state=True)` returns; it is
    updated IN PLACE.  Returns o in the shape of v.  Forward only."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, k2, q2, g, beta, state)):
        raise ValueError("gdn_joint_decode is forward-only: run it under torch.no_grad()")
    squeeze = q.dim() == 4
    if squeeze:
        if q.shape[1] != 1:
            raise ValueError("gdn_joint_decode takes one token per sequence: T must be 1")
        q, k, v, k2, q2, g, beta = (t[:, 0] for t in (q, k, v, k2, q2, g, beta))
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must be (B, H, 128) (or (B, 1, H, 128)) and agree")
    B, H, _ = q.shape
    E = k2.shape[-1]
    if tuple(k2.shape) != (B, H, E) or q2.shape != k2.shape or g.shape != k2.shape or tuple(beta.shape) != (B, H):
        raise ValueError("k2, q2, g must be (B, H, E) and beta (B, H)")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v)) or any(t.dtype != torch.float32 for t in (k2, q2, g, beta)):
        raise ValueError("q, k, v must be bfloat16 and k2, q2, g, beta float32")
    _check_device_and_e(q, E)
    if tuple(state.shape) != (B, H, E, 128, 128) or state.dtype != torch.float32 or state.device != q.device \
            or not state.is_contiguous():
        raise ValueError(f"state must be a contiguous f32 tensor of shape {(B, H, E, 128, 128)} on the inputs' device")
    scale = HEAD_DIM ** -0.5 if scale is None else scale
    q, k, v, k2, q2, g, beta = (t.contiguous() for t in (q, k, v, k2, q2, g, beta))
    o = torch.empty_like(v)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib.tgdn_decode_step(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(k2), _lib.ptr(q2), _lib.ptr(g),
                                             _lib.ptr(beta), float(scale), B, H, E, _lib.ptr(state), _lib.ptr(o),
                                             _lib.stream_of(q)), "tgdn_decode_step")
    return o[:, None] if squeeze else o
