"""Benchmark of the Triadic GDN hot path: forward + backward tokens/s at T=8192, H=32, E=8, B=8 (heads sharded over N GPUs).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|conv]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One step = one forward + backward of the whole (B, T, H) problem through `gdn_joint_call` (the public API).  Prints ONE
JSON line from rank 0.  `value` is timed with the inputs resident in HBM; `e2e` repeats the measurement with the
inputs in pinned host memory, copied to the device every step, and the output and all seven gradients copied back.
`roofline` describes the kernel with the largest share of the step; `cpu_baseline` times the CPU oracle (a port of the
reference's torch path) on a bounded sample; `parity` compares seeded (batch row | document, head) slices of the
full-size run with that oracle and fails the run when a tolerance is broken; `aux` carries the second mode of the headline
configuration (GJ_SAVE_MASKS=0) and the convolution pre-pass; `reference_kernels` is what the reference's own CuTe-DSL
kernels did on this GPU (baseline/time_reference_kernels.py).  `--impl reference` times the CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

U_FLOP = 2 * 64 * 64 * 128          # one 64x64x128 product

WORKLOADS = {
    # name: (B, T, H, E, backward)
    "c2": (8, 8192, 32, 8, True),
    "c1": (4, 4096, 16, 4, False),
    "c3": (1, 131072, 16, 16, True),    # one packed row of lognormal documents (PACKED below)
    "small": (2, 1024, 4, 8, True),
    "c4": (1, 32768, 32, 12, True),     # the core behind the conv pre-pass: eight documents of 4096 tokens (PACKED below)
    "prof": (2, 8192, 16, 8, True),     # 4096 (chunk, head) items, a few GB: the size used for ncu captures
    "prof16": (2, 4096, 16, 16, True),  # 2048 items with sixteen slices, a few GB: the second ncu size
}


def algorithmic_flops(E, items, backward):
    """(15 + 18E) u per (chunk, head) forward + backward, (4 + 6E) u forward only."""
    per = (4 + 6 * E) + ((11 + 12 * E) if backward else 0)
    return per * U_FLOP * items


PACKED = {"c3": ("lognormal", 31), "c4": ("uniform", 4096)}   # workload -> how its packed row is cut into documents

# per-kernel algorithmic work, in u per (chunk, head)
KERNEL_U = {
    "masks": lambda E: 2, "fwd": lambda E: 2 + 6 * E, "rec": lambda E: 3 + 6 * E, "sg": lambda E: 6 * E, "mat": lambda E: 8,
}

# DRAM bytes (read + write) per (chunk, head) item and launch, from ncu captures of each kernel at E = 8 (the `prof`
# workload, 4096 items) and at E = 16 (B=2, T=4096, H=16: 2048 items).  Traffic grows in proportion to the item count and,
# between the two captures, linearly in E (the saved states are E * 32 KB per item), so other E are interpolated (E = 12
# shares the eight value blocks of E = 16 where E = 8 has four: its rec and sg figures come out about 64 KB per item low).
NCU_DRAM_BYTES_PER_ITEM = {
    # kernel: (bytes per item at E = 8, at E = 16); filled from profiles/core_kernels_prof_workload.md
    "masks": (0.255e9 / 4096, 0.135e9 / 2048), "fwd": (1.518e9 / 4096, 1.282e9 / 2048), "rec": (0.751e9 / 4096, 0.549e9 / 2048),
    "sg": (1.865e9 / 4096, 1.574e9 / 2048), "mat": (0.824e9 / 4096, 0.495e9 / 2048),
}

# DRAM bytes (read + write) per element of the conv kernels, from one ncu capture at (1, 8192, 13056)
# (part of the written lines still sat in L2 when the kernel ended).
NCU_DRAM_BYTES_PER_ELEMENT_CONV = {"fwd": (215.9 + 162.0) * 1e6 / (8192 * 13056), "bwd": (431.6 + 184.2) * 1e6 / (8192 * 13056)}


def ncu_traffic(name, E, items):
    lo, hi = NCU_DRAM_BYTES_PER_ITEM[name]
    return (lo + (hi - lo) * (E - 8) / 8.0) * items


# HBM bytes per (chunk, head) item that each kernel of THIS decomposition must read or write once (bf16 tiles of 64x128
# are 16 KB; a state slice is 32 KB; NV = value blocks of the reverse recurrence).  The saved forward states h (E * 32 KB
# written by fwd, read by sg) and the value-block images of the reverse recurrence are consequences of the decomposition,
# not of the algorithm: `io_bytes` below counts only what the algorithm itself must move.
def kernel_bytes(name, E):
    K, NV, gates = 1024, (8 if E > 8 else 4), 3 * 64 * E * 4
    packed = (256 * E + 16) * 4            # the gate tensor of the masks kernel: gc, a, r, c (64 x E each) and d
    factors = packed - 64 * E * 4          # what the recurrences fetch of it: a, r, c, d
    return {
        "masks": 32 * K + gates + 256 + packed + 24 * K,
        "fwd": 48 * K + 16 * K + factors + 256 + 48 * K + 32 * K * E,
        "rec": 64 * K + 16 * K + factors + 256 + 32 * K + NV * 16 * K + NV * 64 * E * 4,
        "sg": 64 * K + 32 * K * E + NV * 16 * K + 2 * 64 * E * 4 + 4 * E + 32 * K + 2 * 64 * E * 4 + 4 * E,
        "mat": 96 * K + 16 * K + 32 * K + gates + 256 + 2 * 64 * E * 4 + 4 * E + NV * 64 * E * 4 + 32 * K + gates + 256,
    }[name]


def io_bytes(E):
    """Inputs and outputs of the whole forward + backward per (chunk, head): q, k, v, dO, o, dq, dk, dv (bf16 tiles),
    k2, q2, g and their gradients, beta and its gradient."""
    return 8 * 16 * 1024 + 6 * 64 * E * 4 + 2 * 256


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"tflops": d.get("bf16_tflops"), "tflops_sustained": d.get("bf16_tflops_sustained", d.get("bf16_tflops")),
                "gbs": d.get("hbm_gbs"), "kind": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "gbs": 6650.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[1]) for r in self.rows if len(r) >= 9 and r[1].isdigit())
        mx = [int(r[2]) for r in self.rows if len(r) >= 9 and r[2].isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _l2norm(t):
    return t * torch.rsqrt((t * t).sum(-1, keepdim=True) + 1e-6)


def host_inputs(B, T, H, E, seed=0):
    """Seeded synthetic inputs of the BASELINE distribution, generated on the CPU in fp32 and then cast:
    q, k = l2norm(N(0,1)) bf16; v = N(0,1) bf16; k2, q2 = l2norm(N(0,1)) over E; g = -softplus(N(0,1)); beta = sigmoid(N(0,1));
    dO = N(0,1) bf16.  One generator, draw order q, k, v, k2, q2, g, beta, dO."""
    gen = torch.Generator().manual_seed(int(seed))
    r = lambda *shape: torch.randn(*shape, generator=gen)
    q = _l2norm(r(B, T, H, 128)).to(torch.bfloat16)
    k = _l2norm(r(B, T, H, 128)).to(torch.bfloat16)
    v = r(B, T, H, 128).to(torch.bfloat16)
    k2 = _l2norm(r(B, T, H, E))
    q2 = _l2norm(r(B, T, H, E))
    g = -torch.nn.functional.softplus(r(B, T, H, E))
    beta = torch.sigmoid(r(B, T, H))
    do = r(B, T, H, 128).to(torch.bfloat16)
    return [t.contiguous() for t in (q, k, v, k2, q2, g, beta)], do


def lognormal_documents(T, seed, median=2048.0, sigma=1.0):
    """cu_seqlens of a packed row: document lengths max(1, round(lognormal(ln median, sigma))) from a seeded numpy
    generator, drawn until they cover T, the last one truncated."""
    import math
    import numpy as np
    rng = np.random.default_rng(int(seed))
    cu = [0]
    while cu[-1] < T:
        cu.append(min(T, cu[-1] + max(1, int(round(float(rng.lognormal(math.log(median), sigma)))))))
    return torch.tensor(cu, dtype=torch.int32)


def cpu_reference_rate(B, T, H, E, backward, budget_s=20.0, threads=None):
    """tokens/s of the CPU oracle, from as many (batch row, head) slices of the workload as fit the time budget."""
    from oracle import triadic_oracle as orc
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    Ts = min(T, 16384)                                # long rows: a 16k-token piece, scaled linearly (the algorithm is linear in T)
    done, t_used = 0, 0.0
    while True:
        ins = orc.make_inputs(1, Ts, 1, E, seed=100 + done)
        do = orc.make_grad_output((1, Ts, 1, 128), 7)
        t0 = time.perf_counter()
        if backward:
            orc.reference_with_grads(orc.chunk_reference, ins, do, dtype=torch.float32)
        else:
            with torch.no_grad():
                orc.chunk_reference(*ins, dtype=torch.float32)
        t_used += time.perf_counter() - t0
        done += 1
        if t_used > budget_s or done >= B * H:
            break
    per_slice = t_used / done
    rate = B * Ts / (per_slice * B * H)               # tokens of the whole job per second: slices are independent
    return rate, done, threads, per_slice


def workload_name(name):
    B, T, H, E, backward = WORKLOADS[name]
    packed = ("packed, " + PACKED[name][0] + " documents, ") if name in PACKED else ""
    return f"{name}: B={B} T={T} H={H} E={E} {packed}{'fwd+bwd' if backward else 'fwd'}"


def run_reference(args, rank, world):
    B, T, H, E, backward = WORKLOADS[args.workload]
    if rank != 0:
        return
    steps, rates = max(1, args.steps), []
    sample = None
    for _ in range(args.warmup + steps):
        rate, n, threads, per_slice = cpu_reference_rate(B, T, H, E, backward, budget_s=max(2.0, 40.0 / (args.warmup + steps)))
        rates.append(rate)
        sample = f"{n} of {B * H} (batch row, head) slices of T={min(T, 16384)} per step, scaled linearly"
    rates = rates[args.warmup:]
    value = sum(rates) / len(rates)
    line = {"impl": "reference", "metric": "fwd+bwd tokens/s" if backward else "fwd tokens/s", "value": value,
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * B * T / value, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.workload),
                       "path": "CPU port of the reference torch path (oracle/triadic_oracle.py); a GPU-over-CPU ratio, not a kernel comparison"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def stage_times(leaves, do, E, cu_dev=None, reps=3):
    """Per-kernel device time (ms) of one forward + backward: CUDA events around each C-ABI call on torch's stream; the
    median of `reps` repetitions (a repetition in which the caching allocator had to go to cudaMalloc between two events
    would otherwise charge those milliseconds to a kernel)."""
    from cute_triadic_gdn_b200 import gdn_joint as gj
    q, k, v, k2, q2, g, beta = [t.detach() for t in leaves]
    scale = 128 ** -0.5
    cs = tm = None
    if cu_dev is not None:
        from cute_triadic_gdn_b200.joint_packing import prepare_documents
        cs, tm = prepare_documents((q, k, v, k2, q2, g, beta), cu_dev)
    names = ["masks", "fwd", "rec", "sg", "mat"]
    acc = {n: [] for n in names}
    for rep in range(reps + 1):                        # the first repetition warms the allocator and is dropped
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        ev[0].record()
        gc, AP, Pm = gj._run_masks(q, k, k2, q2, g, beta, scale, tm)
        ev[1].record()
        o, h, W, U = gj._run_forward(q, k, v, k2, q2, beta, gc, AP, scale, True, cs, tm)
        ev[2].record()
        dV, dU, ds, dkg, dr = gj._run_reverse(q, k, do, k2, q2, beta, gc, AP, Pm, U, scale, cs, tm)
        ev[3].record()
        dkq, da, dc, dd = gj._run_state_grads(q, k, do, dV, h, ds, dkg, k2, q2, gc, scale, tm)
        ev[4].record()
        gj._run_matrix(q, k, do, dU, W, U, AP, k2, q2, beta, gc, dkq, da, dc, dd, dr, scale, tm)
        ev[5].record()
        torch.cuda.synchronize()
        if rep > 0:
            for i, n in enumerate(names):
                acc[n].append(ev[i].elapsed_time(ev[i + 1]))
        del h, ds, dkg, dkq, W, U, dU, o
    return {n: sorted(acc[n])[len(acc[n]) // 2] for n in names}


PARITY_TOL = {"o": 1e-2, "grad": 2e-2}                 # relative L2 against an fp32 run of the reference math


def parity_check(ins, do, o_dev, grads_dev, cu_host, seed=0, n_slices=2):
    """Compares seeded slices of the full-size device result with the CPU oracle (oracle/triadic_oracle.py, the fp32
    restatement of the reference's torch path).  Dense rows: (batch row, head) slices, which are independent problems.
    Packed rows: (document, head) slices, the longest document among them.  Returns the worst relative L2 errors."""
    from oracle import triadic_oracle as orc
    gen = torch.Generator().manual_seed(int(seed))
    B, T, H = ins[0].shape[:3]
    picks = []
    if cu_host is None:
        while len(picks) < n_slices:
            c = (int(torch.randint(B, (1,), generator=gen)), 0, T, int(torch.randint(H, (1,), generator=gen)))
            if c not in picks:
                picks.append(c)
    else:
        lens = (cu_host[1:] - cu_host[:-1]).tolist()
        docs = [max(range(len(lens)), key=lambda d: lens[d])]
        while len(docs) < min(n_slices, len(lens)):
            d = int(torch.randint(len(lens), (1,), generator=gen))
            if d not in docs:
                docs.append(d)
        picks = [(0, int(cu_host[d]), int(cu_host[d + 1]), int(torch.randint(H, (1,), generator=gen))) for d in docs]
    worst_o, worst_g, which = 0.0, 0.0, []
    torch.set_num_threads(os.cpu_count() or 1)
    for (b, lo, hi, h) in picks:
        sl = lambda t: t[b:b + 1, lo:hi, h:h + 1].contiguous()
        cu = None if (hi - lo) % 64 == 0 else torch.tensor([0, hi - lo], dtype=torch.int32)
        if grads_dev is None:                                  # forward-only workload
            o_ref, eg = orc.chunk_reference(*[sl(t) for t in ins], cu_seqlens=cu, dtype=torch.float32), 0.0
        else:
            o_ref, g_ref = orc.reference_with_grads(orc.chunk_reference, [sl(t) for t in ins], sl(do), cu_seqlens=cu, dtype=torch.float32)
            eg = max(orc.rel_l2(sl(gd).float().cpu(), gr) for gd, gr in zip(grads_dev, g_ref))
        eo = orc.rel_l2(sl(o_dev).float().cpu(), o_ref)
        worst_o, worst_g = max(worst_o, eo), max(worst_g, eg)
        which.append({"row": b, "tokens": [lo, hi], "head": h, "o": eo, "max_grad": eg})
    return {"o": worst_o, "max_grad": worst_g, "slices": which, "tolerance": PARITY_TOL,
            "against": "oracle/triadic_oracle.py chunk_reference, fp32, same seeded inputs",
            "ok": worst_o < PARITY_TOL["o"] and worst_g < PARITY_TOL["grad"]}


def conv_rates(dev, T=32768, C=13056, act=12288, reps=5):
    """Achieved GB/s of the convolution pre-pass of configuration 4 at its own size (algorithmic bytes: forward 4*T*C,
    backward 6*T*C), a few launches outside every other timed region."""
    from cute_triadic_gdn_b200 import conv_split_act_call
    from cute_triadic_gdn_b200.conv_split_act import conv_split_act_bwd
    x = torch.randn(1, T, C, device=dev).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, device=dev)).to(torch.bfloat16)
    dy = torch.randn(1, T, C, device=dev).to(torch.bfloat16)
    cu = torch.arange(0, T + 1, 4096, device=dev, dtype=torch.int32)

    def ev_time(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    with torch.no_grad():
        f = ev_time(lambda: conv_split_act_call(x, w, act, cu))
        bw = ev_time(lambda: conv_split_act_bwd(x, dy, w, act, cu))
    return 4 * T * C / (f * 1e-3) / 1e9, 6 * T * C / (bw * 1e-3) / 1e9, f, bw


def glue_rates(dev, T=32768, H=32, E=12, reps=5, unfused_too=True):
    """Achieved GB/s of the convolution with the layer glue fused in, at the shape of configuration 4 (C = 13056).
    Algorithmic bytes: forward x in, q, k, v (bf16) and k2, q2 (f32) out; backward x and the five gradients in, dx out
    (the gradient of the convolution's output, which the backward writes and reads once in between, is not counted)."""
    from cute_triadic_gdn_b200 import conv_split_norm_call
    from cute_triadic_gdn_b200.conv_split_act import conv_split_norm_bwd
    C = H * (3 * 128 + 2 * E)
    x = torch.randn(1, T, C, device=dev).to(torch.bfloat16)
    w = (0.5 * torch.randn(C, 4, device=dev)).to(torch.bfloat16)
    cu = torch.arange(0, T + 1, 4096, device=dev, dtype=torch.int32)
    grads = [torch.randn(1, T, H, 128, device=dev).to(torch.bfloat16) for _ in range(3)] + \
            [torch.randn(1, T, H, E, device=dev) for _ in range(2)]

    def ev_time(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def unfused():                     # what a caller of the plain convolution runs after it: split, activations, norms
        from cute_triadic_gdn_b200 import conv_split_act_call
        y = conv_split_act_call(x, w, 3 * H * 128, cu)
        yq, yk, yv, yk2, yq2 = y.split([H * 128, H * 128, H * 128, H * E, H * E], dim=-1)
        l2 = lambda t: t * torch.rsqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        q, k = (l2(t.float().view(1, T, H, 128)).to(torch.bfloat16) for t in (yq, yk))
        k2, q2 = (l2(torch.nn.functional.softplus(t.float()).view(1, T, H, E)) for t in (yk2, yq2))
        return q, k, yv.reshape(1, T, H, 128).contiguous(), k2, q2

    with torch.no_grad():
        f = ev_time(lambda: conv_split_norm_call(x, w, H, E, cu))
        bw = ev_time(lambda: conv_split_norm_bwd(x, w, *grads, H, E, 1e-6, cu))
        uf = ev_time(unfused) if unfused_too else None
    out_bytes = T * H * (3 * 128 * 2 + 2 * E * 4)
    return (2 * T * C + out_bytes) / (f * 1e-3) / 1e9, (4 * T * C + out_bytes) / (bw * 1e-3) / 1e9, f, bw, uf


def decode_rate(dev, B=32, H=32, E=8, reps=10):
    """Achieved GB/s of the one-token decode step at the head count and slice count of configuration 2, 32 sequences: the
    state (B*H*E*64 KB f32 = 537 MB, four times L2, so that little of it survives in L2 from token to token) is read once
    and written once per token; everything else is a few KB."""
    from cute_triadic_gdn_b200 import gdn_joint_decode
    gen = torch.Generator(device=dev).manual_seed(3)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    q, k, v = (rn(B, H, 128).to(torch.bfloat16) for _ in range(3))
    k2, q2 = rn(B, H, E), rn(B, H, E)
    g, beta = -torch.nn.functional.softplus(rn(B, H, E)), torch.sigmoid(rn(B, H))
    state = torch.zeros(B, H, E, 128, 128, device=dev)
    with torch.no_grad():
        for _ in range(3):
            gdn_joint_decode(q, k, v, k2, q2, g, beta, state)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            gdn_joint_decode(q, k, v, k2, q2, g, beta, state)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return 2 * state.numel() * 4 / (ms * 1e-3) / 1e9, ms


def reference_kernel_timing(timeout_s=420):
    """What the reference's own CuTe-DSL kernels do on this GPU, measured by baseline/time_reference_kernels.py in a child
    process (a compile failure of the DSL must not take the bench down).  Needs the reference installed under
    baseline/_ref; otherwise, or when the child fails, says why."""
    script = os.path.join(ROOT, "baseline", "time_reference_kernels.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "cute_triadic_gdn")):
        return {"ok": False, "unavailable": "baseline/_ref does not hold the reference package"}
    try:
        r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"ok": False, "unavailable": f"no result within {timeout_s} s"}
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            out = json.loads(line)["reference_kernels"]
            out.pop("trace_tail", None)
            return out
    return {"ok": False, "unavailable": f"child exited {r.returncode}: {r.stderr[-300:]}"}


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from cute_triadic_gdn_b200 import _lib, gdn_joint_call
    from cute_triadic_gdn_b200.sharding import document_ranges, head_slice
    B, T, H, E, backward = WORKLOADS[args.workload]
    packed = args.workload in PACKED
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    cu_host = cu_dev = None
    if packed:
        # one packed row: this rank takes a token-balanced range of whole documents, all heads (strong scaling)
        kind, arg = PACKED[args.workload]
        cu_all = lognormal_documents(T, arg) if kind == "lognormal" else torch.arange(0, T + 1, arg, dtype=torch.int32)
        rng = document_ranges(cu_all, world)[rank]
        if rng.doc_hi == rng.doc_lo:
            raise SystemExit(f"rank {rank} of {world} got no document")
        cu_host = (cu_all[rng.doc_lo:rng.doc_hi + 1] - cu_all[rng.doc_lo]).contiguous()
        cu_dev = cu_host.to(dev)
        Tl, Hl = rng.tok_hi - rng.tok_lo, H
        chunks = int(((cu_host[1:] - cu_host[:-1] + 63) // 64).sum())
    else:
        if H % world:
            raise SystemExit(f"H={H} is not divisible by {world} GPUs")
        hs = head_slice(H, world, rank)               # heads of this rank (strong scaling: total work fixed)
        Tl, Hl = T, hs.stop - hs.start
        chunks = B * (T // 64)
    ins, do = host_inputs(B, Tl, Hl, E, seed=1000 + rank)
    # pinned buffers are allocated after the rank has moved to the cores of its GPU's NUMA node (where sysfs says which)
    from cute_triadic_gdn_b200.host_pipeline import bind_host_to_gpu
    numa = bind_host_to_gpu(local_rank)
    pinned = [t.pin_memory() for t in ins]
    do_pinned = do.pin_memory()
    leaves = [t.to(dev).requires_grad_(backward) for t in ins]
    do_dev = do.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        for t in leaves:
            t.grad = None
        o = gdn_joint_call(*leaves, cu_seqlens=cu_dev)
        if backward:
            o.backward(do_dev)
        return o

    # end to end through the host-resident entry point: pinned host inputs -> device -> kernels -> pinned host results,
    # with the three stages of successive batch slices overlapping
    from cute_triadic_gdn_b200 import HostPipeline
    pipe = HostPipeline(pinned, do_pinned if backward else None, slices=8 if packed else B, cu_seqlens=cu_host)

    def step_e2e():
        return pipe.run(pinned, do_pinned if backward else None)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = timed(step_resident, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"metric": "fwd+bwd tokens/s" if backward else "fwd tokens/s", "value": B * T * args.steps / (ms * 1e-3), "unit": "tokens/s",
                              "ms_per_step": ms / args.steps, "config": {"workload": args.workload}, "kernels_only": True}))
        return
    ms_e2e = timed(step_e2e, args.steps, max(1, args.warmup // 2))
    status = _lib.device_status()

    tokens = B * T
    value = tokens * args.steps / (ms * 1e-3)
    e2e_value = tokens * args.steps / (ms_e2e * 1e-3)
    h2d, d2h = int(pipe.h2d_bytes), int(pipe.d2h_bytes)       # counted from the tensors the pipeline copies
    if rank != 0:
        return

    pk = peaks()
    items = chunks * Hl                               # (chunk, head) items of this rank
    step_s = ms / args.steps * 1e-3
    roof = None
    if backward:
        st = stage_times(leaves, do_dev, E, cu_dev)
        total = sum(st.values())
        top = max(st, key=st.get)
        flops = KERNEL_U[top](E) * U_FLOP * items
        achieved = flops / (st[top] * 1e-3) / 1e12
        step_tf = algorithmic_flops(E, items * world, True) / step_s / 1e12     # whole job: every rank's items in the max-over-ranks time
        kb = {k: kernel_bytes(k, E) * items for k in st}
        roof = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                "frac": achieved / pk["tflops"], "peak_name": "bf16_tflops (burst): the kernel is timed alone",
                "traffic": ncu_traffic(top, E, items), "peak_kind": pk["kind"],
                "kernel_ms": {k: round(v, 3) for k, v in st.items()}, "share": round(st[top] / total, 3),
                "step_achieved": step_tf,
                "step_frac": step_tf / (pk["tflops"] * world), "step_peak_name": "bf16_tflops (burst) x GPUs",
                "step_frac_sustained": step_tf / (pk["tflops_sustained"] * world),
                "hbm": {"kernel_gbs": kb[top] / (st[top] * 1e-3) / 1e9, "kernel_frac": kb[top] / (st[top] * 1e-3) / 1e9 / pk["gbs"],
                        "step_gbs": sum(kb.values()) / step_s / 1e9, "step_frac": sum(kb.values()) / step_s / 1e9 / pk["gbs"],
                        "step_bytes_this_decomposition": sum(kb.values()), "step_bytes_algorithm_io": io_bytes(E) * items,
                        "step_traffic_ncu": sum(ncu_traffic(k, E, items) for k in st),
                        "peak": pk["gbs"], "unit": "GB/s",
                        "bytes": "kernel_bytes(): what this decomposition must move; io_bytes(): inputs and outputs of the algorithm only"}}
    else:
        # forward only: masks and the forward recurrence, CUDA events around each call
        from cute_triadic_gdn_b200 import gdn_joint as gj
        qd, kd, vd, k2d, q2d, gd, bd = [t.detach() for t in leaves]
        tm = cs = None
        if cu_dev is not None:
            from cute_triadic_gdn_b200.joint_packing import prepare_documents
            cs, tm = prepare_documents(tuple(t.detach() for t in leaves), cu_dev)
        times = {"masks": [], "fwd": []}
        for rep in range(4):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            gcx, APx, Pmx = gj._run_masks(qd, kd, k2d, q2d, gd, bd, 128 ** -0.5, tm)
            ev[1].record()
            gj._run_forward(qd, kd, vd, k2d, q2d, bd, gcx, APx, 128 ** -0.5, False, cs, tm)
            ev[2].record()
            torch.cuda.synchronize()
            if rep > 0:
                times["masks"].append(ev[0].elapsed_time(ev[1]))
                times["fwd"].append(ev[1].elapsed_time(ev[2]))
        st = {k: sorted(v)[len(v) // 2] for k, v in times.items()}
        top = max(st, key=st.get)
        achieved = KERNEL_U[top](E) * U_FLOP * items / (st[top] * 1e-3) / 1e12
        step_tf = algorithmic_flops(E, items * world, False) / step_s / 1e12
        roof = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                "frac": achieved / pk["tflops"], "peak_name": "bf16_tflops (burst): the kernel is timed alone",
                "traffic": ncu_traffic(top, E, items), "peak_kind": pk["kind"],
                "kernel_ms": {k: round(v, 3) for k, v in st.items()}, "share": round(st[top] / sum(st.values()), 3),
                "step_achieved": step_tf, "step_frac": step_tf / (pk["tflops"] * world),
                "step_peak_name": "bf16_tflops (burst) x GPUs", "step_frac_sustained": step_tf / (pk["tflops_sustained"] * world),
                "note": "inference forward: the saved states are not written, the ncu traffic figure (training forward) is an upper bound"}
    # parity at the size that was timed: seeded slices of the last resident step against the CPU oracle
    parity = None
    if not args.no_parity:
        o_dev = step_resident()
        torch.cuda.synchronize()
        parity = parity_check(ins, do, o_dev, [t.grad for t in leaves] if backward else None, cu_host, seed=args.steps)
    # the second mode of the headline configuration and the convolution pre-pass, a few launches each
    aux = {}
    if backward and not args.no_aux and world == 1:
        prev = os.environ.get("GJ_SAVE_MASKS")
        os.environ["GJ_SAVE_MASKS"] = "0" if prev != "0" else "1"
        other = os.environ["GJ_SAVE_MASKS"]
        try:
            aux[f"save_masks{other}_ms_per_step"] = timed(step_resident, 3, 2) / 3
        finally:
            if prev is None:
                os.environ.pop("GJ_SAVE_MASKS")
            else:
                os.environ["GJ_SAVE_MASKS"] = prev
    if backward and not args.no_aux and world == 1 and not packed:
        # backward state recomputation: only the state every 2048 tokens is kept, every segment's forward runs twice
        from cute_triadic_gdn_b200 import chunk_gdn_joint

        def step_checkpointed():
            for t in leaves:
                t.grad = None
            chunk_gdn_joint(*leaves, checkpoint_tokens=2048).backward(do_dev)
        aux["checkpoint2048_ms_per_step"] = timed(step_checkpointed, 3, 2) / 3
    del pipe
    for t in leaves:
        t.grad = None
    if world == 1 and not args.no_aux:
        del leaves, do_dev
        torch.cuda.empty_cache()
        fg, bg, fms, bms = conv_rates(dev)
        aux.update({"conv_fwd_gbs": fg, "conv_bwd_gbs": bg, "conv_fwd_ms": fms, "conv_bwd_ms": bms,
                    "conv_frac": fg / pk["gbs"], "conv_bwd_frac": bg / pk["gbs"],
                    "conv_workload": "x (1, 32768, 13056) bf16, 8 documents, SiLU on 12288 channels; bytes 4*T*C forward, 6*T*C backward"})
        gf, gb, gfms, gbms, ufms = glue_rates(dev)
        aux.update({"glue_fwd_gbs": gf, "glue_bwd_gbs": gb, "glue_fwd_ms": gfms, "glue_bwd_ms": gbms,
                    "unfused_glue_fwd_ms": ufms,
                    "glue_fwd_frac": gf / pk["gbs"], "glue_bwd_frac": gb / pk["gbs"],
                    "glue_workload": "conv_split_norm_call at x (1, 32768, 13056), H=32, E=12, 8 documents: x -> q, k, v, k2, q2"})
        dg, dms = decode_rate(dev)
        aux.update({"decode_gbs": dg, "decode_us_per_token": dms * 1e3, "decode_frac": dg / pk["gbs"],
                    "decode_workload": "one token, B=32 H=32 E=8: state 537 MB f32 read and written once"})
    cpu_rate, n_slices, threads, per_slice = cpu_reference_rate(B, T, H, E, backward, budget_s=15.0)
    refk = reference_kernel_timing() if (world == 1 and not args.no_reference_kernels) else None
    line = {"metric": "fwd+bwd tokens/s" if backward else "fwd tokens/s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args.workload),
                       "save_masks": os.environ.get("GJ_SAVE_MASKS", "1"),
                       "parallelism": (f"whole documents, token-balanced, over {world} GPU(s), no collective" if packed
                                       else f"heads sharded over {world} GPU(s), no collective"),
                       "l2": "inputs larger than L2",
                       "api": "gdn_joint_call + backward; e2e: HostPipeline (pinned host tensors, batch slices overlapped on three streams)"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps,
                    "h2d_gbs": h2d / (ms_e2e / args.steps * 1e-3) / 1e9, "d2h_gbs": d2h / (ms_e2e / args.steps * 1e-3) / 1e9,
                    "host_numa": numa},
            "gpu_launches": args.steps * (5 if backward else 2),
            "clocks": clocks, "roofline": roof, "parity": parity, "aux": aux, "device_status": status,
            "reference_kernels": refk,
            "cpu_baseline": {"value": cpu_rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{n_slices} of {B * H} (batch row, head) slices of T={min(T, 16384)}, {per_slice:.2f} s each, scaled linearly"}}
    print(json.dumps(line))
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"parity broken at benchmark size: {parity}")


def run_conv(args):
    """Secondary workload: the convolution pre-pass at (1, T, 13056), T = 32768 unless --tokens says otherwise; HBM roofline."""
    from cute_triadic_gdn_b200 import conv_split_act_call
    dev = torch.device("cuda", 0)
    T, C, act = (args.tokens or 32768), 13056, 12288
    if T % 4096:
        raise SystemExit("--tokens must be a multiple of 4096 (documents of 4096 tokens)")
    x = torch.randn(1, T, C, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (0.5 * torch.randn(C, 4, device=dev)).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(1, T, C, device=dev).to(torch.bfloat16)
    cu = torch.arange(0, T + 1, 4096, device=dev, dtype=torch.int32)
    n_docs = T // 4096

    def ev_time(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    with torch.no_grad():
        fwd_ms = ev_time(lambda: conv_split_act_call(x, w, act, cu), args.steps)
    y = conv_split_act_call(x, w, act, cu)
    from cute_triadic_gdn_b200.conv_split_act import conv_split_act_bwd
    bwd_ms = ev_time(lambda: conv_split_act_bwd(x.detach(), dy, w.detach(), act, cu), args.steps)
    pk = peaks()
    fb, bb = 4 * T * C, 6 * T * C
    line = {"metric": "conv_split_act GB/s", "value": fb / (fwd_ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": 3, "ms_per_step": fwd_ms, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": f"conv (1,{T},{C}) act={act}, {n_docs} documents"},
            "roofline": {"bound": "hbm", "kernel": "conv_fwd", "achieved": fb / (fwd_ms * 1e-3) / 1e9, "peak": pk["gbs"],
                         "unit": "GB/s", "frac": fb / (fwd_ms * 1e-3) / 1e9 / pk["gbs"],
                         "traffic": NCU_DRAM_BYTES_PER_ELEMENT_CONV["fwd"] * T * C, "peak_kind": pk["kind"]},
            "conv_bwd": {"ms": bwd_ms, "achieved": bb / (bwd_ms * 1e-3) / 1e9, "frac": bb / (bwd_ms * 1e-3) / 1e9 / pk["gbs"],
                         "traffic": NCU_DRAM_BYTES_PER_ELEMENT_CONV["bwd"] * T * C}}
    print(json.dumps(line))


def run_glue_decode(args):
    """Secondary workloads: the convolution with the layer glue fused in (`--workload glue`, x (1, T, 13056), T = 32768
    unless --tokens says otherwise) and the one-token decode step (`--workload decode`, B=8, H=32, E=8); HBM rooflines."""
    dev = torch.device("cuda", 0)
    pk = peaks()
    if args.workload == "glue":
        T = args.tokens or 32768
        if T % 4096:
            raise SystemExit("--tokens must be a multiple of 4096 (documents of 4096 tokens)")
        gf, gb, fms, bms, _ = glue_rates(dev, T=T, reps=args.steps, unfused_too=False)
        line = {"metric": "conv_split_norm GB/s", "value": gf, "unit": "GB/s", "ms_per_step": fms,
                "config": {"workload": f"conv_split_norm (1,{T},13056) H=32 E=12, {T // 4096} documents"},
                "roofline": {"bound": "hbm", "kernel": "glue_main + glue_gate (forward)", "achieved": gf, "peak": pk["gbs"],
                             "unit": "GB/s", "frac": gf / pk["gbs"], "traffic": None, "peak_kind": pk["kind"]},
                "backward": {"ms": bms, "achieved": gb, "frac": gb / pk["gbs"]}}
    else:
        dg, dms = decode_rate(dev, reps=args.steps)
        line = {"metric": "decode GB/s", "value": dg, "unit": "GB/s", "ms_per_step": dms,
                "config": {"workload": "one token, B=32 H=32 E=8: 537 MB of f32 state read and written"},
                "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": dg, "peak": pk["gbs"], "unit": "GB/s",
                             "frac": dg / pk["gbs"], "traffic": None, "peak_kind": pk["kind"]}}
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": 3, "higher_is_better": True, "dtype": "bf16", "data": "synthetic"})
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=list(WORKLOADS) + ["conv", "glue", "decode"])
    ap.add_argument("--tokens", type=int, default=0,
                    help="conv workload only: sequence length (multiple of 4096; default 32768); small values size a profiler capture")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison of seeded slices with the CPU oracle")
    ap.add_argument("--no-aux", action="store_true", help="skip the GJ_SAVE_MASKS=0 and convolution side measurements")
    ap.add_argument("--no-reference-kernels", action="store_true", help="do not time the reference's own kernels (a child process)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end, per-kernel and CPU-baseline legs (used for profiler captures)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload == "conv":
        run_conv(args)
        return
    if args.workload in ("glue", "decode"):
        run_glue_decode(args)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
