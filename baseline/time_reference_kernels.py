"""Times the reference's own CuTe-DSL sm100 kernels (chunk_gdn_joint, kernel path) on one B200.

Runs the unmodified reference package installed under baseline/_ref (git-ignored; installed with
`pip install --no-deps --target baseline/_ref <reference checkout>`).  Prints ONE JSON line:
  {"reference_kernels": {"ok": true, "forward_ok": true, "check": {...}, "c1_fwd_ms": ..., "c2_ms": ..., "dsl": "..."}}   or
  {"reference_kernels": {"ok": false, "forward_ok": ..., "stage": "...", "error": "..."}}  (what ran before the failure is kept)
First the reference's own smallest test case (B=2, T=256, H=4, E=8; tests/test_joint.py of the reference) is run through
the kernels and compared with its torch path; only if that passes are the BASELINE workloads timed (first call = JIT,
excluded).  Meant to be run as a child process with a timeout by bench.py, so that a compile failure of the DSL cannot
take the bench down.
"""
import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))
sys.path.insert(0, os.path.dirname(HERE))


def main():
    out = {"ok": False}
    stage = "import"
    try:
        import torch
        import cutlass
        out["dsl"] = getattr(cutlass, "__version__", "unknown")
        import cute_triadic_gdn as ref
        from bench import host_inputs
        dev = torch.device("cuda", 0)

        def run(B, T, H, E, backward, reference=False, seed=0):
            ins, do = host_inputs(B, T, H, E, seed)
            leaves = [t.to(dev).requires_grad_(backward) for t in ins]
            o = ref.chunk_gdn_joint(*leaves, reference=reference)
            if backward:
                o.backward(do.to(dev))
            torch.cuda.synchronize()
            return o.detach().float(), [t.grad.float() for t in leaves] if backward else []

        rel = lambda a, b: float((a - b).norm() / b.norm())

        def timed(B, T, H, E, mode, steps=3):
            """mode: 'infer' (no grad), 'train_fwd' (forward that saves for backward), 'fwd_bwd'."""
            ins, do = host_inputs(B, T, H, E, 1)
            leaves = [t.to(dev).requires_grad_(mode != "infer") for t in ins]
            do_d = do.to(dev)

            def step():
                for t in leaves:
                    t.grad = None
                o = ref.chunk_gdn_joint(*leaves)
                if mode == "fwd_bwd":
                    o.backward(do_d)
            step()                       # JIT + warm-up
            step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / steps

        # forward kernels (scan, masks, forward recurrence) first: they are a bar of their own
        stage = "forward: compile+check (2,256,4,8)"
        t0 = time.time()
        o_k, _ = run(2, 256, 4, 8, False)
        out["forward_first_call_s"] = round(time.time() - t0, 1)
        o_r, g_r = run(2, 256, 4, 8, True, reference=True)
        out["forward_check"] = {"o": rel(o_k, o_r)}
        if not out["forward_check"]["o"] < 2e-2:
            raise RuntimeError(f"reference forward kernels fail the reference's own tolerance: {out['forward_check']}")
        stage = "forward: time c1"
        out["c1_fwd_ms"] = timed(4, 4096, 16, 4, "infer")
        stage = "forward: time c2 (inference and training forward)"
        out["c2_fwd_infer_ms"] = timed(8, 8192, 32, 8, "infer")
        out["c2_fwd_train_ms"] = timed(8, 8192, 32, 8, "train_fwd")
        out["forward_ok"] = True

        stage = "backward: compile+check (2,256,4,8)"
        t0 = time.time()
        o_k, g_k = run(2, 256, 4, 8, True)
        out["first_call_s"] = round(time.time() - t0, 1)
        out["check"] = {"o": rel(o_k, o_r), "max_grad": max(rel(a, b) for a, b in zip(g_k, g_r))}
        if not (out["check"]["o"] < 2e-2 and out["check"]["max_grad"] < 5e-2):
            raise RuntimeError(f"reference kernels fail the reference's own tolerance: {out['check']}")
        stage = "time c2 fwd+bwd"
        out["c2_ms"] = timed(8, 8192, 32, 8, "fwd_bwd")
        out["c2_tokens_per_s"] = 8 * 8192 / (out["c2_ms"] * 1e-3)
        out["ok"] = True
    except BaseException as exc:           # the DSL raises its own exception types
        out["stage"] = stage
        out["error"] = f"{type(exc).__name__}: {str(exc)[:600]}"
        out["trace_tail"] = traceback.format_exc()[-1500:]
    print(json.dumps({"reference_kernels": out}))


if __name__ == "__main__":
    main()
