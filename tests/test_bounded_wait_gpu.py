"""The give-up path of the kernels' bounded waits, exercised without provoking any fault.

Every wait of every kernel here polls an mbarrier with a limit; a wait that runs out raises the CTA's abort flag, records a
code in the device status word and lets the kernel run to its normal end.  The self-test kernel waits, with a SHORT limit,
for a barrier nothing arrives at: it must end by itself, report that the wait gave up, leave status 1 (a load barrier
timed out), and the context must stay usable (the reference's waits are unbounded: kernels/sm100_tc.py:116-119)."""
import ctypes

import pytest
import torch

from cute_triadic_gdn_b200 import _lib, gdn_joint_call
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_returns_and_reports():
    assert _lib.device_status() == 0
    out = torch.full((3,), -1, dtype=torch.int32, device="cuda")
    limit = 1 << 20                                            # about half a millisecond of SM clocks
    rc = _lib.lib.tgdn_selftest_wait(limit, ctypes.c_void_p(out.data_ptr()),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()                                   # the kernel ended on its own
    satisfied, abort, waited = out.tolist()
    assert satisfied == 0 and abort == 1
    assert limit < waited < 64 * limit                         # it did wait for the limit, and not much longer
    assert _lib.device_status() == 1                           # DEV_TIMEOUT_LOAD, and the read clears it
    assert _lib.device_status() == 0
    # the context is intact: a real kernel chain runs and reports nothing
    ins = [t.cuda() for t in orc.make_inputs(1, 128, 1, 2, seed=3)]
    with torch.no_grad():
        o = gdn_joint_call(*ins)
    assert torch.isfinite(o.float()).all() and _lib.device_status() == 0


def test_limits_outside_the_allowed_range_are_rejected():
    out = torch.zeros(3, dtype=torch.int32, device="cuda")
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _lib.lib.tgdn_selftest_wait(0, ctypes.c_void_p(out.data_ptr()), s) == -1
    assert _lib.lib.tgdn_selftest_wait(1 << 40, ctypes.c_void_p(out.data_ptr()), s) == -1
    assert _lib.lib.tgdn_selftest_wait(1 << 10, None, s) == -2
