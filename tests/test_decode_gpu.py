"""One-token decode on a resident state against the token-by-token definition (cute_triadic_gdn/ops/gdn_joint.py:1-8).

A prefix goes through the chunk kernels, which hand out the f32 state; the following tokens go through the decode step
one at a time.  The outputs must match the f64 sequential oracle over the whole sequence (o within 1e-2 relative L2, the
tolerance of the chunk path), and the state after the last token the definition's state."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib, chunk_gdn_joint, gdn_joint_decode
from oracle import triadic_oracle as orc
from test_state_gpu import final_state_by_definition

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E", [1, 2, 4, 8, 12, 16])
def test_decode_continues_a_prefix(E):
    B, T0, n, H = 2, 128, 24, 3
    ins = orc.make_inputs(B, T0 + n, H, E, seed=900 + E, dist="mild")
    dev = [t.cuda() for t in ins]
    with torch.no_grad():
        o0, state = chunk_gdn_joint(*[t[:, :T0].contiguous() for t in dev], output_final_state=True)
        outs = [o0]
        for t in range(T0, T0 + n):
            outs.append(gdn_joint_decode(*[x[:, t:t + 1] for x in dev], state))
    assert _lib.device_status() == 0
    o = torch.cat(outs, 1)
    ref = orc.sequential_reference(*ins, dtype=torch.float64)
    assert orc.rel_l2(o.float().cpu(), ref.float()) < 1e-2
    assert orc.rel_l2(o[:, T0:].float().cpu(), ref[:, T0:].float()) < 1e-2
    assert orc.rel_l2(state.double().cpu(), final_state_by_definition(*ins)) < 1e-2


def test_decode_from_zero_state_is_exact_to_rounding_and_checks_arguments():
    """From a zero state the decode path is f32 throughout: it follows the f64 definition to bf16 output rounding."""
    B, n, H, E = 3, 40, 2, 8
    ins = orc.make_inputs(B, n, H, E, seed=77, dist="baseline")
    dev = [t.cuda() for t in ins]
    state = torch.zeros(B, H, E, 128, 128, device="cuda")
    with torch.no_grad():
        o = torch.cat([gdn_joint_decode(*[x[:, t] for x in dev], state)[:, None] for t in range(n)], 1)
    ref = orc.sequential_reference(*ins, dtype=torch.float64)
    assert orc.rel_l2(o.float().cpu(), ref.float()) < 4e-3
    assert orc.rel_l2(state.double().cpu(), final_state_by_definition(*ins)) < 1e-5
    with pytest.raises(ValueError):
        gdn_joint_decode(*[x[:, :2] for x in dev], state)                      # two tokens
    with pytest.raises(ValueError):
        gdn_joint_decode(*[x[:, :1] for x in dev], state[:, :, :4])            # wrong state shape
    with pytest.raises(ValueError):
        gdn_joint_decode(*[x[:, :1].requires_grad_(x.is_floating_point()) for x in dev], state)
