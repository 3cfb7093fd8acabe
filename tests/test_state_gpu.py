"""State in / state out of the forward recurrence (inference that continues a sequence).

The recurrent state is handed over in f32, so a sequence cut in two and continued from the first half's final state must
give bitwise the outputs and the final state of the uninterrupted run; the final state itself is checked against the
token-by-token definition (cute_triadic_gdn/ops/gdn_joint.py:1-8): S_e <- exp(g_te) S_e, then
S <- S + beta_t kappa_t (v_t - S^T kappa_t)^T with kappa_t = k2_t (x) k_t."""
import pytest
import torch

from cute_triadic_gdn_b200 import _lib, chunk_gdn_joint
from oracle import triadic_oracle as orc

pytestmark = pytest.mark.gpu


def final_state_by_definition(q, k, v, k2, q2, g, beta):
    B, T, H, D = k.shape
    E = k2.shape[-1]
    kd, vd, k2d, gd, bd = (t.double() for t in (k, v, k2, g, beta))
    S = torch.zeros(B, H, E, D, D, dtype=torch.float64)
    for t in range(T):
        S = S * gd[:, t].exp()[..., None, None]
        kappa = k2d[:, t][..., None] * kd[:, t][:, :, None, :]                       # (B,H,E,D)
        pred = torch.einsum('bhedv,bhed->bhv', S, kappa)
        S = S + bd[:, t][..., None, None, None] * kappa[..., None] * (vd[:, t] - pred)[:, :, None, None, :]
    return S


@pytest.mark.parametrize("E", [1, 4, 8, 16])
def test_final_state_and_continuation(E):
    B, T, H = 2, 256, 2
    ins = orc.make_inputs(B, T, H, E, seed=700 + E, dist="mild")
    dev = [t.cuda() for t in ins]
    with torch.no_grad():
        o_full, s_full = chunk_gdn_joint(*dev, output_final_state=True)
        half = T // 2
        first = [t[:, :half].contiguous() for t in dev]
        second = [t[:, half:].contiguous() for t in dev]
        o1, s1 = chunk_gdn_joint(*first, output_final_state=True)
        o2, s2 = chunk_gdn_joint(*second, initial_state=s1, output_final_state=True)
    assert _lib.device_status() == 0
    assert torch.equal(torch.cat([o1, o2], 1), o_full)
    assert torch.equal(s2, s_full)
    ref = final_state_by_definition(*ins)
    assert orc.rel_l2(s_full.double().cpu(), ref) < 1e-2
    # and the plain call is unchanged by the extra outputs
    with torch.no_grad():
        assert torch.equal(chunk_gdn_joint(*dev), o_full)


def test_state_of_packed_documents_and_argument_checks():
    T, H, E = 300, 2, 4
    ins = orc.make_inputs(1, T, H, E, seed=71, dist="mild")
    cu = torch.tensor([0, 70, 133, 300], dtype=torch.int32)
    dev = [t.cuda() for t in ins]
    with torch.no_grad():
        o, s = chunk_gdn_joint(*dev, cu_seqlens=cu.cuda(), output_final_state=True)
    assert s.shape == (3, H, E, 128, 128)
    for d, (lo, hi) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        ref = final_state_by_definition(*[t[:, lo:hi] for t in ins])
        assert orc.rel_l2(s[d:d + 1].double().cpu(), ref) < 1e-2
    with pytest.raises(ValueError):
        chunk_gdn_joint(*[t.requires_grad_(t.is_floating_point()) for t in dev], cu_seqlens=cu.cuda(), output_final_state=True)
    with pytest.raises(ValueError):
        with torch.no_grad():                                  # three documents need a state of three sequences
            chunk_gdn_joint(*[t.detach() for t in dev], cu_seqlens=cu.cuda(),
                            initial_state=torch.zeros(2, H, E, 128, 128, device="cuda"))
    assert _lib.device_status() == 0
