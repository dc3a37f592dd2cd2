"""Decode shapes: one or a few new tokens on top of a stored state.  The decode kernel is the exact fp32 recurrence,
so it is held to a tighter bound than the chunked paths (only the bf16 rounding of the output separates it from
the fp32 oracle), and the automatic path must pick it for S <= 8."""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs
from oracle import gdn_chunk_oracle as O

from helpers import oracle_f32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S,Hq,Hv", [(1, 1, 2, 4), (3, 1, 16, 32), (2, 2, 2, 4), (5, 4, 1, 4), (1, 17, 2, 2), (64, 1, 16, 32)])
@pytest.mark.parametrize("gates", ["fp32", "bf16"])
def test_decode_matches_recurrent_oracle(B, S, Hq, Hv, gates):
    q, k, v, g, beta, _ = make_inputs("default", seed=B * 100 + S, B=B, S=S, Hq=Hq, Hv=Hv)
    if gates == "bf16":
        g, beta = g.bfloat16(), beta.bfloat16()
    h0 = torch.randn(B, Hv, 128, 128, generator=torch.Generator().manual_seed(9))
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    out, st = gdn_chunk(*d, initial_state=h0.to(dev), path="decode")
    check_device_status()
    ro, rs = oracle_f32(q, k, v, g, beta, h0, form="recurrent")
    assert O.rel_l2(st.cpu().numpy(), rs) < 1e-5
    assert O.rel_l2(out.float().cpu().numpy(), ro) < 3e-3          # bf16 rounding of the output only
    assert np.all(np.abs(out.float().cpu().numpy() - ro) <= 2.0 ** -7 * np.abs(ro) + 1e-6)
    if S <= 8:   # the automatic choice for these shapes
        o2, s2 = gdn_chunk(*d, initial_state=h0.to(dev))
        assert torch.equal(o2, out) and torch.equal(s2, st)
    # token-by-token calls chained through the state give the same bits as one call
    s_run = h0.to(dev)
    pieces = []
    for t in range(S):
        o1, s_run = gdn_chunk(*[x[:, t:t + 1] for x in d], initial_state=s_run, path="decode")
        pieces.append(o1)
    assert torch.equal(torch.cat(pieces, 1), out) and torch.equal(s_run, st)


def test_decode_without_initial_or_final_state():
    q, k, v, g, beta, _ = make_inputs("default", seed=4, B=2, S=3, Hq=2, Hv=4)
    dev = "cuda"
    out, st = gdn_chunk(*[t.to(dev) for t in (q, k, v, g, beta)], output_final_state=False, path="decode")
    assert st is None
    ro, _ = oracle_f32(q, k, v, g, beta, None, form="recurrent")
    assert O.rel_l2(out.float().cpu().numpy(), ro) < 3e-3


def test_decode_updates_the_state_in_place_through_the_c_abi():
    """h0 and hT may be the same buffer for the decode kernel (a CTA reads its whole state before it writes it)."""
    from gdn_qsa_sm80_b200 import _lib
    B, S, Hq, Hv = 4, 1, 2, 4
    q, k, v, g, beta, _ = make_inputs("default", seed=21, B=B, S=S, Hq=Hq, Hv=Hv)
    dev = "cuda"
    d = [t.to(dev).contiguous() for t in (q, k, v, g.float(), beta.float())]
    h0 = torch.randn(B, Hv, 128, 128, device=dev)
    ref_o, ref_s = gdn_chunk(*d, initial_state=h0, path="decode")
    state = h0.clone()
    out = torch.empty_like(d[2])
    scratch = torch.empty(256, dtype=torch.uint8, device=dev)
    st = _lib.load().gdn_chunk_fwd_sm100(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                         d[4].data_ptr(), state.data_ptr(), out.data_ptr(), state.data_ptr(),
                                         scratch.data_ptr(), 256, B, S, Hq, Hv, _lib.GATE_F32, _lib.PATHS["decode"],
                                         torch.cuda.current_stream().cuda_stream)
    assert st == _lib.GDN_OK
    torch.cuda.synchronize()
    assert torch.equal(out, ref_o) and torch.equal(state, ref_s)
