"""GPU tests of the gated RMS normalisation (the reference's rmsnorm_gated, csrc/output_gate/output_gate.cu:47-98)
alone and chained behind gdn_chunk (output_gate=...), against the oracle and the golden vector made with the
reference's own torch expression (tests/test_output_gate.py:12-16).  Tolerance of the reference's test: rel < 1e-2;
here tighter where only bf16 rounding of the result separates the two."""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk, rmsnorm_gated
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs
from oracle import gdn_chunk_oracle as O

from helpers import assert_close, golden, oracle_f32

pytestmark = pytest.mark.gpu


def test_golden_from_reference_expression():
    z = golden("rmsnorm_gated.npz")
    y, zz, w = (torch.from_numpy(z[n]).bfloat16().cuda() for n in ("y", "z", "weight"))
    out = rmsnorm_gated(y, zz, w).float().cpu().numpy()
    assert O.rel_l2(out, z["out_f32"]) < 3e-3
    # bf16 rounding of the result is the only difference allowed: one ulp around the fp32 value
    assert np.all(np.abs(out - z["out_f32"]) <= 2.0 ** -7 * np.abs(z["out_f32"]) + 1e-30)
    assert np.mean(out == z["out_bf16"]) > 0.98


@pytest.mark.parametrize("n_rows", [1, 2, 15, 16, 17, 63, 64, 65, 1000, 4097, 300001])
def test_row_counts_and_in_place(n_rows):
    gen = torch.Generator().manual_seed(n_rows)
    y = (0.1 * torch.randn(n_rows, 128, generator=gen)).bfloat16()
    z = (1.5 * torch.randn(n_rows, 128, generator=gen)).bfloat16()
    w = (1 + 0.1 * torch.randn(128, generator=gen)).bfloat16()
    ref = O.rmsnorm_gated(y.float().numpy(), z.float().numpy(), w.float().numpy())
    yd = y.cuda()
    guard = torch.full((n_rows + 2, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    out = rmsnorm_gated(yd, z.cuda(), w.cuda(), out=guard[1:-1])
    assert O.rel_l2(out.float().cpu().numpy(), ref) < 3e-3
    assert float(guard[0].min()) == 7.0 and float(guard[-1].max()) == 7.0   # nothing outside the rows is written
    same = rmsnorm_gated(yd, z.cuda(), w.cuda(), out=yd)                     # in place
    assert same.data_ptr() == yd.data_ptr() and torch.equal(same, out)


def test_leading_shape_eps_and_errors():
    y = torch.zeros(2, 3, 4, 128, dtype=torch.bfloat16, device="cuda")
    z = torch.ones_like(y)
    w = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    out = rmsnorm_gated(y, z, w, eps=1e-3)
    assert out.shape == y.shape and float(out.abs().max()) == 0.0           # zero rows stay finite zeros
    with pytest.raises(ValueError):
        rmsnorm_gated(y, z[..., :64], w)
    with pytest.raises(RuntimeError):
        rmsnorm_gated(y.cpu(), z.cpu(), w.cpu())


@pytest.mark.parametrize("path", ["auto", "twopass_nv64", "twopass_t", "simt"])
@pytest.mark.parametrize("S", [100, 1024])
def test_chained_behind_the_forward_pass(path, S):
    q, k, v, g, beta, _ = make_inputs("default", seed=S, B=2, S=S, Hq=2, Hv=4)
    gen = torch.Generator().manual_seed(S + 1)
    z = (1.5 * torch.randn(2, S, 4, 128, generator=gen)).bfloat16()
    w = (1 + 0.1 * torch.randn(128, generator=gen)).bfloat16()
    dev = "cuda"
    out, st = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), path=path, output_gate=(z, w))
    check_device_status()
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, None)
    ref = O.rmsnorm_gated(ref_o, z.float().numpy(), w.float().numpy())
    # normalised rows have unit rms before the gate, so max-abs is on the scale of silu(z): use the relative bound
    assert_close(out.float().cpu().numpy(), ref, f"{path} gated out", mabs=1e-1)
    assert_close(st.cpu().numpy(), ref_s, f"{path} state")
    # same bits as the two separate calls
    o2, _ = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), path=path)
    assert torch.equal(rmsnorm_gated(o2, z.to(dev), w.to(dev)), out)


def test_behind_the_transposed_chain_with_split_sequences():
    """Long sequences, few heads: the transposed chain splits them on the device (segments with unstored
    warm-up chunks); the gate behind it gives the same bits as the forward pass followed by the separate call."""
    S = 4096
    q, k, v, g, beta, h0 = make_inputs("default", seed=31, B=1, S=S, Hq=4, Hv=8)
    gen = torch.Generator().manual_seed(32)
    z = (1.5 * torch.randn(1, S, 8, 128, generator=gen)).bfloat16()
    w = (1 + 0.1 * torch.randn(128, generator=gen)).bfloat16()
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    out, st = gdn_chunk(*d, initial_state=h0.to(dev), output_gate=(z, w))
    check_device_status()
    o2, s2 = gdn_chunk(*d, initial_state=h0.to(dev))
    assert torch.equal(rmsnorm_gated(o2, z.to(dev), w.to(dev)), out) and torch.equal(st, s2)
    ref_o, _ = oracle_f32(q, k, v, g, beta, h0)
    ref = O.rmsnorm_gated(ref_o, z.float().numpy(), w.float().numpy())
    # outputs are on the scale of silu(z) (up to ~6 here) with bf16 rounding: the relative bound is the meaningful one
    assert_close(out.float().cpu().numpy(), ref, "gated out", mabs=2.5e-1)
