"""GPU parity of the in-kernel q/k L2 normalisation (use_qk_l2norm_in_kernel of the reference's torch
definition, gdn_qsa_sm80/reference/gdn_chunk_ref.py:29, :43-45) against the oracle and the golden vector
the reference produced with the switch on.  q and k are deliberately NOT normalised (0.5 * randn)."""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200 import _lib
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, golden, oracle_f32

pytestmark = pytest.mark.gpu

PATHS = ["simt", "twopass_nv64", "twopass_nv32", "twopass_t", "coop", "auto", "decode"]


def run(q, k, v, g, beta, h0=None, path="auto", l2=True):
    dev = "cuda"
    out, st = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), output_final_state=True,
                        initial_state=None if h0 is None else h0.to(dev), path=path, use_qk_l2norm_in_kernel=l2)
    check_device_status()
    return out.float().cpu().numpy(), st.cpu().numpy()


def raw_inputs(S, seed, B=1, Hq=2, Hv=4, amp=0.5):
    _, _, v, g, beta, _ = make_inputs("default", seed=seed, B=B, S=S, Hq=Hq, Hv=Hv)
    gen = torch.Generator().manual_seed(seed + 7)
    # per-token amplitudes spread over two decades so the norms really differ from row to row
    amp_q = amp * torch.exp(1.5 * torch.randn(B, S, Hq, 1, generator=gen))
    amp_k = amp * torch.exp(1.5 * torch.randn(B, S, Hq, 1, generator=gen))
    q = (amp_q * torch.randn(B, S, Hq, 128, generator=gen)).bfloat16()
    k = (amp_k * torch.randn(B, S, Hq, 128, generator=gen)).bfloat16()
    return q, k, v, g, beta


@pytest.mark.parametrize("path", PATHS)
def test_golden_from_reference_switch(path):
    z = golden("l2norm.npz")
    q, k, v = (torch.from_numpy(z[n]).bfloat16() for n in ("q", "k", "v"))
    g, beta = torch.from_numpy(z["g"]), torch.from_numpy(z["beta"])
    out, st = run(q, k, v, g, beta, path=path)
    assert_close(out, z["out_chunk"], f"{path} out vs reference (l2norm on)")
    assert_close(st, z["state_chunk"], f"{path} state vs reference (l2norm on)")


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("S", [64, 100, 1000])
def test_vs_oracle(path, S):
    q, k, v, g, beta = raw_inputs(S, seed=S)
    h0 = 0.1 * torch.randn(1, 4, 128, 128, generator=torch.Generator().manual_seed(5))
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, h0, l2norm=True)
    out, st = run(q, k, v, g, beta, h0, path=path)
    assert_close(out, ref_o, f"{path} S={S} out")
    assert_close(st, ref_s, f"{path} S={S} state")


def test_batched_problem_and_switch_off_is_unchanged():
    q, k, v, g, beta = raw_inputs(640, seed=3, B=3, Hq=4, Hv=8, amp=0.09)
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, None, l2norm=True)
    out, st = run(q, k, v, g, beta, path="auto")
    assert_close(out, ref_o, "batched out")
    assert_close(st, ref_s, "batched state")
    # flags = 0 through the new entry point is the old entry point: same bits
    a, sa = run(q, k, v, g, beta, path="twopass_nv64", l2=False)
    lib = _lib.load()
    dev = torch.device("cuda")
    qd, kd, vd, gd, bd = (x.to(dev).contiguous() for x in (q, k, v, g.float(), beta.float()))
    o2 = torch.empty_like(vd)
    s2 = torch.empty(3, 8, 128, 128, device=dev)
    n = lib.gdn_chunk_scratch_bytes(3, 640, 4, 8, _lib.PATHS["twopass_nv64"])
    scratch = torch.empty(n, dtype=torch.uint8, device=dev)
    code = lib.gdn_chunk_fwd_sm100(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), gd.data_ptr(), bd.data_ptr(), None,
                                   o2.data_ptr(), s2.data_ptr(), scratch.data_ptr(), n, 3, 640, 4, 8, _lib.GATE_F32,
                                   _lib.PATHS["twopass_nv64"], torch.cuda.current_stream().cuda_stream)
    assert code == _lib.GDN_OK
    torch.cuda.synchronize()
    assert np.array_equal(o2.float().cpu().numpy(), a)
    assert np.array_equal(s2.cpu().numpy(), sa)


def test_scale_invariance_of_q_and_k():
    # with the switch on, multiplying every q or k vector by a power of two changes nothing but rounding of eps
    q, k, v, g, beta = raw_inputs(256, seed=9)
    a, sa = run(q, k, v, g, beta, path="twopass_nv32")
    b, sb = run(q * 4, k * 8, v, g, beta, path="twopass_nv32")
    assert_close(b, a, "scaled out", rel=1e-3, mabs=5e-3)
    assert_close(sb, sa, "scaled state", rel=1e-3, mabs=5e-3)


def test_unknown_flag_bits_are_rejected():
    lib = _lib.load()
    x = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16, device="cuda")
    gt = torch.zeros(1, 64, 1, device="cuda")
    scratch = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    o = torch.empty_like(x)
    code = lib.gdn_chunk_fwd_sm100_ex(x.data_ptr(), x.data_ptr(), x.data_ptr(), gt.data_ptr(), gt.data_ptr(), None,
                                      o.data_ptr(), None, scratch.data_ptr(), scratch.numel(), 1, 64, 1, 1,
                                      _lib.GATE_F32, 0, 0x80, torch.cuda.current_stream().cuda_stream)
    assert code == _lib.GDN_ERR_BAD_ARGUMENT


@pytest.mark.parametrize("path", PATHS)
def test_gate_activations_inside_the_kernel(path):
    # raw gate projections in, g = -softplus(.), beta = sigmoid(.) applied by the kernels; ragged tail included
    q, k, v, _, _ = raw_inputs(300, seed=12)
    gen = torch.Generator().manual_seed(99)
    g_raw = 2.0 * torch.randn(1, 300, 4, generator=gen)
    b_raw = 2.0 * torch.randn(1, 300, 4, generator=gen)
    dev = "cuda"
    out, st = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g_raw.to(dev), b_raw.to(dev), path=path,
                        use_qk_l2norm_in_kernel=True, gate_activations=True)
    check_device_status()
    g = -torch.nn.functional.softplus(g_raw)
    beta = torch.sigmoid(b_raw)
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, None, l2norm=True)
    assert_close(out.float().cpu().numpy(), ref_o, f"{path} gate activations out")
    assert_close(st.cpu().numpy(), ref_s, f"{path} gate activations state")
