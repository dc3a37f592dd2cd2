"""Seeded random shapes, paths and options against the fp32 oracle: every combination the entry point accepts should
meet the parity bar (rel-L2 <= 1e-2, max-abs <= 2e-2 on bf16 O and the fp32 final state)."""

import random

import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu

HEADS = [(1, 1), (1, 2), (2, 4), (1, 8), (3, 3), (4, 8), (2, 16)]


def _case(seed):
    rnd = random.Random(seed)
    B = rnd.randint(1, 5)
    S = rnd.choice([1, 2, 7, 8, 9, 31, 64, 65, 100, 127, 128, 129, 200, 333, 400])
    Hq, Hv = rnd.choice(HEADS)
    paths = ["auto", "twopass_nv64", "twopass_nv32", "twopass_t", "simt"]
    if 4 * B * Hv <= 148:
        paths.append("coop")
    if 8 * B * Hv <= 3 * 148:
        paths.append("twopass_t")
    if S <= 40:
        paths.append("decode")
    return dict(B=B, S=S, Hq=Hq, Hv=Hv, path=rnd.choice(paths), bf16_gates=rnd.random() < 0.4, h0=rnd.random() < 0.6,
                l2norm=rnd.random() < 0.4, gate_act=rnd.random() < 0.4, final=rnd.random() < 0.8,
                workload=rnd.choice(["default", "long_context"]))


@pytest.mark.parametrize("seed", range(40))
def test_random_configuration(seed):
    c = _case(seed)
    B, S, Hq, Hv = c["B"], c["S"], c["Hq"], c["Hv"]
    q, k, v, g, beta, _ = make_inputs(c["workload"], seed=1000 + seed, B=B, S=S, Hq=Hq, Hv=Hv)
    gen = torch.Generator().manual_seed(2000 + seed)
    if c["l2norm"]:      # un-normalised keys and queries
        q = (q.float() * torch.exp(torch.randn(B, S, Hq, 1, generator=gen))).bfloat16()
        k = (k.float() * torch.exp(torch.randn(B, S, Hq, 1, generator=gen))).bfloat16()
    g_in, b_in = g, beta
    if c["gate_act"]:    # raw projections in, the activations happen inside
        g_in = torch.randn(B, S, Hv, generator=gen) * 1.5
        b_in = torch.randn(B, S, Hv, generator=gen) * 1.5
    if c["bf16_gates"]:
        g_in, b_in = g_in.bfloat16(), b_in.bfloat16()
    g_ref = -torch.nn.functional.softplus(g_in.float()) if c["gate_act"] else g_in.float()
    b_ref = torch.sigmoid(b_in.float()) if c["gate_act"] else b_in.float()
    h0 = 0.1 * torch.randn(B, Hv, 128, 128, generator=gen) if c["h0"] else None
    dev = "cuda"
    out, st = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g_in.to(dev), b_in.to(dev), output_final_state=c["final"],
                        initial_state=None if h0 is None else h0.to(dev), path=c["path"],
                        use_qk_l2norm_in_kernel=c["l2norm"], gate_activations=c["gate_act"])
    check_device_status()
    ro, rs = oracle_f32(q, k, v, g_ref, b_ref, h0, l2norm=c["l2norm"])
    assert_close(out.float().cpu().numpy(), ro, f"{c} out")
    if c["final"]:
        assert_close(st.cpu().numpy(), rs, f"{c} state")
    else:
        assert st is None
