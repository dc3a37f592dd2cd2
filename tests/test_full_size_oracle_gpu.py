"""The benchmark configurations at FULL size against the CPU oracle (the C restatement of the reference's torch
function, fp32), with the benchmark's tolerance: rel-L2 <= 1e-2 and max-abs <= 2e-2 on the bf16 output and on the
fp32 final state, the oracle fed the same bf16-rounded values.

  * default (B1 S8192 Hq16 Hv32, random initial state): the whole output and the whole final state;
  * short_batch (B16 S2048): whole;
  * throughput (B64 S4096): the whole batch runs on the device, four batch elements are compared;
  * long_context (B1 S131072, weak decay): the whole sequence runs on the device, four value heads (two qk heads)
    are compared over all 131072 tokens;
  * the reference's own four (S, gate scale) cases at B1 Hk16 Hv32 with its input generator and its metric
    (tests/test_gdn_chunk.py:24-36: max-abs error over max |reference| < 2e-2), including (32768, 2.0) and the
    weak-decay (8192, 0.2).
Sequences are independent across (batch, value head), so comparing a slice of heads of a full-size run is a
comparison of those sequences at full length.
"""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import WORKLOADS, make_inputs, make_reference_test_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


def _run(q, k, v, g, beta, h0=None):
    dev = "cuda"
    out, st = gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev),
                        initial_state=None if h0 is None else h0.to(dev))
    check_device_status()
    return out, st


def test_default_workload_whole_against_cpu_oracle():
    q, k, v, g, beta, h0 = make_inputs("default", seed=0)
    out, st = _run(q, k, v, g, beta, h0)
    ro, rs = oracle_f32(q, k, v, g, beta, h0)
    r = assert_close(out.float().cpu().numpy(), ro, "default O vs CPU oracle")
    s = assert_close(st.cpu().numpy(), rs, "default final state vs CPU oracle")
    print(f"default: O rel-L2 {r[0]:.2e} max-abs {r[1]:.2e}; state rel-L2 {s[0]:.2e} max-abs {s[1]:.2e}")


def test_short_batch_workload_whole_against_cpu_oracle():
    q, k, v, g, beta, _ = make_inputs("short_batch", seed=0)
    out, st = _run(q, k, v, g, beta)
    ro, rs = oracle_f32(q, k, v, g, beta)
    r = assert_close(out.float().cpu().numpy(), ro, "short_batch O vs CPU oracle")
    s = assert_close(st.cpu().numpy(), rs, "short_batch final state vs CPU oracle")
    print(f"short_batch: O rel-L2 {r[0]:.2e} max-abs {r[1]:.2e}; state rel-L2 {s[0]:.2e} max-abs {s[1]:.2e}")


def _device_inputs(workload, seed):
    """The workload's distributions drawn on the GPU generator (the CPU generator would take minutes at these sizes);
    the oracle is given the very same values, copied back for the slice it checks."""
    w = WORKLOADS[workload]
    gen = torch.Generator(device="cuda").manual_seed(seed)
    F = torch.nn.functional
    rn = lambda *s: torch.randn(*s, generator=gen, device="cuda")
    q = F.normalize(rn(w.B, w.S, w.Hq, 128), dim=-1).bfloat16()
    k = F.normalize(rn(w.B, w.S, w.Hq, 128), dim=-1).bfloat16()
    v = rn(w.B, w.S, w.Hv, 128).bfloat16()
    g = -F.softplus(rn(w.B, w.S, w.Hv)) * w.gate_scale
    beta = torch.sigmoid(rn(w.B, w.S, w.Hv))
    h0 = 0.1 * rn(w.B, w.Hv, 128, 128) if w.h0 != "zeros" else None
    return w, q, k, v, g, beta, h0


def test_throughput_workload_four_batch_elements_against_cpu_oracle():
    w, q, k, v, g, beta, h0 = _device_inputs("throughput", 4)
    out, st = gdn_chunk(q, k, v, g, beta, initial_state=h0)
    check_device_status()
    for b in (0, 21, 42, 63):
        sl = slice(b, b + 1)
        ro, rs = oracle_f32(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), g[sl].cpu(), beta[sl].cpu(), h0[sl].cpu())
        assert_close(out[sl].float().cpu().numpy(), ro, f"throughput O[b={b}] vs CPU oracle")
        assert_close(st[sl].cpu().numpy(), rs, f"throughput state[b={b}] vs CPU oracle")


def test_long_context_workload_four_heads_whole_sequence_against_cpu_oracle():
    w, q, k, v, g, beta, _ = _device_inputs("long_context", 3)
    out, st = gdn_chunk(q, k, v, g, beta)
    check_device_status()
    hq, hv = slice(6, 8), slice(12, 16)          # value heads 12..15 read qk heads 6..7
    ro, rs = oracle_f32(q[:, :, hq].cpu(), k[:, :, hq].cpu(), v[:, :, hv].cpu(), g[:, :, hv].cpu(), beta[:, :, hv].cpu())
    r = assert_close(out[:, :, hv].float().cpu().numpy(), ro, "long_context O vs CPU oracle")
    s = assert_close(st[:, hv].cpu().numpy(), rs, "long_context final state vs CPU oracle")
    print(f"long_context: O rel-L2 {r[0]:.2e} max-abs {r[1]:.2e}; state rel-L2 {s[0]:.2e} max-abs {s[1]:.2e}")


@pytest.mark.parametrize("S,gs", [(2048, 2.0), (8192, 2.0), (32768, 2.0), (8192, 0.2)])
def test_reference_cases_against_cpu_oracle(S, gs):
    """The reference's test_vs_chunk_reference cases (tests/test_gdn_chunk.py:24-36), its generator, its metric."""
    q, k, v, g, beta = make_reference_test_inputs(S, gs=gs)
    out, st = _run(q, k, v, g, beta)
    ro, rs = oracle_f32(q, k, v, g, beta)
    o, s = out.float().cpu().numpy(), st.cpu().numpy()
    orr = np.abs(o - ro).max() / (np.abs(ro).max() + 1e-9)
    srr = np.abs(s - rs).max() / (np.abs(rs).max() + 1e-9)
    assert orr < 2e-2, f"S={S} gs={gs} out rel={orr:.2e}"
    assert srr < 2e-2, f"S={S} gs={gs} state rel={srr:.2e}"
    assert_close(o, ro, f"S={S} gs={gs} O")
    assert_close(s, rs, f"S={S} gs={gs} state")
