"""Checks at the benchmark's full sizes through properties that need no CPU oracle run of that size.

Default workload (B1 S8192 Hq16 Hv32, the configuration the headline metric is quoted on):
  * two independent device implementations agree: the production path (tcgen05 kernels) against the
    token-by-token fp32 CUDA-core kernel, which follows the recurrent definition
    (gdn_qsa_sm80/reference/gdn_chunk_ref.py:133-141) and shares no code with it;
  * the operator is linear in v: doubling v doubles O and the final state bit for bit (a power-of-two scale
    commutes with every bf16/fp32 rounding on the way);
  * splitting the sequence in two and chaining the final state reproduces the unsplit run;
  * a slice of the result is compared with the CPU oracle run on that slice's prefix only (first 1024 tokens
    of 4 heads).
Short-batch workload (B16 S2048): production path against the fp32 kernel on a batch slice.
Long-context (B1 S131072) and throughput (B64 S4096) workloads at full size: production path against the fp32
recurrent kernel, two-level scan, split-and-chain, batch independence.
"""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def default_problem():
    q, k, v, g, beta, h0 = make_inputs("default", seed=0)
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta, h0)]
    out, st = gdn_chunk(*d[:5], initial_state=d[5])
    check_device_status()
    return (q, k, v, g, beta, h0), d, out, st


def test_default_workload_matches_independent_fp32_kernel(default_problem):
    _, d, out, st = default_problem
    o2, s2 = gdn_chunk(*d[:5], initial_state=d[5], path="simt")
    check_device_status()
    assert_close(out.float().cpu().numpy(), o2.float().cpu().numpy(), "O vs fp32 recurrent kernel")
    assert_close(st.cpu().numpy(), s2.cpu().numpy(), "final state vs fp32 recurrent kernel")


def test_default_workload_is_linear_in_v(default_problem):
    _, d, out, st = default_problem
    o2, s2 = gdn_chunk(d[0], d[1], d[2] * 2, d[3], d[4], initial_state=d[5] * 2)
    check_device_status()
    assert torch.equal(o2.float(), out.float() * 2)
    assert torch.equal(s2, st * 2)


def test_default_workload_split_and_chain(default_problem):
    _, d, out, st = default_problem
    h = d[0].shape[1] // 2
    oa, sa = gdn_chunk(*[t[:, :h] for t in d[:5]], initial_state=d[5])
    ob, sb = gdn_chunk(*[t[:, h:] for t in d[:5]], initial_state=sa)
    check_device_status()
    assert_close(torch.cat([oa, ob], 1).float().cpu().numpy(), out.float().cpu().numpy(), "chained O", rel=2e-3, mabs=2e-3)
    assert_close(sb.cpu().numpy(), st.cpu().numpy(), "chained state", rel=1e-4, mabs=1e-4)


def test_default_workload_prefix_against_cpu_oracle(default_problem):
    (q, k, v, g, beta, h0), _, out, _ = default_problem
    S, heads = 1024, slice(8, 12)          # value heads 8..11 use qk heads 4..5
    ro, _ = oracle_f32(q[:, :S, 4:6], k[:, :S, 4:6], v[:, :S, heads], g[:, :S, heads], beta[:, :S, heads], h0[:, heads])
    assert_close(out[:, :S, heads].float().cpu().numpy(), ro, "O prefix vs CPU oracle")


def test_short_batch_workload_slice_matches_fp32_kernel():
    q, k, v, g, beta, _ = make_inputs("short_batch", seed=0)
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    out, st = gdn_chunk(*d)
    check_device_status()
    sl = slice(5, 7)
    o2, s2 = gdn_chunk(*[t[sl] for t in d], path="simt")
    assert_close(out[sl].float().cpu().numpy(), o2.float().cpu().numpy(), "O vs fp32 recurrent kernel")
    assert_close(st[sl].cpu().numpy(), s2.cpu().numpy(), "state vs fp32 recurrent kernel")


def _device_inputs(workload, seed):
    """The workload's distributions generated on the GPU (the CPU generator would take minutes at these sizes; no
    oracle is run on these inputs, only properties between device results)."""
    from gdn_qsa_sm80_b200.synthetic import WORKLOADS
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


def _rel(x, ref):
    x, ref = x.float(), ref.float()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))


def test_long_context_workload_full_size():
    """B1 S131072: the production path (single launch, 2048 chunks per head) against the fp32 recurrent kernel over the
    whole sequence, the two-level scan against the serial path, and a split at an odd chunk boundary."""
    from gdn_qsa_sm80 import gdn_chunk_twolevel
    w, q, k, v, g, beta, _ = _device_inputs("long_context", 3)
    out, st = gdn_chunk(q, k, v, g, beta)
    check_device_status()
    o2, s2 = gdn_chunk(q, k, v, g, beta, path="simt")
    assert _rel(out, o2) <= 1e-2 and _rel(st, s2) <= 1e-2
    assert float((out.float() - o2.float()).abs().max()) <= 2e-2
    o3, s3, info = gdn_chunk_twolevel(q, k, v, g, beta, group_chunks=256)
    assert float(info[0]) == 8.0 and 1.0 < float(info[1]) < 1.3   # 16384-token groups forget their past early
    o4, s4, info4 = gdn_chunk_twolevel(q, k, v, g, beta, group_chunks=256, decay_early_out=False)
    assert float(info4[1]) == 3.0
    assert _rel(o4, o3) <= 1e-6 and _rel(s4, s3) <= 1e-6        # skipping them changes nothing
    assert _rel(o3, out) <= 3e-3 and _rel(s3, st) <= 3e-3
    cut = 64 * 777
    oa, sa = gdn_chunk(q[:, :cut], k[:, :cut], v[:, :cut], g[:, :cut], beta[:, :cut])
    ob, sb = gdn_chunk(q[:, cut:], k[:, cut:], v[:, cut:], g[:, cut:], beta[:, cut:], initial_state=sa)
    assert _rel(torch.cat([oa, ob], 1), out) <= 1e-3 and _rel(sb, st) <= 1e-3


def test_throughput_workload_full_size():
    """B64 S4096 (2048 independent sequences, prepare + transposed chain): against the fp32 recurrent kernel on the whole batch,
    and batch independence: a batch slice run alone gives the same bits as its part of the full run."""
    w, q, k, v, g, beta, h0 = _device_inputs("throughput", 4)
    out, st = gdn_chunk(q, k, v, g, beta, initial_state=h0)
    check_device_status()
    o2, s2 = gdn_chunk(q, k, v, g, beta, initial_state=h0, path="simt")
    assert _rel(out, o2) <= 1e-2 and _rel(st, s2) <= 1e-2
    assert float((out.float() - o2.float()).abs().max()) <= 2e-2
    del o2, s2
    sl = slice(40, 44)
    o3, s3 = gdn_chunk(q[sl], k[sl], v[sl], g[sl], beta[sl], initial_state=h0[sl], path="twopass_t")
    assert torch.equal(o3, out[sl]) and torch.equal(s3, st[sl])
