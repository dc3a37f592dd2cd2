"""Packed batches of sequences of different lengths (gdn_chunk_varlen) against the oracle run per sequence."""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk, gdn_chunk_varlen
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lens,n_streams", [([64], 1), ([1, 63, 65, 200, 7], 4), ([300, 300, 1024, 5], 2), ([17] * 9, 3), ([1] * 40 + [2, 2, 3], 4)])
def test_packed_batch_matches_oracle_per_sequence(lens, n_streams):
    T = sum(lens)
    q, k, v, g, beta, _ = make_inputs("default", seed=T, B=1, S=T, Hq=2, Hv=4)
    h0 = 0.1 * torch.randn(len(lens), 4, 128, 128, generator=torch.Generator().manual_seed(T + 1))
    cu = np.concatenate([[0], np.cumsum(lens)]).tolist()
    dev = "cuda"
    guard = torch.full((1, T + 2, 4, 128), 7.0, dtype=torch.bfloat16, device=dev)
    out, st = gdn_chunk_varlen(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), cu, initial_state=h0.to(dev),
                               n_streams=n_streams)
    torch.cuda.synchronize()
    assert out.shape == (1, T, 4, 128) and st.shape == (len(lens), 4, 128, 128)
    for i, (a, b) in enumerate(zip(cu, cu[1:])):
        ro, rs = oracle_f32(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b], h0[i:i + 1])
        assert_close(out[:, a:b].float().cpu().numpy(), ro, f"sequence {i} out")
        assert_close(st[i:i + 1].cpu().numpy(), rs, f"sequence {i} state")
        # and the same bits as the sequence run on its own
        o1, s1 = gdn_chunk(q[:, a:b].to(dev), k[:, a:b].to(dev), v[:, a:b].to(dev), g[:, a:b].to(dev),
                           beta[:, a:b].to(dev), initial_state=h0[i:i + 1].to(dev))
        assert torch.equal(o1, out[:, a:b]) and torch.equal(s1, st[i:i + 1])
    del guard


def test_shapes_without_batch_axis_options_and_errors():
    q, k, v, g, beta, _ = make_inputs("default", seed=3, B=1, S=160, Hq=2, Hv=4)
    dev = "cuda"
    d = [t[0].to(dev) for t in (q, k, v, g, beta)]
    out, st = gdn_chunk_varlen(*d, torch.tensor([0, 100, 160]), output_final_state=False, path="twopass_nv32")
    assert out.shape == (160, 4, 128) and st is None
    ref, _ = gdn_chunk(*[t[:, :100].to(dev) for t in (q, k, v, g, beta)], path="twopass_nv32")
    assert torch.equal(out[:100], ref[0])
    for bad in ([0, 160, 100], [1, 160], [0, 100], [0, 0, 160]):
        with pytest.raises(ValueError):
            gdn_chunk_varlen(*d, bad)
    with pytest.raises(ValueError):
        gdn_chunk_varlen(*d, [0, 100, 160], initial_state=torch.zeros(3, 4, 128, 128, device=dev))


def test_calls_on_two_streams_do_not_share_scratch():
    """Two forward passes in flight on different streams (each stream has its own scratch buffer)."""
    q, k, v, g, beta, _ = make_inputs("default", seed=8, B=1, S=2048, Hq=4, Hv=8)
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    d2 = [t.to(dev) for t in make_inputs("default", seed=9, B=1, S=2048, Hq=4, Hv=8)[:5]]
    ref1, _ = gdn_chunk(*d)
    ref2, _ = gdn_chunk(*d2)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(4):
        with torch.cuda.stream(s1):
            o1, _ = gdn_chunk(*d)
        with torch.cuda.stream(s2):
            o2, _ = gdn_chunk(*d2)
        outs.append((o1, o2))
    torch.cuda.synchronize()
    for o1, o2 in outs:
        assert torch.equal(o1, ref1) and torch.equal(o2, ref2)
    with torch.cuda.stream(s1):
        check_device_status()


@pytest.mark.parametrize("lens", [[150, 130, 164, 101, 177, 200, 133, 164, 164, 190, 108, 120], [3] * 5 + [100] * 4 + [7] * 6])
@pytest.mark.parametrize("opts", [{}, {"gate_activations": True, "use_qk_l2norm_in_kernel": True}])
def test_padded_strategy_equals_views_strategy(lens, opts):
    """Padding tokens carry g = 0 and beta = 0: the padded batch gives the per-sequence results (same parity bar
    against the oracle; the two strategies may pick different kernels, so they are compared with a tolerance)."""
    T = sum(lens)
    q, k, v, g, beta, _ = make_inputs("default", seed=T + 5, B=1, S=T, Hq=2, Hv=4)
    if opts:
        gen = torch.Generator().manual_seed(T)
        g, beta = 1.5 * torch.randn(1, T, 4, generator=gen), 1.5 * torch.randn(1, T, 4, generator=gen)
    h0 = 0.1 * torch.randn(len(lens), 4, 128, 128, generator=torch.Generator().manual_seed(T + 6))
    cu = np.concatenate([[0], np.cumsum(lens)]).tolist()
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    o1, s1 = gdn_chunk_varlen(*d, cu, initial_state=h0.to(dev), strategy="views", **opts)
    o2, s2 = gdn_chunk_varlen(*d, cu, initial_state=h0.to(dev), strategy="padded", **opts)
    o3, s3 = gdn_chunk_varlen(*d, cu, initial_state=h0.to(dev), **opts)
    torch.cuda.synchronize()
    # auto: many launches and little padding -> padded (first case); three runs of equal lengths -> views (second)
    same_o, same_s = (o2, s2) if len(set(lens)) > 8 else (o1, s1)
    assert torch.equal(o3, same_o) and torch.equal(s3, same_s)
    assert_close(o2.float().cpu().numpy(), o1.float().cpu().numpy(), "padded vs views out", rel=5e-3, mabs=1e-2)
    assert_close(s2.cpu().numpy(), s1.cpu().numpy(), "padded vs views state", rel=5e-3, mabs=1e-2)
    g_ref = -torch.nn.functional.softplus(g) if opts else g
    b_ref = torch.sigmoid(beta) if opts else beta
    for i, (a, b) in enumerate(zip(cu, cu[1:])):
        ro, rs = oracle_f32(q[:, a:b], k[:, a:b], v[:, a:b], g_ref[:, a:b], b_ref[:, a:b], h0[i:i + 1], l2norm=bool(opts))
        assert_close(o2[:, a:b].float().cpu().numpy(), ro, f"sequence {i} out (padded)")
        assert_close(s2[i:i + 1].cpu().numpy(), rs, f"sequence {i} state (padded)")
