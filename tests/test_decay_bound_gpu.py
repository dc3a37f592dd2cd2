"""GPU side of the exact decay bound: the one-pass key-norm kernel and the forgetting horizon computed on device
tensors agree with their plain torch / CPU forms, and what the horizon promises holds for the CUDA operator."""

import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.distributed import _key_norm_sq_max, forgetting_horizon, transfer_is_negligible
from gdn_qsa_sm80_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows", [1, 31, 32, 33, 1000, 262145])
def test_key_norm_kernel_matches_torch(rows):
    gen = torch.Generator().manual_seed(rows)
    k = (torch.randn(rows, 128, generator=gen) * torch.exp(torch.randn(rows, 1, generator=gen))).bfloat16()
    ref = float(k.float().pow(2).sum(-1).max())
    got = float(_key_norm_sq_max(k.cuda()))
    assert abs(got - ref) <= 1e-5 * ref
    # the largest row anywhere in the tensor is found (first, last, middle)
    for pos in (0, rows - 1, rows // 2):
        k2 = k.clone()
        k2[pos] = 1024.0
        assert float(_key_norm_sq_max(k2.cuda())) == 128 * 1024.0 ** 2


def test_horizon_on_device_equals_cpu_and_holds_for_the_operator():
    q, k, v, g, beta, _ = make_inputs("default", seed=3, B=2, S=1024, Hq=2, Hv=4)
    g = 1.5 * g
    p_cpu = forgetting_horizon(k.float(), g, beta)
    d = [t.cuda() for t in (q, k, v, g, beta)]
    p = forgetting_horizon(d[1], d[3], d[4])
    assert p == p_cpu and p is not None and 0 < p < 1024 and p % 64 == 0
    assert not transfer_is_negligible(d[1][:, :64], d[3][:, :64], d[4][:, :64])
    assert transfer_is_negligible(d[1], d[3], d[4])
    h0 = torch.randn(2, 4, 128, 128, device="cuda")
    o0, s0 = gdn_chunk(*d)
    o1, s1 = gdn_chunk(*d, initial_state=h0)
    assert torch.equal(o0[:, p:], o1[:, p:]) and torch.equal(s0, s1)
    assert not torch.equal(o0[:, :64], o1[:, :64])
    # premise violated: keys three times too long
    assert forgetting_horizon(3 * d[1], d[3], d[4]) is None
