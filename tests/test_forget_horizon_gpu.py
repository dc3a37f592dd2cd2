"""The library's forgetting-horizon kernels against the same question answered with torch reductions.

`forgetting_horizon` (sequence-parallel driver) asks after how many leading tokens every (batch, head) of a stretch
has forgotten the state it started from, and whether the premise of the bound holds.  On CUDA tensors two small
kernels answer; the torch formulation stays the definition (and the path for CPU ranks).
"""

import pytest
import torch

from gdn_qsa_sm80_b200 import distributed as D

pytestmark = pytest.mark.gpu


def _torch_answer(k, g, beta, keys_are_normalized=False):
    # the non-kernel branch of forgetting_horizon_launch, forced by moving the tensors to the CPU
    return D.forgetting_horizon(k.cpu(), g.cpu(), beta.cpu(), keys_are_normalized=keys_are_normalized)


def _inputs(B, S, Hq, Hv, seed, g_scale, dtype=torch.float32):
    gen = torch.Generator().manual_seed(seed)
    k = torch.nn.functional.normalize(torch.randn(B, S, Hq, 128, generator=gen), dim=-1).bfloat16()
    g = (-torch.nn.functional.softplus(torch.randn(B, S, Hv, generator=gen)) * g_scale).to(dtype)
    beta = torch.sigmoid(torch.randn(B, S, Hv, generator=gen)).to(dtype)
    return k, g, beta


@pytest.mark.parametrize("B,S,Hq,Hv,g_scale,dtype", [
    (1, 8192, 16, 32, 0.5, torch.float32),       # forgets after a few chunks
    (2, 5000, 4, 8, 0.5, torch.float32),         # ragged length, two batch elements
    (1, 4096, 2, 48, 0.5, torch.bfloat16),       # more heads than lanes, bf16 gates
    (1, 2048, 4, 8, 0.001, torch.float32),       # never forgets inside the stretch -> None
    (3, 100, 1, 2, 5.0, torch.float32),          # shorter than the horizon's first chunks
])
def test_kernel_matches_torch(B, S, Hq, Hv, g_scale, dtype):
    k, g, beta = _inputs(B, S, Hq, Hv, seed=S + Hv, g_scale=g_scale, dtype=dtype)
    want = _torch_answer(k, g, beta)
    got = D.forgetting_horizon(k.cuda(), g.cuda(), beta.cuda())
    assert got == want
    assert D.forgetting_horizon(k.cuda(), g.cuda(), beta.cuda(), keys_are_normalized=True) == \
        _torch_answer(k, g, beta, keys_are_normalized=True)


def test_premise_failures_give_none():
    k, g, beta = _inputs(1, 4096, 4, 8, seed=1, g_scale=0.5)
    assert D.forgetting_horizon(k.cuda(), g.cuda(), beta.cuda()) is not None
    g_pos = g.clone(); g_pos[0, 3000, 5] = 0.25                     # a growing gate
    assert D.forgetting_horizon(k.cuda(), g_pos.cuda(), beta.cuda()) is None
    b_neg = beta.clone(); b_neg[0, 17, 0] = -0.1                    # a negative update gate
    assert D.forgetting_horizon(k.cuda(), g.cuda(), b_neg.cuda()) is None
    b_nan = beta.clone(); b_nan[0, 4000, 7] = float("nan")
    assert D.forgetting_horizon(k.cuda(), g.cuda(), b_nan.cuda()) is None
    k_big = (k.float() * 2.0).bfloat16()                            # beta |k|^2 up to 4
    assert D.forgetting_horizon(k_big.cuda(), g.cuda(), beta.cuda()) is None
    assert D.forgetting_horizon(k_big.cuda(), g.cuda(), beta.cuda(), keys_are_normalized=True) is not None


def test_one_slow_head_sets_the_horizon():
    k, g, beta = _inputs(1, 8192, 4, 8, seed=2, g_scale=0.5)
    g[:, :, 3] *= 0.1                                               # this head decays ten times more slowly
    want = _torch_answer(k, g, beta)
    assert want is not None and want > 1000
    assert D.forgetting_horizon(k.cuda(), g.cuda(), beta.cuda()) == want
