"""Long sequences split into segments by the transposed chain (path "twopass_t" when there are few sequences).

The split rests on a bound on the segment's transfer matrix that is checked per head on the device; heads whose gates
do not make every segment forget its incoming state run serially inside the same launch.  Every case is compared
with the CPU oracle at the benchmark's tolerance (rel-L2 <= 1e-2, max-abs <= 2e-2) and, tightly, with the unsplit
two-kernel path on the same device.
"""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs, make_reference_test_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


def _both(q, k, v, g, beta, h0=None):
    dev = "cuda"
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    h = None if h0 is None else h0.to(dev)
    o1, s1 = gdn_chunk(*d, initial_state=h, path="twopass_t")
    check_device_status()
    o2, s2 = gdn_chunk(*d, initial_state=h, path="twopass_nv64")
    check_device_status()
    return (o1.float().cpu().numpy(), s1.cpu().numpy()), (o2.float().cpu().numpy(), s2.cpu().numpy())


def _check(q, k, v, g, beta, h0=None, what=""):
    (o, s), (o2, s2) = _both(q, k, v, g, beta, h0)
    ro, rs = oracle_f32(q, k, v, g, beta, h0)
    assert_close(o, ro, f"{what} O vs oracle")
    assert_close(s, rs, f"{what} state vs oracle")
    # against the unsplit run of the other chain kernel: the two differ only by bf16 operand rounding
    assert_close(o, o2, f"{what} O vs unsplit path", rel=6e-3, mabs=6e-3)
    assert_close(s, s2, f"{what} state vs unsplit path", rel=6e-3, mabs=1e-2)


def test_default_workload_split_in_four():
    q, k, v, g, beta, h0 = make_inputs("default", seed=0)
    _check(q, k, v, g, beta, h0, "default")


@pytest.mark.parametrize("S,gs", [(8192, 2.0), (8192, 0.2)])
def test_reference_cases_split(S, gs):
    q, k, v, g, beta = make_reference_test_inputs(S, gs=gs)
    _check(q, k, v, g, beta, None, f"S={S} gs={gs}")


def test_weak_decay_runs_serially():
    """g = -U(0,1) * 0.02: no segment forgets its incoming state, so every head takes the serial branch."""
    q, k, v, g, beta = make_reference_test_inputs(4096, gs=0.02, Hk=2, Hv=4, seed=5)
    _check(q, k, v, g, beta, None, "weak decay")


def test_heads_with_and_without_forgetting_in_one_launch():
    q, k, v, g, beta, h0 = make_inputs("default", seed=3, S=4096, Hq=4, Hv=8)
    g = g.clone()
    g[:, :, ::2] *= 0.01          # every other head keeps its state for thousands of tokens
    _check(q, k, v, g, beta, h0, "mixed heads")


def test_ragged_length_and_uneven_segments():
    q, k, v, g, beta, h0 = make_inputs("default", seed=4, S=5000, Hq=2, Hv=4)
    _check(q, k, v, g, beta, h0, "S=5000")


def test_key_norms_outside_the_premise_run_serially():
    """A few keys with beta |k|^2 > 2 void the bound for their head: that head must not be split."""
    q, k, v, g, beta, _ = make_inputs("default", seed=6, S=4096, Hq=2, Hv=4)
    k = k.clone()
    k[:, 1000:1003, 0] *= 2.0     # |k|^2 = 4 for three tokens of qk head 0 (value heads 0 and 1)
    beta = beta.clone()
    beta[:, 1000:1003] = 0.9
    _check(q, k, v, g, beta, None, "large keys")
