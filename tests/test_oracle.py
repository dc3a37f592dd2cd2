"""The CPU oracles against golden vectors produced by the real reference implementation.

The fixtures under tests/golden/ were written by tests/golden/make_golden.py from
gdn_qsa_sm80/reference/gdn_chunk_ref.py (torch, fp32).  Both restatements (numpy and C),
in both forms (chunked :20-100 and recurrent :103-147), must reproduce them.
"""

import numpy as np
import pytest

from gdn_qsa_sm80_b200.synthetic import make_inputs
from oracle import c_oracle
from oracle import gdn_chunk_oracle as O

from helpers import checksum, golden

# fp32 torch vs fp32 C / fp64 numpy on the same inputs: rounding-order differences only.
TOL = 2e-5


def _case(name):
    z = golden(name)
    h0 = z["h0"] if "h0" in z.files else None
    return z, (z["q"], z["k"], z["v"], z["g"], z["beta"]), h0


@pytest.mark.parametrize("name", ["tail_h0.npz", "ref_style.npz"])
def test_numpy_chunk_matches_reference(name):
    z, x, h0 = _case(name)
    out, st = O.chunk_gated_delta_rule(*x, initial_state=h0)
    assert O.rel_l2(out, z["out_chunk"]) < TOL
    assert O.rel_l2(st, z["state_chunk"]) < TOL


@pytest.mark.parametrize("name", ["tail_h0.npz", "ref_style.npz"])
def test_numpy_recurrent_matches_reference(name):
    z, x, h0 = _case(name)
    out, st = O.recurrent_gated_delta_rule(*x, initial_state=h0)
    assert O.rel_l2(out, z["out_recurrent"]) < TOL
    assert O.rel_l2(st, z["state_recurrent"]) < TOL


@pytest.mark.parametrize("name", ["tail_h0.npz", "ref_style.npz"])
@pytest.mark.parametrize("form", ["chunk", "recurrent"])
def test_c_oracle_matches_reference(name, form):
    z, x, h0 = _case(name)
    fn = c_oracle.chunk_f32 if form == "chunk" else c_oracle.recurrent_f32
    out, st = fn(*x, initial_state=h0)
    assert O.rel_l2(out, z[f"out_{form}"]) < TOL
    assert O.rel_l2(st, z[f"state_{form}"]) < TOL


@pytest.mark.parametrize("form", ["chunk", "recurrent"])
def test_l2norm_switch_matches_reference(form):
    # golden made by the reference with use_qk_l2norm_in_kernel=True on un-normalised q/k
    z, x, _ = _case("l2norm.npz")
    fn = O.chunk_gated_delta_rule if form == "chunk" else O.recurrent_gated_delta_rule
    out, st = fn(*x, use_qk_l2norm_in_kernel=True)
    assert O.rel_l2(out, z[f"out_{form}"]) < TOL
    assert O.rel_l2(st, z[f"state_{form}"]) < TOL
    # the fp32 C oracle on inputs normalised beforehand in fp32 (how the GPU tests use it)
    q, k = (O.l2norm(a.astype(np.float32)) for a in x[:2])
    cfn = c_oracle.chunk_f32 if form == "chunk" else c_oracle.recurrent_f32
    out, st = cfn(q, k, *x[2:])
    assert O.rel_l2(out, z[f"out_{form}"]) < TOL
    assert O.rel_l2(st, z[f"state_{form}"]) < TOL
    # and the switch matters on these inputs
    out_off, _ = fn(*x)
    assert O.rel_l2(out_off, z[f"out_{form}"]) > 0.1


def test_rmsnorm_gated_matches_reference_function():
    z = golden("rmsnorm_gated.npz")
    out = O.rmsnorm_gated(z["y"], z["z"], z["weight"])
    assert O.rel_l2(out, z["out_f32"]) < 1e-6
    # the reference rounds its result to bf16: one bf16 ulp at most between the two
    assert np.all(np.abs(out - z["out_bf16"]) <= 2.0 ** -8 * np.abs(z["out_f32"]) + 1e-30)


def test_cpu_small_workload_matches_reference():
    """The CPU benchmark workload (B1 S512 Hq4 Hv8 fp32 seed 0) regenerated from its seed."""
    z = golden("cpu_small.npz")
    q, k, v, g, beta, h0 = make_inputs("cpu_small", seed=0)
    assert h0 is None
    assert checksum(q, k, v, g, beta) == str(z["input_sha256"]), "seeded inputs changed"
    x = [t.numpy() for t in (q, k, v, g, beta)]
    out, st = c_oracle.chunk_f32(*x)
    assert O.rel_l2(out[:, ::8], z["out_chunk_every8"]) < TOL
    assert O.rel_l2(st, z["state_chunk"]) < TOL
    out_r, st_r = c_oracle.recurrent_f32(*x)
    assert O.rel_l2(out_r[:, ::8], z["out_recurrent_every8"]) < TOL
    assert O.rel_l2(st_r[:, :1], z["state_recurrent_head0"]) < TOL
    out_n, st_n = O.chunk_gated_delta_rule(*x)
    assert O.rel_l2(out_n[:, ::8], z["out_chunk_every8"]) < TOL
    assert O.rel_l2(st_n, z["state_chunk"]) < TOL


def test_chunk_and_recurrent_forms_agree():
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=3, S=130, Hq=2, Hv=4)
    x = [t.numpy() for t in (q, k, v, g, beta)]
    oc, sc = O.chunk_gated_delta_rule(*x)
    orr, sr = O.recurrent_gated_delta_rule(*x)
    assert O.rel_l2(oc, orr) < 1e-10 and O.rel_l2(sc, sr) < 1e-10


def test_chunk_size_independence():
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=4, S=96, Hq=1, Hv=2)
    x = [t.numpy() for t in (q, k, v, g, beta)]
    o64, s64 = O.chunk_gated_delta_rule(*x, chunk_size=64)
    o16, s16 = O.chunk_gated_delta_rule(*x, chunk_size=16)
    assert O.rel_l2(o64, o16) < 1e-10 and O.rel_l2(s64, s16) < 1e-10


def test_sequence_split_and_state_chaining_is_exact():
    """Running two halves with the first half's final state as the second's initial state
    reproduces the unsplit run (the property the sequence-partitioned multi-GPU path uses)."""
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=5, S=256, Hq=1, Hv=2)
    x = [t.numpy() for t in (q, k, v, g, beta)]
    o, s = O.chunk_gated_delta_rule(*x)
    a = [t[:, :128] for t in x]
    b = [t[:, 128:] for t in x]
    oa, sa = O.chunk_gated_delta_rule(*a)
    ob, sb = O.chunk_gated_delta_rule(*b, initial_state=sa)
    assert O.max_abs(np.concatenate([oa, ob], axis=1), o) < 1e-12
    assert O.max_abs(sb, s) < 1e-12


def test_gqa_mapping_equals_repeat_interleave():
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=6, S=64, Hq=2, Hv=4)
    x = [t.numpy() for t in (q, k, v, g, beta)]
    o1, s1 = O.chunk_gated_delta_rule(*x)
    qe = np.repeat(x[0], 2, axis=2)
    ke = np.repeat(x[1], 2, axis=2)
    o2, s2 = O.chunk_gated_delta_rule(qe, ke, *x[2:])
    assert O.max_abs(o1, o2) == 0.0 and O.max_abs(s1, s2) == 0.0
    with pytest.raises(ValueError):
        O.expand_qk_heads(np.zeros((1, 4, 3, 128)), 4)


def test_empty_sequence():
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=7, S=0, Hq=1, Hv=2)
    h0 = np.random.default_rng(0).standard_normal((1, 2, 128, 128)).astype(np.float32)
    out, st = c_oracle.chunk_f32(*[t.numpy() for t in (q, k, v, g, beta)], initial_state=h0)
    assert out.shape == (1, 0, 2, 128)
    assert np.array_equal(st, h0)
