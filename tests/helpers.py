"""Shared helpers for the tests: golden files, tolerances, oracle wrappers (checker side only)."""

from __future__ import annotations

import hashlib
import os

import numpy as np
import torch

from oracle import c_oracle
from oracle import gdn_chunk_oracle as np_oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Parity bar of the benchmark specification for bf16 O and the fp32 final state.
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2


def golden(name):
    return np.load(os.path.join(GOLDEN, name), allow_pickle=False)


def checksum(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(t.detach().float().numpy()).tobytes())
    return h.hexdigest()


def oracle_f32(q, k, v, g, beta, h0=None, form="chunk", l2norm=False):
    """fp32 C oracle on torch CPU tensors (values upcast as they are); returns numpy arrays.
    l2norm: normalise q and k first, in fp32, as the reference's use_qk_l2norm_in_kernel does."""
    args = [x.detach().float().cpu().numpy() for x in (q, k, v, g, beta)]
    if l2norm:
        args[0], args[1] = np_oracle.l2norm(args[0]), np_oracle.l2norm(args[1])
    h = None if h0 is None else h0.detach().float().cpu().numpy()
    fn = c_oracle.chunk_f32 if form == "chunk" else c_oracle.recurrent_f32
    return fn(*args, initial_state=h)


def assert_close(x, ref, what, rel=REL_L2_TOL, mabs=MAX_ABS_TOL):
    r = np_oracle.rel_l2(x, ref)
    m = np_oracle.max_abs(x, ref)
    assert np.isfinite(np.asarray(x, dtype=np.float64)).all(), f"{what}: non-finite values"
    assert r <= rel, f"{what}: rel-L2 {r:.3e} > {rel:.1e} (max-abs {m:.3e})"
    assert m <= mabs, f"{what}: max-abs {m:.3e} > {mabs:.1e} (rel-L2 {r:.3e})"
    return r, m
