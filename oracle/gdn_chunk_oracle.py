"""CPU oracle for the gdn_chunk forward pass (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing that ships imports this module: only the
tests, the smoke check and the CPU-baseline leg of the benchmark may use it.
It restates, in plain numpy, the two pure-torch functions of the reference
project that define the operator:

* ``chunk_gated_delta_rule``      follows
  ``gdn_qsa_sm80/reference/gdn_chunk_ref.py:20-100``
  (``torch_chunk_gated_delta_rule``): chunked WY form with the pairwise decay
  mask and two unit-lower-triangular solves per chunk.
* ``recurrent_gated_delta_rule``  follows
  ``gdn_qsa_sm80/reference/gdn_chunk_ref.py:103-147``
  (``torch_recurrent_gated_delta_rule``): one token at a time.

Parity is pinned: ``tests/golden/*.npz`` hold outputs of the real reference
(imported from its source tree by ``tests/golden/make_golden.py``) and
``tests/test_oracle.py`` checks both functions here against them.

Layouts are the reference's: q, k ``[B,S,Hk,D]``; v ``[B,S,Hv,D]``; g, beta
``[B,S,Hv]``; state ``[B,Hv,Dk,Dv]``.  Unlike the torch functions (which need
q/k already expanded to Hv heads, ``tests/test_gdn_chunk.py:28-30``), v-head
``h`` reads qk-head ``h // (Hv // Hk)`` here, which equals
``repeat_interleave(Hv // Hk, dim=2)`` (``csrc/gdn_chunk/gdn_kernel.cu:385-387``).
"""

from __future__ import annotations

import numpy as np

__all__ = [
    "chunk_gated_delta_rule",
    "recurrent_gated_delta_rule",
    "expand_qk_heads",
    "rel_l2",
    "max_abs",
    "l2norm",
    "rmsnorm_gated",
]


def expand_qk_heads(x: np.ndarray, hv: int) -> np.ndarray:
    """[B,S,Hk,D] -> [B,S,Hv,D]; v-head h takes qk-head h // (Hv // Hk)."""
    hk = x.shape[2]
    if hv % hk:
        raise ValueError(f"Hv={hv} is not a multiple of Hk={hk}")
    return np.repeat(x, hv // hk, axis=2)


def l2norm(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """x * rsqrt(sum x^2 + eps) over the last axis (gdn_chunk_ref.py:15-17)."""
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + x.dtype.type(eps))


def rmsnorm_gated(y, z, weight, eps=1e-6, dtype=np.float32):
    """RMSNorm(y) * weight * silu(z) over rows of the last axis, in `dtype`; restates the reference's
    torch_ref_rmsnorm_gated (tests/test_output_gate.py:12-16) and its CUDA kernel's arithmetic
    (csrc/output_gate/output_gate.cu:64-98)."""
    y, z, weight = (np.asarray(x, dtype=dtype) for x in (y, z, weight))
    normed = y / np.sqrt((y * y).mean(axis=-1, keepdims=True) + dtype(eps))
    return normed * weight * (z / (1 + np.exp(-z)))


def _solve_unit_lower(a: np.ndarray, rhs: np.ndarray) -> np.ndarray:
    """Solve (I + tril(a,-1)) x = rhs by forward substitution, batched.

    a: [..., C, C] (only the strict lower triangle is read), rhs: [..., C, N].
    Same result as torch.linalg.solve_triangular(upper=False, unitriangular=True)
    at gdn_chunk_ref.py:77-78.
    """
    c = a.shape[-1]
    x = rhs.copy()
    for i in range(1, c):
        x[..., i, :] -= np.einsum("...j,...jn->...n", a[..., i, :i], x[..., :i, :])
    return x


def chunk_gated_delta_rule(q, k, v, g, beta, chunk_size=64, initial_state=None,
                           output_final_state=True, dtype=np.float64, use_qk_l2norm_in_kernel=False):
    """Chunked gated delta rule; returns (out [B,S,Hv,Dv], final_state or None).

    Step numbers in the comments are line numbers of gdn_chunk_ref.py.
    """
    q, k, v, g, beta = (np.asarray(x, dtype=dtype) for x in (q, k, v, g, beta))
    b, s, hv, dv = v.shape
    dk = k.shape[-1]
    if use_qk_l2norm_in_kernel:   # :43-45
        q, k = l2norm(q), l2norm(k)
    q = expand_qk_heads(q, hv)
    k = expand_qk_heads(k, hv)
    # :39-42 head-major; :46-47 query scaling
    q, k, v = (x.transpose(0, 2, 1, 3) for x in (q, k, v))
    g, beta = (x.transpose(0, 2, 1) for x in (g, beta))
    q = q * dtype(dk) ** dtype(-0.5)
    # :49-51 zero padding to a whole number of chunks
    pad = (-s) % chunk_size
    if pad:
        q, k, v = (np.pad(x, ((0, 0), (0, 0), (0, pad), (0, 0))) for x in (q, k, v))
        g, beta = (np.pad(x, ((0, 0), (0, 0), (0, pad))) for x in (g, beta))
    nt = (s + pad) // chunk_size
    c = chunk_size
    q, k, v = (x.reshape(b, hv, nt, c, x.shape[-1]) for x in (q, k, v))
    g = g.reshape(b, hv, nt, c)
    beta = beta.reshape(b, hv, nt, c)
    # :56-57
    v_beta = v * beta[..., None]
    k_beta = k * beta[..., None]
    # :67-71 cumulative log decay and the pairwise mask exp(gamma_i - gamma_j), j <= i
    gamma = np.cumsum(g, axis=-1)
    diff = gamma[..., :, None] - gamma[..., None, :]
    lower = np.tril(np.ones((c, c), dtype=bool))
    pair = np.where(lower, np.exp(np.where(lower, diff, 0.0)), 0.0)
    # :73-75
    ut_system = (k_beta @ k.swapaxes(-1, -2)) * pair
    intra = (q @ k.swapaxes(-1, -2)) * pair
    decayed_k_beta = k_beta * np.exp(gamma)[..., None]
    # :77-78  U ("new_values") and W ("k_cumdecay")
    u = _solve_unit_lower(ut_system, v_beta)
    w = _solve_unit_lower(ut_system, decayed_k_beta)
    # :80-83
    if initial_state is None:
        state = np.zeros((b, hv, dk, dv), dtype=dtype)
    else:
        state = np.asarray(initial_state, dtype=dtype).copy()
    out = np.zeros((b, hv, nt, c, dv), dtype=dtype)
    # :86-88
    q_dec = q * np.exp(gamma)[..., None]
    k_dec = k * np.exp(gamma[..., -1:] - gamma)[..., None]
    chunk_decay = np.exp(gamma[..., -1])
    # :90-94 the serial loop over chunks
    for t in range(nt):
        v_new = u[:, :, t] - w[:, :, t] @ state
        out[:, :, t] = q_dec[:, :, t] @ state + intra[:, :, t] @ v_new
        state = state * chunk_decay[:, :, t, None, None] + k_dec[:, :, t].swapaxes(-1, -2) @ v_new
    out = out.reshape(b, hv, nt * c, dv)[:, :, :s].transpose(0, 2, 1, 3)
    return np.ascontiguousarray(out), (state if output_final_state else None)


def recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=None,
                               output_final_state=True, dtype=np.float64, use_qk_l2norm_in_kernel=False):
    """Token-by-token gated delta rule (gdn_chunk_ref.py:103-147)."""
    q, k, v, g, beta = (np.asarray(x, dtype=dtype) for x in (q, k, v, g, beta))
    b, s, hv, dv = v.shape
    dk = k.shape[-1]
    if use_qk_l2norm_in_kernel:   # :116-118
        q, k = l2norm(q), l2norm(k)
    q = expand_qk_heads(q, hv) / dtype(dk) ** dtype(0.5)   # :123
    k = expand_qk_heads(k, hv)
    if initial_state is None:
        state = np.zeros((b, hv, dk, dv), dtype=dtype)
    else:
        state = np.asarray(initial_state, dtype=dtype).copy()
    out = np.zeros((b, s, hv, dv), dtype=dtype)
    for i in range(s):                                     # :133-141
        state = state * np.exp(g[:, i])[..., None, None]
        kv_mem = np.einsum("bhkv,bhk->bhv", state, k[:, i])
        delta = (v[:, i] - kv_mem) * beta[:, i][..., None]
        state = state + k[:, i][..., :, None] * delta[..., None, :]
        out[:, i] = np.einsum("bhkv,bhk->bhv", state, q[:, i])
    return out, (state if output_final_state else None)


def rel_l2(x, ref) -> float:
    """||x - ref||_2 / ||ref||_2 over all elements."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = float(np.sqrt((ref * ref).sum()))
    return float(np.sqrt(((x - ref) ** 2).sum())) / (den if den > 0 else 1.0)


def max_abs(x, ref) -> float:
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(x - ref).max()) if x.size else 0.0
