"""The operator's mathematical definition in plain torch (fp32), exposed as
``gdn_chunk_reference`` because the reference project exposes one under that name
(``gdn_qsa_sm80/gdn_chunk_interface.py:65-72``).  It is NOT an execution path of
``gdn_chunk``: nothing in the CUDA path calls it and it is never used as a fallback.

Inputs follow the reference's torch functions: q, k, v ``[B,S,H,D]`` with q/k already expanded
to the value heads, g and beta ``[B,S,H]``; state ``[B,H,Dk,Dv]``.
"""

from __future__ import annotations

import torch


def _prep(q, k, v, g, beta):
    q, k, v = (x.float().permute(0, 2, 1, 3) for x in (q, k, v))       # [B,H,S,D]
    g, beta = (x.float().permute(0, 2, 1) for x in (g, beta))          # [B,H,S]
    return q * q.shape[-1] ** -0.5, k, v, g, beta


def recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=None, output_final_state=True):
    """S <- e^{g_t} S;  S <- S + k_t (beta_t (v_t - S^T k_t))^T;  o_t = S^T q_t."""
    dtype = q.dtype
    q, k, v, g, beta = _prep(q, k, v, g, beta)
    B, H, S, Dk = k.shape
    state = (torch.zeros(B, H, Dk, v.shape[-1], device=q.device) if initial_state is None
             else initial_state.float().clone())
    out = torch.empty_like(v)
    for t in range(S):
        state = state * g[:, :, t].exp()[..., None, None]
        delta = (v[:, :, t] - torch.einsum("bhkv,bhk->bhv", state, k[:, :, t])) * beta[:, :, t, None]
        state = state + k[:, :, t, :, None] * delta[:, :, None, :]
        out[:, :, t] = torch.einsum("bhkv,bhk->bhv", state, q[:, :, t])
    return out.permute(0, 2, 1, 3).contiguous().to(dtype), (state if output_final_state else None)


def chunk_gated_delta_rule(q, k, v, g, beta, chunk_size=64, initial_state=None, output_final_state=True):
    """Chunked WY form: per chunk T = (I + tril(beta K K^T * decay, -1))^-1, W = T (beta e^gamma K),
    U = T (beta V); v_new = U - W S; O = (q e^gamma) S + tril(Q K^T * decay) v_new;
    S <- e^{gamma_C} S + (K e^{gamma_C - gamma})^T v_new."""
    dtype = q.dtype
    q, k, v, g, beta = _prep(q, k, v, g, beta)
    B, H, S, Dk = k.shape
    C = chunk_size
    pad = (-S) % C
    if pad:
        q, k, v = (torch.nn.functional.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
        g, beta = (torch.nn.functional.pad(x, (0, pad)) for x in (g, beta))
    NT = (S + pad) // C
    q, k, v = (x.reshape(B, H, NT, C, -1) for x in (q, k, v))
    g, beta = (x.reshape(B, H, NT, C) for x in (g, beta))
    gamma = g.cumsum(-1)
    tri = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    decay = torch.where(tri, (gamma[..., :, None] - gamma[..., None, :]).masked_fill(~tri, 0.0).exp(), 0.0)
    A = (k * beta[..., None]) @ k.transpose(-1, -2) * decay
    eye = torch.eye(C, device=q.device)
    T = torch.linalg.solve_triangular(eye + A.tril(-1), eye.expand_as(A), upper=False)
    W = T @ (k * (beta * gamma.exp())[..., None])
    U = T @ (v * beta[..., None])
    P = (q @ k.transpose(-1, -2)) * decay
    state = (torch.zeros(B, H, Dk, v.shape[-1], device=q.device) if initial_state is None
             else initial_state.float().clone())
    out = torch.empty_like(v)
    for t in range(NT):
        v_new = U[:, :, t] - W[:, :, t] @ state
        out[:, :, t] = (q[:, :, t] * gamma[:, :, t].exp()[..., None]) @ state + P[:, :, t] @ v_new
        k_tail = k[:, :, t] * (gamma[:, :, t, -1:] - gamma[:, :, t]).exp()[..., None]
        state = state * gamma[:, :, t, -1].exp()[..., None, None] + k_tail.transpose(-1, -2) @ v_new
    out = out.reshape(B, H, NT * C, -1)[:, :, :S].permute(0, 2, 1, 3).contiguous().to(dtype)
    return out, (state if output_final_state else None)
