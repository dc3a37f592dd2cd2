"""Stage-level check of the prepare kernel: the per-chunk quantities it leaves in the workspace
(W, U, P and the per-token decay factors) against a float64 numpy restatement of
gdn_qsa_sm80/reference/gdn_chunk_ref.py:56-78 on the same inputs.  The reference exposes its
prepare stage for this kind of test (prepare_workspace, csrc/gdn_chunk/gdn_ops.cu:1026-1030) but
ships no such test."""

import ctypes

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200 import _lib
from gdn_qsa_sm80_b200 import gdn_chunk_interface as iface
from gdn_qsa_sm80_b200.synthetic import make_inputs
from oracle import gdn_chunk_oracle as O

pytestmark = pytest.mark.gpu


def numpy_prepare(q, k, v, g, beta):
    """W, U, P, factors per (b, h, chunk) in float64; inputs [B,S,H*,D] numpy."""
    B, S, Hv, D = v.shape
    q = O.expand_qk_heads(q, Hv).transpose(0, 2, 1, 3) * D ** -0.5
    k = O.expand_qk_heads(k, Hv).transpose(0, 2, 1, 3)
    v = v.transpose(0, 2, 1, 3)
    g = g.transpose(0, 2, 1)
    beta = beta.transpose(0, 2, 1)
    pad = (-S) % 64
    q, k, v = (np.pad(x, ((0, 0), (0, 0), (0, pad), (0, 0))) for x in (q, k, v))
    g, beta = (np.pad(x, ((0, 0), (0, 0), (0, pad))) for x in (g, beta))
    NT = (S + pad) // 64
    q, k, v = (x.reshape(B, Hv, NT, 64, D) for x in (q, k, v))
    g, beta = (x.reshape(B, Hv, NT, 64) for x in (g, beta))
    gam = np.cumsum(g, -1)
    low = np.tril(np.ones((64, 64), bool))
    dec = np.where(low, np.exp(np.where(low, gam[..., :, None] - gam[..., None, :], 0)), 0)
    A = np.tril((k * beta[..., None]) @ k.swapaxes(-1, -2) * dec, -1)
    T = np.linalg.inv(np.eye(64) + A)
    W = T @ (k * (beta * np.exp(gam))[..., None])
    U = T @ (v * beta[..., None])
    P = (q @ k.swapaxes(-1, -2)) * dec
    vec = np.zeros((B, Hv, NT, 256))
    vec[..., :64] = np.exp(gam[..., -1:] - gam)
    vec[..., 64:128] = np.exp(gam) * D ** -0.5
    vec[..., 128] = np.exp(gam[..., -1])
    return W, U, P, vec


@pytest.mark.parametrize("S,workload", [(256, "default"), (100, "default"), (192, "long_context")])
def test_prepare_outputs(S, workload):
    B, Hq, Hv = 2, 2, 4
    q, k, v, g, beta, _ = make_inputs(workload, seed=77 + S, B=B, S=S, Hq=Hq, Hv=Hv)
    dev = torch.device("cuda")
    gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), path="twopass_nv32")
    iface.check_device_status(dev)
    torch.cuda.synchronize()
    off = (ctypes.c_size_t * 5)()
    assert _lib.load().gdn_chunk_workspace_offsets(B, S, Hq, Hv, off) == 0
    raw = iface._scratch[(torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)]
    NT = (S + 63) // 64
    tiles = B * Hv * NT
    Wg = raw[off[0]:off[0] + tiles * 16384].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 128)
    Pg = raw[off[1]:off[1] + tiles * 8192].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 64)
    Ug = raw[off[2]:off[2] + tiles * 16384].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 128)
    vg = raw[off[3]:off[3] + tiles * 1024].view(torch.float32).cpu().numpy().reshape(B, Hv, NT, 256)
    W, U, P, vec = numpy_prepare(*[t.float().numpy().astype(np.float64) for t in (q, k, v, g, beta)])
    # bf16 operands (T rounded to bf16, 8 mantissa bits) bound the accuracy of W and U; P is one rounding
    assert O.rel_l2(Pg, P) < 4e-3, O.rel_l2(Pg, P)
    assert O.rel_l2(Wg, W) < 6e-3, O.rel_l2(Wg, W)
    assert O.rel_l2(Ug, U) < 6e-3, O.rel_l2(Ug, U)
    assert O.rel_l2(vg[..., :129], vec[..., :129]) < 1e-5
    assert np.abs(Pg - P).max() < 2e-2 and np.abs(Ug - U).max() < 5e-2


@pytest.mark.parametrize("S,workload,Hq,Hv", [(256, "default", 2, 4), (100, "default", 2, 4), (192, "long_context", 1, 4),
                                               (128, "default", 3, 3)])
def test_prepare_outputs_for_the_transposed_chain(S, workload, Hq, Hv):
    """The producer of path "twopass_t": W, P, T'' = T diag(beta) (at the start of the U array) and the factors.
    Two value heads per CTA when every qk head has an even number of them, else the one-head kernel without U."""
    B = 2
    q, k, v, g, beta, _ = make_inputs(workload, seed=11 + S, B=B, S=S, Hq=Hq, Hv=Hv)
    dev = torch.device("cuda")
    gdn_chunk(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), path="prepare_only_t")
    iface.check_device_status(dev)
    torch.cuda.synchronize()
    off = (ctypes.c_size_t * 5)()
    assert _lib.load().gdn_chunk_workspace_offsets(B, S, Hq, Hv, off) == 0
    raw = iface._scratch[(torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)]
    NT = (S + 63) // 64
    tiles = B * Hv * NT
    Wg = raw[off[0]:off[0] + tiles * 16384].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 128)
    Pg = raw[off[1]:off[1] + tiles * 8192].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 64)
    T2g = raw[off[2]:off[2] + tiles * 8192].view(torch.bfloat16).float().cpu().numpy().reshape(B, Hv, NT, 64, 64)
    vg = raw[off[3]:off[3] + tiles * 1024].view(torch.float32).cpu().numpy().reshape(B, Hv, NT, 256)
    x = [t.float().numpy().astype(np.float64) for t in (q, k, v, g, beta)]
    W, U, P, vec = numpy_prepare(*x)
    assert O.rel_l2(Pg, P) < 4e-3, O.rel_l2(Pg, P)
    assert O.rel_l2(Wg, W) < 6e-3, O.rel_l2(Wg, W)
    assert O.rel_l2(vg[..., :129], vec[..., :129]) < 1e-5
    # T'' V must reproduce U (V padded with zero rows like the kernel's tiles)
    vv = x[2].transpose(0, 2, 1, 3)
    vv = np.pad(vv, ((0, 0), (0, 0), (0, NT * 64 - S), (0, 0))).reshape(B, Hv, NT, 64, 128)
    assert O.rel_l2(T2g @ vv, U) < 6e-3, O.rel_l2(T2g @ vv, U)
