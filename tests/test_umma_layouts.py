"""Pins every shared-memory operand layout / UMMA descriptor combination the fused kernel uses
against a plain matmul, one tcgen05 product at a time (through the C ABI's probe entry).

Cases mirror the fused kernel's products:
  K-major x K-major                [K;Q] K^T
  K-major x MN-major (128 B rows)  [T';T''] K, [T';T''] V, [Q;W] S, P v_new     (64 value columns per CTA)
  K-major x MN-major (64 B rows)   the same with 32 value columns per CTA
  MN-major x MN-major              K^T v~
Each is checked with thread-staged tiles and with TMA-staged tiles.
"""

import pytest
import torch

from gdn_qsa_sm80_b200.diagnostics import umma_probe

pytestmark = pytest.mark.gpu

CASES = [
    # M,   N,  K,  a_major, b_major, b_span
    (128, 64, 128, 0, 0, 128),
    (128, 64, 64, 0, 0, 128),
    (128, 128, 64, 0, 1, 128),
    (128, 64, 64, 0, 1, 128),
    (128, 64, 128, 0, 1, 128),
    (128, 32, 64, 0, 1, 64),
    (128, 32, 128, 0, 1, 64),
    (128, 64, 64, 1, 1, 128),
    (128, 32, 64, 1, 1, 64),
]


def _mats(M, N, K, seed):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-4, 5, (M, K), generator=gen).to(torch.bfloat16)   # small integers: exact in bf16 and fp32
    b = torch.randint(-4, 5, (N, K), generator=gen).to(torch.bfloat16)
    return a, b


# A operand in tensor memory (written by tcgen05.st, one row per lane), as the transposed chain kernel uses it:
#   S^T W^T / S^T Q^T   (K-major B, 64 tokens, contraction over 128 dk)      v_new^T P^T  (K-major B, contraction over 64)
#   v~^T K              (MN-major B, 128 dk, contraction over 64 tokens)
TMEM_A_CASES = [
    (128, 64, 128, 2, 0, 128),
    (128, 64, 64, 2, 0, 128),
    (128, 128, 64, 2, 1, 128),
    (128, 64, 128, 3, 0, 128),     # negate-A bit
]


@pytest.mark.parametrize("M,N,K,a_major,b_major,b_span", TMEM_A_CASES)
def test_product_with_a_in_tensor_memory(M, N, K, a_major, b_major, b_span):
    a, b = _mats(M, N, K, seed=11 + N + K + a_major)
    d = umma_probe(a.cuda(), b.cuda(), a_major, b_major, b_span, False).cpu()
    ref = a.float() @ b.float().t()
    if a_major == 3:
        ref = -ref
    assert torch.equal(d[:M], ref), f"max |diff| = {(d[:M] - ref).abs().max().item()}"


def test_mn_major_a_with_k_major_b():
    """U^T I (later V^T T''^T): A = a [tokens][dv] tile read MN-major (M = 128 dv), B K-major."""
    a, b = _mats(128, 64, 64, seed=3)
    d = umma_probe(a.cuda(), b.cuda(), 1, 0, 128, False).cpu()
    assert torch.equal(d[:128], a.float() @ b.float().t())


@pytest.mark.parametrize("use_tma", [False, True])
@pytest.mark.parametrize("M,N,K,a_major,b_major,b_span", CASES)
def test_product_matches_matmul(M, N, K, a_major, b_major, b_span, use_tma):
    a, b = _mats(M, N, K, seed=M + N + K + 7 * a_major + 3 * b_major)
    d = umma_probe(a.cuda(), b.cuda(), a_major, b_major, b_span, use_tma).cpu()
    ref = a.float() @ b.float().t()
    assert torch.equal(d[:M], ref), f"max |diff| = {(d[:M] - ref).abs().max().item()}"


def test_m64_rows_live_on_the_first_16_lanes_of_each_warp():
    """An M = 64 accumulator puts row m on TMEM lane 32*(m // 16) + m % 16."""
    a, b = _mats(64, 64, 64, seed=5)
    d = umma_probe(a.cuda(), b.cuda(), 0, 0, 128, False).cpu()
    ref = a.float() @ b.float().t()
    lanes = torch.tensor([32 * (m // 16) + m % 16 for m in range(64)])
    assert torch.equal(d[lanes], ref)
