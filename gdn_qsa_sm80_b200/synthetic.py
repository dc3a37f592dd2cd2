"""Seeded synthetic inputs with the shapes and value distributions of the benchmark workloads.

No dataset is involved anywhere in this operator's evaluation: the reference's own tests and
benchmark draw random tensors (``tests/test_gdn_chunk.py:12-21``,
``benchmarks/bench_gdn_chunk.py:20-28``), and so do the workloads below.  Everything is
generated on the CPU generator (CPU and CUDA generators differ) in a fixed order, so the same
seed gives the same tensors on any machine with the same torch build.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

__all__ = ["Workload", "WORKLOADS", "make_inputs", "make_reference_test_inputs"]


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    S: int
    Hq: int
    Hv: int
    gate_scale: float      # g = -softplus(N(0,1)) * gate_scale
    h0: str                # "zeros" or "randn0.1" (N(0, 0.01): variance 0.01)
    dtype: str             # "fp32" (CPU reference case) or "bf16"

    @property
    def tokens(self) -> int:
        return self.B * self.S


# The five workloads the benchmark specification names (D = 128, chunk 64 everywhere).
WORKLOADS = {
    "cpu_small": Workload("cpu_small", 1, 512, 4, 8, 0.5, "zeros", "fp32"),
    "default": Workload("default", 1, 8192, 16, 32, 0.5, "randn0.1", "bf16"),
    "short_batch": Workload("short_batch", 16, 2048, 16, 32, 0.5, "zeros", "bf16"),
    "throughput": Workload("throughput", 64, 4096, 16, 32, 0.5, "randn0.1", "bf16"),
    "long_context": Workload("long_context", 1, 131072, 16, 32, 0.1, "zeros", "bf16"),
}


def make_inputs(w: Workload | str, seed: int = 0, B: int | None = None, S: int | None = None,
                Hq: int | None = None, Hv: int | None = None):
    """Return (q, k, v, g, beta, h0) on the CPU for a workload (optionally resized).

    q, k: L2-normalised N(0,1) vectors; v: N(0,1); g = -softplus(N(0,1)) * gate_scale;
    beta = sigmoid(N(0,1)).  q, k, v are bf16 for the bf16 workloads (fp32 otherwise); g and
    beta stay fp32 (the operator accepts either); h0 is fp32 ``[B,Hv,128,128]`` or None.
    """
    if isinstance(w, str):
        w = WORKLOADS[w]
    B = w.B if B is None else B
    S = w.S if S is None else S
    Hq = w.Hq if Hq is None else Hq
    Hv = w.Hv if Hv is None else Hv
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q = F.normalize(torch.randn(B, S, Hq, 128, generator=gen), dim=-1)
    k = F.normalize(torch.randn(B, S, Hq, 128, generator=gen), dim=-1)
    v = torch.randn(B, S, Hv, 128, generator=gen)
    g = -F.softplus(torch.randn(B, S, Hv, generator=gen)) * w.gate_scale
    beta = torch.sigmoid(torch.randn(B, S, Hv, generator=gen))
    if w.h0 == "zeros":
        h0 = None
    else:
        h0 = 0.1 * torch.randn(B, Hv, 128, 128, generator=gen)
    if w.dtype == "bf16":
        q, k, v = (x.to(torch.bfloat16) for x in (q, k, v))
    return q, k, v, g, beta, h0


def make_reference_test_inputs(S: int, gs: float = 2.0, Hk: int = 16, Hv: int = 32, seed: int = 0,
                               B: int = 1):
    """Inputs distributed like the reference's own test generator
    (``tests/test_gdn_chunk.py:12-21``): 0.05*N(0,1) q/k/v, g = -U(0,1)*gs, beta = sigmoid(U(0,1)),
    all bf16, drawn on the CPU generator."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(B, S, Hk, 128, generator=gen) * 0.05).to(torch.bfloat16)
    k = (torch.randn(B, S, Hk, 128, generator=gen) * 0.05).to(torch.bfloat16)
    v = (torch.randn(B, S, Hv, 128, generator=gen) * 0.05).to(torch.bfloat16)
    g = (-torch.rand(B, S, Hv, generator=gen) * gs).to(torch.bfloat16)
    beta = torch.rand(B, S, Hv, generator=gen).to(torch.bfloat16).sigmoid()
    return q, k, v, g, beta
