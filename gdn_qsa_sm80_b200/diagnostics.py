"""Diagnostics that go through the C ABI: the UMMA layout probe."""

from __future__ import annotations

import torch

from . import _lib


def umma_probe(a: torch.Tensor, b: torch.Tensor, a_major: int = 0, b_major: int = 0, b_span: int = 128,
               use_tma: bool = False) -> torch.Tensor:
    """D = A @ B^T through one tcgen05 product; returns the raw TMEM dump [128, N] (fp32).

    a: [M, K] bf16, b: [N, K] bf16 on a CUDA device.  a_major / b_major: 0 = K-major, 1 = MN-major.
    With ``use_tma`` an MN-major operand is handed to the library transposed ([K, M] / [K, N]),
    because that is the global layout such a tile is loaded from.
    """
    M, K = a.shape
    N = b.shape[0]
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.shape[1] == K
    lib = _lib.load()
    dev = a.device
    a_arg = a.t().contiguous() if (use_tma and a_major == 1) else a.contiguous()
    b_arg = b.t().contiguous() if (use_tma and b_major == 1) else b.contiguous()
    d = torch.empty((128, N), dtype=torch.float32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        st = lib.gdn_umma_probe(a_arg.data_ptr(), b_arg.data_ptr(), d.data_ptr(), status.data_ptr(), M, N, K,
                                a_major, b_major, b_span, int(use_tma),
                                torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "gdn_umma_probe")
    return d
