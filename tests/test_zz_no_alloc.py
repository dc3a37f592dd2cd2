"""The allocation-free entry point (gdn_chunk_fwd_sm100_noalloc) against the regular one.

Some callers of this library cannot allocate device memory when they call it (a runtime that handed
out all of its memory budget at start-up, a latency-critical loop that must never hit cudaMalloc),
so the library offers one entry point whose workspace is a fixed array inside its own device image.
This test drives it through the C ABI, twice in a row with different inputs, and requires the same
bits as the regular entry point given caller-owned scratch; it also checks that a problem beyond the
fixed capacity is refused.  It lives in its own file, collected last, so a failure here cannot hide
the results of the other GPU tests when pytest stops at the first failure.
"""

import pytest
import torch

from gdn_qsa_sm80_b200 import _lib
from gdn_qsa_sm80_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, tensors, B, S, Hq, Hv, scratch=None):
    q, k, v, g, beta, h0 = tensors
    dev = q.device
    out = torch.empty((B, S, Hv, 128), dtype=torch.bfloat16, device=dev)
    hT = torch.empty((B, Hv, 128, 128), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    if fn_name == "noalloc":
        st = lib.gdn_chunk_fwd_sm100_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                             h0.data_ptr(), out.data_ptr(), hT.data_ptr(), B, S, Hq, Hv,
                                             _lib.GATE_F32, stream)
    else:
        st = lib.gdn_chunk_fwd_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                     h0.data_ptr(), out.data_ptr(), hT.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                     B, S, Hq, Hv, _lib.GATE_F32, _lib.PATH_AUTO, stream)
    torch.cuda.synchronize(dev)
    return st, out, hT


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, Hq, Hv = 1, 2, 4
    for call, S in enumerate((512, 300)):        # second call: other inputs, ragged tail, stale workspace contents
        q, k, v, g, beta, _ = make_inputs("default", seed=900 + call, B=B, S=S, Hq=Hq, Hv=Hv)
        h0 = 0.1 * torch.randn(B, Hv, 128, 128, generator=torch.Generator().manual_seed(call))
        tensors = [t.to(dev).contiguous() for t in (q, k, v, g, beta, h0)]
        nbytes = int(lib.gdn_chunk_scratch_bytes(B, S, Hq, Hv, _lib.PATH_AUTO))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        st_ref, out_ref, hT_ref = _call(lib, "regular", tensors, B, S, Hq, Hv, scratch)
        st_new, out_new, hT_new = _call(lib, "noalloc", tensors, B, S, Hq, Hv)
        assert st_ref == _lib.GDN_OK and st_new == _lib.GDN_OK
        # same kernels, same inputs, different scratch location: the results must be bit-identical
        # (the tolerance of the other GPU tests, rel-L2 <= 1e-2, is trivially met)
        assert torch.equal(out_new, out_ref), f"call {call}: outputs differ"
        assert torch.equal(hT_new, hT_ref), f"call {call}: final states differ"
        assert torch.isfinite(out_new.float()).all()


def test_noalloc_entry_rejects_problems_beyond_its_fixed_workspace():
    lib = _lib.load()
    # 32 value heads x 8192 tokens = 4096 tiles > 399: refused on the host, no pointer is touched
    st = lib.gdn_chunk_fwd_sm100_noalloc(None, None, None, None, None, None, None, None, 1, 8192, 16, 32,
                                         _lib.GATE_F32, None)
    assert st == _lib.GDN_ERR_SCRATCH
