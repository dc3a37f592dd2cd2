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


def test_noalloc_entry_allocates_no_device_memory_after_its_first_call():
    """What the entry point promises: once the first call on a device has looked up the array's address, a call
    changes neither the driver's free-memory figure nor torch's allocator."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, S, Hq, Hv = 1, 256, 2, 4
    q, k, v, g, beta, _ = make_inputs("default", seed=77, B=B, S=S, Hq=Hq, Hv=Hv)
    h0 = torch.zeros(B, Hv, 128, 128)
    tensors = [t.to(dev).contiguous() for t in (q, k, v, g, beta, h0)]
    out = torch.empty((B, S, Hv, 128), dtype=torch.bfloat16, device=dev)
    hT = torch.empty((B, Hv, 128, 128), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call():
        return lib.gdn_chunk_fwd_sm100_noalloc(*[t.data_ptr() for t in tensors], out.data_ptr(), hT.data_ptr(), B, S,
                                               Hq, Hv, _lib.GATE_F32, stream)

    assert call() == _lib.GDN_OK              # set-up call
    torch.cuda.synchronize(dev)
    free0, _ = torch.cuda.mem_get_info(dev)
    alloc0, reserved0 = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for _ in range(3):
        assert call() == _lib.GDN_OK
    torch.cuda.synchronize(dev)
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0
    assert torch.cuda.memory_allocated(dev) == alloc0 and torch.cuda.memory_reserved(dev) == reserved0


def test_noalloc_entry_capacity_boundary_and_single_token_route():
    """399 tiles fit the fixed array, 400 do not; a one-token call (the decode kernel) works as well."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def run(B, S, Hq, Hv):
        q, k, v, g, beta, _ = make_inputs("default", seed=5, B=B, S=S, Hq=Hq, Hv=Hv)
        h0 = 0.1 * torch.randn(B, Hv, 128, 128, generator=torch.Generator().manual_seed(3))
        tensors = [t.to(dev).contiguous() for t in (q, k, v, g, beta, h0)]
        nbytes = int(lib.gdn_chunk_scratch_bytes(B, S, Hq, Hv, _lib.PATH_AUTO))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        st_ref, out_ref, hT_ref = _call(lib, "regular", tensors, B, S, Hq, Hv, scratch)
        st_new, out_new, hT_new = _call(lib, "noalloc", tensors, B, S, Hq, Hv)
        return st_ref, st_new, out_ref, out_new, hT_ref, hT_new

    # 3 value heads x 133 chunks = 399 tiles: accepted, and equal to the regular entry within the tests' tolerance
    # (the regular entry may split these long sequences into segments, the fixed array has no room for that)
    st_ref, st_new, out_ref, out_new, hT_ref, hT_new = run(1, 133 * 64, 1, 3)
    assert st_ref == _lib.GDN_OK and st_new == _lib.GDN_OK
    rel = lambda x, r: float((x.float() - r.float()).norm() / r.float().norm())
    assert rel(out_new, out_ref) <= 1e-2 and rel(hT_new, hT_ref) <= 1e-2
    # 4 value heads x 100 chunks = 400 tiles: refused, nothing is launched
    st = lib.gdn_chunk_fwd_sm100_noalloc(None, None, None, None, None, None, None, None, 1, 6400, 2, 4, _lib.GATE_F32, stream)
    assert st == _lib.GDN_ERR_SCRATCH
    # one new token on top of a stored state: the decode route, bit-identical to the regular entry
    st_ref, st_new, out_ref, out_new, hT_ref, hT_new = run(2, 1, 2, 4)
    assert st_ref == _lib.GDN_OK and st_new == _lib.GDN_OK
    assert torch.equal(out_new, out_ref) and torch.equal(hT_new, hT_ref)
