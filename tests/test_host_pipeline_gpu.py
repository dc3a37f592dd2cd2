"""GPU tests of gdn_chunk_host: inputs and results in host memory, copies pipelined against the kernels
(C ABI gdn_chunk_fwd_host_sm100).  Checked against the oracle and against gdn_chunk on device tensors."""

import numpy as np
import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk, gdn_chunk_host
from gdn_qsa_sm80_b200 import _lib
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


def inputs(S, B=1, Hq=2, Hv=4, seed=0, h0=True, pinned=True):
    q, k, v, g, beta, _ = make_inputs("default", seed=seed, B=B, S=S, Hq=Hq, Hv=Hv)
    h = 0.1 * torch.randn(B, Hv, 128, 128, generator=torch.Generator().manual_seed(seed + 100)) if h0 else None
    t = [q, k, v, g, beta, h]
    if pinned:
        t = [None if x is None else x.pin_memory() for x in t]
    return t


def device_result(q, k, v, g, beta, h):
    o, s = gdn_chunk(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), output_final_state=True,
                     initial_state=None if h is None else h.cuda())
    return o.float().cpu().numpy(), s.cpu().numpy()


@pytest.mark.parametrize("S,seg", [(2048, 0), (2048, 256), (700, 128), (64, 0), (100, 64), (1000, 448)])
def test_matches_oracle_and_device_path(S, seg):
    q, k, v, g, beta, h = inputs(S, B=2, seed=S)
    out, st = gdn_chunk_host(q, k, v, g, beta, initial_state=h, seg_tokens=seg)
    assert not out.is_cuda and out.is_pinned() and st.is_pinned()
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, h)
    assert_close(out.float().numpy(), ref_o, f"host S={S} seg={seg} out")
    assert_close(st.numpy(), ref_s, f"host S={S} seg={seg} state")
    dev_o, dev_s = device_result(q, k, v, g, beta, h)
    assert_close(out.float().numpy(), dev_o, "host vs device out", rel=2e-3, mabs=1e-2)
    assert_close(st.numpy(), dev_s, "host vs device state", rel=2e-3, mabs=1e-2)


def test_single_segment_is_bit_identical_to_the_device_path():
    q, k, v, g, beta, h = inputs(512, B=1, seed=4)
    out, st = gdn_chunk_host(q, k, v, g, beta, initial_state=h, seg_tokens=512)
    dev_o, dev_s = device_result(q, k, v, g, beta, h)
    assert np.array_equal(out.float().numpy(), dev_o)
    assert np.array_equal(st.numpy(), dev_s)


def test_pageable_memory_bf16_gates_no_initial_state_no_final_state():
    q, k, v, g, beta, _ = inputs(600, B=3, seed=8, h0=False, pinned=False)
    g, beta = g.bfloat16(), beta.bfloat16()
    out, st = gdn_chunk_host(q, k, v, g, beta, output_final_state=False, seg_tokens=192)
    assert st is None
    ref_o, _ = oracle_f32(q, k, v, g, beta, None)
    assert_close(out.float().numpy(), ref_o, "pageable out")


def test_repeated_and_interleaved_calls_give_the_same_bits():
    q, k, v, g, beta, h = inputs(1536, B=1, seed=2)
    a, sa = gdn_chunk_host(q, k, v, g, beta, initial_state=h, seg_tokens=256)
    a, sa = a.clone(), sa.clone()
    # two calls in flight at once on two streams with an arena each, results into caller-owned buffers
    outs = [torch.empty_like(a).pin_memory() for _ in range(4)]
    sts = [torch.empty_like(sa).pin_memory() for _ in range(4)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for i in range(4):
        with torch.cuda.stream(streams[i % 2]):
            gdn_chunk_host(q, k, v, g, beta, initial_state=h, seg_tokens=256, out=outs[i], final_state_out=sts[i],
                           synchronize=False, arena_slot=i % 2)
    torch.cuda.synchronize()
    for o, s in zip(outs, sts):
        assert torch.equal(o, a) and torch.equal(s, sa)


def test_l2norm_switch_and_empty_sequence():
    q, k, v, g, beta, h = inputs(640, B=1, seed=5)
    q, k = (q.float() * 7).bfloat16().pin_memory(), (k.float() * 0.3).bfloat16().pin_memory()
    out, st = gdn_chunk_host(q, k, v, g, beta, initial_state=h, seg_tokens=128, use_qk_l2norm_in_kernel=True)
    ref_o, ref_s = oracle_f32(q, k, v, g, beta, h, l2norm=True)
    assert_close(out.float().numpy(), ref_o, "host l2norm out")
    assert_close(st.numpy(), ref_s, "host l2norm state")
    e = [x[:, :0].contiguous() for x in (q, k, v, g, beta)]
    out, st = gdn_chunk_host(*e, initial_state=h)
    assert out.shape[1] == 0 and torch.equal(st, h)
    out, st = gdn_chunk_host(*e)
    assert float(st.abs().max()) == 0.0


def test_argument_errors():
    q, k, v, g, beta, h = inputs(128, pinned=False)
    with pytest.raises(ValueError):
        gdn_chunk_host(q.cuda(), k, v, g, beta)
    with pytest.raises(ValueError):
        gdn_chunk_host(q, k, v, g, beta, out=torch.empty(1, 128, 4, 64, dtype=torch.bfloat16))
    lib = _lib.load()
    assert lib.gdn_chunk_fwd_host_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), None,
                                        q.data_ptr(), None, None, 0, 1, 128, 2, 4, _lib.GATE_F32, 0, 0,
                                        None) == _lib.GDN_ERR_SCRATCH
    small = torch.empty(4096, dtype=torch.uint8, device="cuda")
    assert lib.gdn_chunk_fwd_host_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), None,
                                        q.data_ptr(), None, small.data_ptr(), small.numel(), 1, 128, 2, 4,
                                        _lib.GATE_F32, 0, 0, None) == _lib.GDN_ERR_SCRATCH
    assert lib.gdn_chunk_host_arena_bytes(1, 128, 2, 4, _lib.GATE_F32, 0) > 0
