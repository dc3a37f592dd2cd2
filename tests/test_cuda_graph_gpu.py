"""The forward pass captured in a CUDA graph and replayed.

The operator never reads a result on the host, allocates nothing below the Python wrapper and launches on the
caller's stream, so a call can be captured like any other kernel launch - including the chain's programmatic
dependent launch behind prepare, its clusters of two CTAs and the cooperative single-launch kernel.  A replay must
give the bits of the eager call, also after the inputs were rewritten in place.
"""

import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,Hq,Hv", [
    (4096, 4, 8),      # prepare + transposed chain, sequences split into segments on the device
    (4096, 16, 32),    # the same with enough sequences that nothing is split
    (1024, 16, 32),    # the cooperative single launch
])
def test_graph_replay_matches_eager(S, Hq, Hv):
    dev = torch.device("cuda", 0)
    q, k, v, g, beta, h0 = make_inputs("default", seed=7, B=1, S=S, Hq=Hq, Hv=Hv)
    d = [t.to(dev) for t in (q, k, v, g, beta, h0)]
    eager_out, eager_state = gdn_chunk(*d[:5], initial_state=d[5])
    check_device_status(dev)

    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):                 # warm-up on a side stream, as torch asks before a capture
        gdn_chunk(*d[:5], initial_state=d[5])
    torch.cuda.current_stream(dev).wait_stream(side)
    with torch.cuda.graph(graph):
        out, state = gdn_chunk(*d[:5], initial_state=d[5])
    graph.replay()
    torch.cuda.synchronize(dev)
    assert torch.equal(out, eager_out) and torch.equal(state, eager_state)

    # new values in the captured tensors: the replay computes on them
    gen = torch.Generator().manual_seed(8)
    d[2].copy_((torch.randn(d[2].shape, generator=gen) * 1.0).to(d[2].dtype))
    d[5].mul_(-0.5)
    eager_out, eager_state = gdn_chunk(*d[:5], initial_state=d[5])
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(dev)
    check_device_status(dev)
    assert torch.equal(out, eager_out) and torch.equal(state, eager_state)
