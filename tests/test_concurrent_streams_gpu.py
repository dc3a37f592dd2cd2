"""Two forward passes in flight on two streams of one GPU, many times over.

Nothing in the automatic path waits, inside a launch, for a CTA of another launch, and the one kernel whose CTAs wait
for each other is launched cooperatively (all of its CTAs resident or none), so calls that overlap on the GPU can
neither stall one another nor change a result: every status stays GDN_OK and every result has the bits of the run
made alone.
"""

import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S", [4096, 1024])      # 4096: prepare + transposed chain; 1024: the cooperative single launch
def test_two_streams_fifty_rounds(S):
    dev = torch.device("cuda", 0)
    probs = []
    for seed in (1, 2):
        q, k, v, g, beta, h0 = make_inputs("default", seed=seed, S=S, Hq=16, Hv=32)
        d = [t.to(dev) for t in (q, k, v, g, beta, h0)]
        ref = gdn_chunk(*d[:5], initial_state=d[5])
        check_device_status(dev)
        probs.append((d, ref))
    streams = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    torch.cuda.synchronize(dev)
    for it in range(50):
        outs = []
        for (d, _), s in zip(probs, streams):
            with torch.cuda.stream(s):
                outs.append(gdn_chunk(*d[:5], initial_state=d[5]))
        for s in streams:
            s.synchronize()
        for s in streams:
            with torch.cuda.stream(s):
                check_device_status(dev)
        for (o, st), (_, (ro, rs)) in zip(outs, probs):
            assert torch.equal(o, ro) and torch.equal(st, rs), f"round {it}: result differs from the run made alone"
