"""A device-side wait that nothing satisfies must end by itself and be reported, and the GPU must stay usable.

Every wait inside the kernels (mbarrier phases, tile flags written by other CTAs) is bounded (2 s).  Here the
single-launch kernel runs with its prepare roles switched off and no tile flag raised (a test hook), so each chain
CTA's first wait runs out: the kernel sets the status word, drains and returns; the host sees GDN_ERR_DEVICE through
the status read; the next ordinary call works and gives the right result.  No fault, no trap, no endless loop.
"""

import os
import time

import pytest
import torch

from gdn_qsa_sm80 import gdn_chunk
from gdn_qsa_sm80_b200 import _lib
from gdn_qsa_sm80_b200.gdn_chunk_interface import check_device_status
from gdn_qsa_sm80_b200.synthetic import make_inputs

from helpers import assert_close, oracle_f32

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_next_call_succeeds():
    q, k, v, g, beta, _ = make_inputs("default", seed=12, S=256, Hq=2, Hv=4)
    dev = torch.device("cuda", 0)
    d = [t.to(dev) for t in (q, k, v, g, beta)]
    gdn_chunk(*d, path="coop")
    check_device_status(dev)
    os.environ["GDN_CHUNK_DBG"] = "7"
    try:
        t0 = time.time()
        gdn_chunk(*d, path="coop_chain_only")
        with pytest.raises(_lib.GdnLibraryError, match="0x307"):
            check_device_status(dev)
        waited = time.time() - t0
    finally:
        del os.environ["GDN_CHUNK_DBG"]
    assert 1.5 < waited < 20.0, waited          # the wait limit, once (all CTAs wait at the same time)
    out, st = gdn_chunk(*d, path="coop")
    check_device_status(dev)
    ro, rs = oracle_f32(q, k, v, g, beta)
    assert_close(out.float().cpu().numpy(), ro, "out after the timed-out launch")
    assert_close(st.cpu().numpy(), rs, "state after the timed-out launch")
