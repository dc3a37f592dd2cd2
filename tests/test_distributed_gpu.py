"""Two-GPU checks (skipped with fewer than two devices): batch x head sharding with no communication and the
sequence-partitioned chain over NCCL send/recv, both against the single-GPU result."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gdn_qsa_sm80_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem(S, g_scale):
    q, k, v, g, beta, _ = make_inputs("long_context", seed=5, B=2, S=S, Hq=2, Hv=4)
    h0 = 0.1 * torch.randn(2, 4, 128, 128, generator=torch.Generator().manual_seed(6))
    return q, k, v, g * g_scale, beta, h0


def _worker(rank, world, port, mode, S, q_out, g_scale=1.0):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from gdn_qsa_sm80 import gdn_chunk
        from gdn_qsa_sm80_b200.distributed import plan_shards, segment_bounds, sequence_parallel_forward, shard_inputs
        q, k, v, g, beta, h0 = _problem(S, g_scale)
        if mode == "shard":
            sh = plan_shards(2, 2, 4, world)[rank]
            part = [None if t is None else t.to(dev) for t in shard_inputs(q, k, v, g, beta, h0, sh)]
            out, st = gdn_chunk(*part[:5], initial_state=part[5])
            q_out.put((rank, (sh.b0, sh.b1, sh.hv0, sh.hv1), out.float().cpu().numpy(), st.cpu().numpy()))
        else:
            lo, hi = segment_bounds(S, world)[rank]
            seg = [t[:, lo:hi].to(dev) for t in (q, k, v, g, beta)]
            out, st = sequence_parallel_forward(*seg, initial_state=h0.to(dev), mode=mode)
            q_out.put((rank, (lo, hi), out.float().cpu().numpy(), st.cpu().numpy()))
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,g_scale", [("shard", 1.0), ("pipeline", 1.0), ("scan", 1.0), ("scan", 40.0)])
def test_two_gpus_match_one_gpu(mode, g_scale):
    """g_scale 40: the decay is strong enough for the scan mode's early-out (segment forgotten within its first
    chunks: the second rank sends nothing extra and recomputes only a prefix); g_scale 1: full three-pass scan."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from gdn_qsa_sm80 import gdn_chunk
    world, S = 2, 512
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, S, q_out, g_scale)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q_out.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    q, k, v, g, beta, h0 = _problem(S, g_scale)
    if g_scale > 1.0:
        from gdn_qsa_sm80_b200.distributed import forgetting_horizon
        p = forgetting_horizon(k[:, 256:].float(), g[:, 256:], beta[:, 256:])
        assert p is not None and p < 256          # the early-out path is the one under test
    ref_o, ref_s = gdn_chunk(*[t.cuda() for t in (q, k, v, g, beta)], initial_state=h0.cuda())
    ref_o, ref_s = ref_o.float().cpu().numpy(), ref_s.cpu().numpy()
    if mode == "shard":
        for _, (b0, b1, h0_, h1), o, s in results:       # no communication: bit-identical to the unsharded run
            assert np.array_equal(o, ref_o[b0:b1, :, h0_:h1]) and np.array_equal(s, ref_s[b0:b1, h0_:h1])
    else:
        out = np.concatenate([r[2] for r in results], axis=1)
        assert np.abs(out - ref_o).max() < 2e-2 and np.linalg.norm(out - ref_o) <= 5e-3 * np.linalg.norm(ref_o)
        assert np.linalg.norm(results[-1][3] - ref_s) <= 5e-3 * np.linalg.norm(ref_s)
