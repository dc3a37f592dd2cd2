"""Host-side logic of the multi-GPU paths, run as gloo ranks on the CPU (world size 2 and 3):
shard planning over batch x value head, and the sequence-partitioned chain of boundary states in both
modes.  The per-rank compute is the CPU oracle here (the checker standing in for the CUDA operator), so
what is tested is the partitioning, the affine-transfer algebra and the send/recv protocol."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gdn_qsa_sm80_b200.distributed import (plan_shards, segment_bounds, sequence_parallel_forward, shard_inputs)
from gdn_qsa_sm80_b200.synthetic import make_inputs
from oracle import gdn_chunk_oracle as O


def oracle_compute(q, k, v, g, beta, h0):
    out, st = O.chunk_gated_delta_rule(*[t.double().numpy() for t in (q, k, v, g, beta)],
                                       initial_state=None if h0 is None else h0.double().numpy())
    return torch.from_numpy(out).float(), torch.from_numpy(st).float()


def test_plan_shards_partitions_every_unit_once_in_whole_qk_groups():
    for B, Hq, Hv, world in [(64, 16, 32, 8), (16, 16, 32, 4), (1, 16, 32, 8), (2, 4, 8, 8), (3, 2, 4, 1)]:
        plan = plan_shards(B, Hq, Hv, world)
        assert len(plan) == world
        cover = np.zeros((B, Hv), int)
        for s in plan:
            cover[s.b0:s.b1, s.hv0:s.hv1] += 1
            assert s.hv0 % (Hv // Hq) == 0 and s.hv1 % (Hv // Hq) == 0
            assert s.units == B * Hv // world
        assert (cover == 1).all()
    with pytest.raises(ValueError):
        plan_shards(1, 2, 4, 8)      # 8 ranks but only 2 qk groups
    with pytest.raises(ValueError):
        plan_shards(1, 3, 4, 2)


def test_sharded_compute_equals_unsharded():
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=1, B=2, S=128, Hq=2, Hv=4)
    h0 = 0.1 * torch.randn(2, 4, 128, 128, generator=torch.Generator().manual_seed(2))
    ref_o, ref_s = oracle_compute(q, k, v, g, beta, h0)
    for world in (2, 4):
        for s in plan_shards(2, 2, 4, world):
            o, st = oracle_compute(*shard_inputs(q, k, v, g, beta, h0, s))
            assert torch.equal(o, ref_o[s.b0:s.b1, :, s.hv0:s.hv1])
            assert torch.equal(st, ref_s[s.b0:s.b1, s.hv0:s.hv1])


def test_segment_bounds_are_chunk_aligned_and_cover_the_sequence():
    for S, world in [(131072, 8), (1000, 3), (64, 4), (65, 2)]:
        b = segment_bounds(S, world)
        assert b[0][0] == 0 and b[-1][1] == S and all(x[1] == y[0] for x, y in zip(b, b[1:]))
        assert all(lo % 64 == 0 for lo, _ in b)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem(S, g_scale=1.0):
    q, k, v, g, beta, _ = make_inputs("cpu_small", seed=5, B=1, S=S, Hq=1, Hv=2)
    h0 = 0.1 * torch.randn(1, 2, 128, 128, generator=torch.Generator().manual_seed(6))
    return q, k, v, g * g_scale, beta, h0


def _worker(rank, world, port, mode, S, q_out, g_scale=1.0):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, g, beta, h0 = _problem(S, g_scale)
        lo, hi = segment_bounds(S, world)[rank]
        seg = [t[:, lo:hi] for t in (q, k, v, g, beta)]
        calls = [0]

        def counted(*a):
            calls[0] += 1
            return oracle_compute(*a)

        out, st = sequence_parallel_forward(*seg, initial_state=h0, mode=mode, compute=counted)
        q_out.put((rank, out.numpy(), st.numpy(), calls[0]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["pipeline", "scan"])
@pytest.mark.parametrize("world,S", [(2, 256), (3, 320)])
def test_sequence_parallel_chain_matches_single_process(mode, world, S):
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, S, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q_out.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, k, v, g, beta, h0 = _problem(S)
    ref_o, ref_s = oracle_compute(q, k, v, g, beta, h0)
    out = np.concatenate([r[1] for r in results], axis=1)
    tol = 1e-6 if mode == "pipeline" else 2e-5      # the scan mode re-associates the state products (fp32 hop)
    assert O.rel_l2(out, ref_o.numpy()) < tol
    assert O.rel_l2(results[-1][2], ref_s.numpy()) < tol
    # weak decay: nothing may be skipped - 1 pass per rank in the pipeline; in the scan 1 on rank 0 (its incoming
    # state is known), 3 on the ranks in the middle, 2 on the last (it forwards nothing)
    assert [r[3] for r in results] == ([1] * world if mode == "pipeline" else [1] + [3] * (world - 2) + [2])


def test_scan_mode_skips_vanishing_transfer_matrices_exactly():
    """Strong decay: within 64 tokens the sum of g falls below -115 and exp of it underflows fp32, so ranks 1 and 2
    send the final state of their zero-state pass at once and recompute only their first 64 tokens (the second
    call of each); the result is that of the single process."""
    world, S, g_scale = 3, 384, 6.0
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, "scan", S, q_out, g_scale)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q_out.get(timeout=120) for _ in range(world)], key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, k, v, g, beta, h0 = _problem(S, g_scale)
    assert float(g[:, :128].sum(1).max()) < -115
    ref_o, ref_s = oracle_compute(q, k, v, g, beta, h0)
    out = np.concatenate([r[1] for r in results], axis=1)
    assert O.rel_l2(out, ref_o.numpy()) < 1e-6
    assert O.rel_l2(results[-1][2], ref_s.numpy()) < 1e-6
    assert [r[3] for r in results] == [1, 2, 2]


def test_forgetting_horizon():
    from gdn_qsa_sm80_b200.distributed import forgetting_horizon
    q, k, v, g, beta, _ = _problem(256, 6.0)
    p = forgetting_horizon(k, g, beta)
    assert p == 64 and float(g[:, :p].sum(1).max()) < -115
    assert forgetting_horizon(k, g / 6.0, beta) is None                 # never forgotten inside 256 tokens
    assert forgetting_horizon(3.0 * k, g, beta) is None                 # no norm bound
    assert forgetting_horizon(3.0 * k, g, beta, keys_are_normalized=True) == 64
    # what the horizon promises: from token p on, outputs and the final state ignore the initial state
    h0 = torch.randn(1, 2, 128, 128)
    o0, s0 = oracle_compute(q, k, v, g, beta, None)
    o1, s1 = oracle_compute(q, k, v, g, beta, h0)
    assert torch.equal(o0[:, p:], o1[:, p:]) and torch.equal(s0, s1) and not torch.equal(o0[:, :p], o1[:, :p])


def test_transfer_bound_premises():
    from gdn_qsa_sm80_b200.distributed import transfer_is_negligible
    q, k, v, g, beta, _ = _problem(256, 6.0)
    assert transfer_is_negligible(k, g, beta)
    assert not transfer_is_negligible(k, g / 6.0, beta)                 # decay too weak
    assert not transfer_is_negligible(3.0 * k, g, beta)                 # beta |k|^2 may exceed 2: no norm bound
    assert transfer_is_negligible(3.0 * k, g, beta, use_qk_l2norm_in_kernel=True)
    assert not transfer_is_negligible(k, g, beta * 1.5 + 1.0)           # beta outside [0, 1] by far
    assert not transfer_is_negligible(k, -g, beta)                      # growth instead of decay
    # the bound itself: the true transfer matrix of such a stretch is zero in fp32
    eye = torch.eye(128).expand(1, 2, 128, 128).contiguous()
    _, a = oracle_compute(q, k, torch.zeros_like(v), g, beta, eye)
    assert float(a.abs().max()) == 0.0


def _failing_worker(rank, world, port, failure, q_out):
    """Rank 0 fails on the host before it would send its boundary state; rank 1 must get an error, not wait."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    import datetime
    import time
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        S = 128
        q, k, v, g, beta, h0 = _problem(S)
        lo, hi = segment_bounds(S, world)[rank]
        seg = [t[:, lo:hi] for t in (q, k, v, g, beta)]

        def compute(*a):
            if rank == 0 and failure == "raises":
                raise ValueError("injected failure before the send")
            if rank == 0 and failure == "stalls":
                time.sleep(8.0)             # far longer than the neighbour is willing to wait
            return oracle_compute(*a)

        t0 = time.time()
        try:
            sequence_parallel_forward(*seg, initial_state=h0, mode="pipeline", compute=compute, timeout_s=2.0)
            q_out.put((rank, "ok", time.time() - t0))
        except ValueError as e:
            q_out.put((rank, "raised:" + str(e), time.time() - t0))
        except RuntimeError as e:
            q_out.put((rank, "timeout:" + str(e), time.time() - t0))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("failure", ["raises", "stalls"])
def test_a_failed_neighbour_ends_the_wait_with_an_error(failure):
    """Host-side failure detection of the sequence-parallel chain: a rank that raises before its send, or does not
    send in time, makes its successor's bounded receive raise instead of blocking."""
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, failure, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict()
    for _ in range(2):
        r = q_out.get(timeout=120)
        results[r[0]] = r
    for p in procs:
        p.join(timeout=60)
    assert results[1][1].startswith("timeout:") and "no boundary state from rank 0" in results[1][1]
    assert results[1][2] < 7.0                        # the 2 s limit, not the process group's 60 s
    assert results[0][1].startswith("raised:") if failure == "raises" else results[0][1] in ("ok",) or results[0][1].startswith("timeout:")
