"""Multi-GPU use of gdn_chunk: one process per GPU, `torch.distributed` for the plumbing.

The reference has no distributed code at all; this module is new.  Two cases:

* Independent sequences (`plan_shards`, `shard_inputs`): every (batch, value head) pair is its own
  recurrence (the reference's grids are (B, H, ...), csrc/gdn_chunk/gdn_kernel.cu:2892), so B x Hv is
  split over the ranks - batch first, then value heads in whole qk groups so q/k are never duplicated -
  and NO communication is needed.
* One long sequence (`sequence_parallel_forward`): the sequence is cut into contiguous segments, one per
  rank; the 128x128 fp32 boundary states per value head are passed rank to rank with send/recv (NCCL over
  NVLink on GPUs, gloo in the CPU tests).  Splitting a sequence and chaining states is exact.
  mode="pipeline": rank r waits for its incoming state, runs, sends its final state (serial, 1x work).
  mode="scan":     all ranks busy at once.  Rank 0 runs its segment from the known initial state.  Every other
                   rank first runs its segment from a zero state (giving B of S_out = A S_in + B).  If the decay
                   makes the segment forget its incoming state within its first p tokens (a bound checked on the
                   data), that pass was already right from token p on: the rank sends B at once and recomputes
                   only the first p tokens when its incoming state arrives.  Otherwise it also computes A (final
                   state from identity with zero values), the states ripple down the ranks (one small matrix
                   product per hop), and it reruns the segment from its true incoming state (3x work).
The received state always lands in this rank's own memory before any kernel reads it.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

__all__ = ["Shard", "plan_shards", "shard_inputs", "sequence_parallel_forward", "segment_bounds",
           "transfer_is_negligible", "forgetting_horizon"]

# exp(x) is below the smallest positive fp32 number (2^-149) for x < -103.3; the margin covers the 128-term sums a
# state product adds up and the slack of bf16-rounded key norms
_LOG_UNDERFLOW = -115.0


_side_streams = {}


def _side_stream(dev):
    key = torch.device(dev).index
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(dev)
    return _side_streams[key]


def _key_norm_sq_max(k):
    """max over all key vectors of |k|^2 as a 0-dim fp32 tensor on k's device: the library's one-pass kernel for
    contiguous bf16 CUDA tensors, torch otherwise."""
    if k.is_cuda and k.dtype == torch.bfloat16 and k.is_contiguous() and k.shape[-1] == 128:
        from . import _lib
        out = torch.empty((), dtype=torch.float32, device=k.device)
        with torch.cuda.device(k.device):
            st = _lib.load().gdn_key_norm_sq_max_sm100(k.data_ptr(), k.numel() // 128, out.data_ptr(),
                                                       torch.cuda.current_stream(k.device).cuda_stream)
        _lib.check(st, "gdn_key_norm_sq_max_sm100")
        return out
    return torch.linalg.vector_norm(k, ord=2, dim=-1, dtype=torch.float32).max() ** 2


def transfer_is_negligible(k, g, beta, use_qk_l2norm_in_kernel=False):
    """True when the transfer matrix A of this stretch of tokens (S_out = A S_in + B) is zero to fp32 resolution for
    every (batch, value head), by a bound that needs no pass over the state:

        A = prod_t exp(g_t) (I - beta_t k_t k_t^T),   ||I - beta k k^T||_2 <= 1  if  0 <= beta ||k||^2 <= 2,
        so  ||A||_2 <= exp(sum_t g_t)  and every entry of A S_in is below exp(sum_t g_t) ||S_in||.

    With sum_t g_t < -115 that is under 2^-149 times any state norm met in practice: the exact fp32 result of
    A S_in + B is B.  This is the rigorous form of the reference's approximate "reset" test, which thresholds a
    measured max |A| (csrc/gdn_chunk/gdn_scan_stage1_reset.cu:17-21, gdn_scan_stage3_reset.cu:1-9).  The check costs
    two small reductions and one host read; it returns False whenever the premise on beta ||k||^2 fails.
    """
    if g.numel() == 0:
        return False
    gsum_max = g.sum(dim=1, dtype=torch.float32).max()
    if use_qk_l2norm_in_kernel:
        kk_max = torch.ones((), device=k.device)
    else:   # one pass over k, no fp32 copy of it
        kk_max = _key_norm_sq_max(k)
    b_lo, b_hi = torch.aminmax(beta)
    ok = (gsum_max < _LOG_UNDERFLOW) & (kk_max * b_hi.float() <= 2.0) & (b_lo >= 0) & (g.max() <= 0)
    return bool(ok.item())


def _horizon_from(first: int, ok: int, S: int, chunk: int):
    if not ok:
        return None
    p = (first + 1) * chunk                                             # chunks [0, first] are needed
    return p if p < S else None


def forgetting_horizon_launch(k, g, beta, chunk: int = 64, keys_are_normalized=False):
    """Enqueues the computation of `forgetting_horizon` on the current stream and returns a handle for
    `forgetting_horizon_read`; nothing is read on the host.  On CUDA tensors this is the library's two small kernels
    (plus its pass over k unless keys_are_normalized); elsewhere a few torch reductions."""
    S = g.shape[1]
    if g.numel() == 0:
        return None
    if (g.is_cuda and chunk == 64 and g.is_contiguous() and beta.is_contiguous() and g.dtype == beta.dtype
            and g.dtype in (torch.float32, torch.bfloat16)):
        from . import _lib
        B, Hv = g.shape[0], g.shape[2]
        nt = (S + chunk - 1) // chunk
        kk = None if keys_are_normalized else _key_norm_sq_max(k)
        scratch = torch.empty(B * nt * Hv + 2, dtype=torch.float32, device=g.device)
        result = torch.empty(2, dtype=torch.int32, device=g.device)
        with torch.cuda.device(g.device):
            st = _lib.load().gdn_forgetting_horizon_sm100(
                g.data_ptr(), beta.data_ptr(), 1 if g.dtype == torch.float32 else 0, B, S, Hv,
                None if kk is None else kk.data_ptr(), scratch.data_ptr(), result.data_ptr(),
                torch.cuda.current_stream(g.device).cuda_stream)
        _lib.check(st, "gdn_forgetting_horizon_sm100")
        return ("kernel", result, S, chunk, (scratch, kk))
    # sums per chunk first (p is a multiple of the chunk anyway), then a short scan over the chunks
    nt = (S + chunk - 1) // chunk
    gf = g.float()
    if nt * chunk != S:
        gf = torch.nn.functional.pad(gf, (0, 0, 0, nt * chunk - S))
    per_chunk = gf.reshape(g.shape[0], nt, chunk, g.shape[2]).sum(dim=2)            # [B, nt, Hv]
    csum = torch.cumsum(per_chunk, dim=1).amax(dim=(0, 2))            # [nt]: the least-decayed head after every chunk
    below = csum < _LOG_UNDERFLOW                                       # monotone, because g <= 0
    first = torch.where(below.any(), below.float().argmax(), torch.full((), nt, device=g.device))
    if keys_are_normalized:
        kk_max = torch.ones((), device=k.device)
    else:
        kk_max = _key_norm_sq_max(k)
    b_lo, b_hi = torch.aminmax(beta)
    ok = (kk_max * b_hi.float() <= 2.0) & (b_lo >= 0) & (g.max() <= 0)
    return ("torch", torch.stack([first.float(), ok.float()]), S, chunk, None)


def forgetting_horizon_read(handle):
    """The host read that completes `forgetting_horizon_launch` (waits for the stream the launch ran on)."""
    if handle is None:
        return None
    _, result, S, chunk, _keep = handle
    first, ok = (int(x) for x in result.tolist())                       # one host read
    return _horizon_from(first, ok, S, chunk)


def forgetting_horizon(k, g, beta, chunk: int = 64, keys_are_normalized=False):
    """Number of leading tokens p (a multiple of `chunk`, or None) after which the state the stretch started from
    no longer shows in fp32: for every (batch, head) the sum of g over tokens [0, p) is below -115, so by the bound
    of `transfer_is_negligible` the transfer matrix of [0, t) vanishes for every t >= p.  Outputs at tokens >= p and
    the final state are then the same whatever the initial state was.  None when there is no such p inside the
    stretch or the premise (0 <= beta |k|^2 <= 2, g <= 0) fails.  keys_are_normalized=True skips the pass over k
    (for callers whose keys are L2-normalised by construction, or normalised inside the kernels)."""
    return forgetting_horizon_read(forgetting_horizon_launch(k, g, beta, chunk, keys_are_normalized))


@dataclass(frozen=True)
class Shard:
    b0: int
    b1: int
    hv0: int
    hv1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.hv1 - self.hv0)


def plan_shards(B: int, Hq: int, Hv: int, world: int) -> list[Shard]:
    """Partition the B x Hv independent sequences evenly over `world` ranks.

    Batch is split first; when world > B (or does not divide it) the remaining factor splits the value
    heads in whole qk groups (Hv // Hq value heads share one qk head).  Raises ValueError when no even
    partition exists.
    """
    if world <= 0 or B <= 0 or Hq <= 0 or Hv <= 0 or Hv % Hq:
        raise ValueError("bad shape")
    import math
    nb = math.gcd(B, world)          # ranks along the batch
    nh = world // nb                 # ranks along the heads
    if Hq % nh:
        raise ValueError(f"cannot split B={B}, Hq={Hq} evenly over {world} ranks")
    rep = Hv // Hq
    bs, hs = B // nb, (Hq // nh) * rep
    return [Shard(ib * bs, (ib + 1) * bs, ih * hs, (ih + 1) * hs) for ib in range(nb) for ih in range(nh)]


def shard_inputs(q, k, v, g, beta, h0, shard: Shard):
    """This rank's slice of every tensor (views; the operator makes them contiguous)."""
    rep = v.shape[2] // q.shape[2]
    hq0, hq1 = shard.hv0 // rep, shard.hv1 // rep
    sb = slice(shard.b0, shard.b1)
    out = (q[sb, :, hq0:hq1], k[sb, :, hq0:hq1], v[sb, :, shard.hv0:shard.hv1], g[sb, :, shard.hv0:shard.hv1],
           beta[sb, :, shard.hv0:shard.hv1], None if h0 is None else h0[sb, shard.hv0:shard.hv1])
    return out


def segment_bounds(S: int, world: int, chunk: int = 64) -> list[tuple[int, int]]:
    """Contiguous token ranges, one per rank, every boundary a multiple of the chunk size."""
    nt = (S + chunk - 1) // chunk
    per, extra = divmod(nt, world)
    bounds, c = [], 0
    for r in range(world):
        n = per + (1 if r < extra else 0)
        bounds.append((min(c * chunk, S), min((c + n) * chunk, S)))
        c += n
    return bounds


def sequence_parallel_forward(q, k, v, g, beta, initial_state=None, group=None, mode="pipeline", compute=None,
                              timeout_s: float | None = None, decay_early_out=True, keys_are_normalized=False):
    """Forward over THIS rank's contiguous segment of one long sequence.

    q..beta: the segment's tensors ([B, S_seg, H, ...]); initial_state: state before the whole sequence
    (only rank 0's is used).  `compute(q, k, v, g, beta, initial_state) -> (out, final_state)` defaults to
    the CUDA operator.  Returns (out_segment, final_state); the final state is the whole sequence's on the
    last rank and this segment's outgoing state elsewhere.

    decay_early_out (mode "scan"): when the decay makes a segment forget its incoming state within its first p
    tokens (`forgetting_horizon`), the rank's pass from a zero state already yields the right outputs from token p on
    and the right outgoing state.  It sends that state at once (no transfer matrix, no waiting: the rank leaves the
    serial ripple) and, once its incoming state has arrived, recomputes only the first p tokens.  A rank then does
    1 + p / S_seg passes instead of 3, and rank 0, whose incoming state is known from the start, always does one.
    Exact in fp32.

    timeout_s: upper bound, in seconds, on every wait for a neighbour's boundary state.  A rank whose predecessor
    has failed (raised before its send, left the job) then gets a RuntimeError from this call instead of waiting for
    the process group's own, much longer, time-out; None waits as long as the process group does.
    """
    if compute is None:
        from .gdn_chunk_interface import gdn_chunk

        def compute(q_, k_, v_, g_, b_, h_):
            return gdn_chunk(q_, k_, v_, g_, b_, output_final_state=True, initial_state=h_)

    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    B, Hv, D = v.shape[0], v.shape[2], v.shape[3]
    dev = v.device
    shape = (B, Hv, D, D)

    def recv_state():
        buf = torch.empty(shape, dtype=torch.float32, device=dev)
        src = dist.get_global_rank(group, rank - 1) if group is not None else rank - 1
        if timeout_s is None:
            dist.recv(buf, src=src, group=group)
            return buf
        import datetime
        work = dist.irecv(buf, src=src, group=group)
        try:
            done = work.wait(timeout=datetime.timedelta(seconds=float(timeout_s)))
        except RuntimeError as e:
            raise RuntimeError(f"rank {rank}: no boundary state from rank {rank - 1} within {timeout_s} s") from e
        if done is False:
            raise RuntimeError(f"rank {rank}: no boundary state from rank {rank - 1} within {timeout_s} s")
        return buf

    def send_state(s):
        dist.send(s.to(torch.float32).contiguous(), dst=dist.get_global_rank(group, rank + 1) if group is not None else rank + 1,
                  group=group)

    if mode == "pipeline":
        s_in = initial_state if rank == 0 else recv_state()
        out, s_out = compute(q, k, v, g, beta, s_in)
        if rank + 1 < world:
            send_state(s_out)
        return out, s_out
    if mode != "scan":
        raise ValueError(f"unknown mode {mode!r}")
    forwards = rank + 1 < world     # the last rank never forwards a state, so it needs no transfer matrix
    if rank == 0:                   # the incoming state is known: one ordinary pass, its final state goes on
        s0 = None if initial_state is None else initial_state.to(device=dev, dtype=torch.float32)
        out, s_fin = compute(q, k, v, g, beta, s0)
        if forwards:
            send_state(s_fin)
        return out, s_fin
    # The bound's reductions go first, on a side stream (they wait for the inputs only), so that they run before
    # pass A fills the GPU; their host read comes after pass A has been enqueued and returns while it executes.
    handle = None
    if decay_early_out and v.is_cuda:
        inputs_ready = torch.cuda.current_stream(dev).record_event()
        side = _side_stream(dev)
        side.wait_event(inputs_ready)
        with torch.cuda.stream(side):
            handle = forgetting_horizon_launch(k, g, beta, keys_are_normalized=keys_are_normalized)
    elif decay_early_out:
        handle = forgetting_horizon_launch(k, g, beta, keys_are_normalized=keys_are_normalized)
    # pass A: this segment from a zero state (outputs, and B_seg = its final state), on every rank at the same time
    out, b_seg = compute(q, k, v, g, beta, None)
    if decay_early_out and v.is_cuda:
        with torch.cuda.stream(_side_stream(dev)):       # the copy to the host must not queue behind pass A
            p = forgetting_horizon_read(handle)
    else:
        p = forgetting_horizon_read(handle)
    if p is not None:
        if forwards:
            send_state(b_seg)       # the outgoing state does not depend on the incoming one
        s_in = recv_state()
        head, _ = compute(q[:, :p], k[:, :p], v[:, :p], g[:, :p], beta[:, :p], s_in)
        out[:, :p] = head           # tokens >= p and the final state are already right
        return out, b_seg
    a_seg = None
    if forwards:
        eye = torch.eye(D, dtype=torch.float32, device=dev).expand(shape).contiguous()
        _, a_seg = compute(q, k, torch.zeros_like(v), g, beta, eye)
    s_in = recv_state()             # the true states ripple down the ranks
    if forwards:
        if s_in.is_cuda:    # S_out = A_seg S_in + B_seg per (batch, head), fp32, by the library's scan kernel
            from .gdn_chunk_interface import scan_transfers
            n = B * Hv
            _, s_out = scan_transfers(a_seg.to(torch.float32).reshape(n, 1, D, D), b_seg.to(torch.float32).reshape(n, 1, D, D),
                                      s_in.reshape(n, D, D))
            send_state(s_out.reshape(shape))
        else:               # CPU ranks (host-logic tests)
            send_state(torch.matmul(a_seg.to(torch.float32), s_in) + b_seg.to(torch.float32))
    # pass B: the segment from its true incoming state
    out, s_fin = compute(q, k, v, g, beta, s_in)
    return out, s_fin
