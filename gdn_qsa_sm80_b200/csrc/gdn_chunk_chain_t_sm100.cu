// "chain", transposed form: one CTA per (batch, value head[, segment]) runs the serial state recurrence and the
// outputs of all 128 value columns, reading what "prepare" left in the workspace.  The roles and the math are in
// gdn_chain_t_device.cuh; this file is the stand-alone kernel (the workspace is complete before it starts) and its
// launcher.  Stands in for the reference's gdn_recurrence_kernel (csrc/gdn_chunk/gdn_kernel.cu:1027-1271).
//
// Split sequences (ws.n_seg = G > 1, chosen from the shape when there are too few sequences to fill the GPU): every
// sequence is cut into G segments of L chunks that run as independent CTAs of ONE launch.  The second level of the
// reference's scan has the same purpose (csrc/gdn_chunk/gdn_ops.cu:1002-1012, gdn_scan_stage1.cu:7-18); here it rests
// on an exact bound instead of a propagated transfer matrix.  A stretch of tokens maps its incoming state by
// S_out = A S_in + B with A = prod_t exp(g_t)(I - beta_t k_t k_t^T), and |I - beta k k^T|_2 <= 1 whenever
// 0 <= beta |k|^2 <= 2, so |A|_2 <= exp(sum of g).  Once that sum is below -115 (exp(-115) < 2^-149) the incoming
// state no longer shows in fp32: the state after the stretch is the same from a zero state.  So segment s >= 1
// starts from a ZERO state p_s chunks before its first chunk, where p_s is the shortest stretch ending at the segment
// boundary whose sum of g is below -115 ("warm-up": its outputs are not stored), and from its first chunk on its
// state, its outputs and its final state are those of the serial run.  Per head, on the device, from the per-chunk
// scalars the prepare kernel left (ws.meta):
//   * if every segment s >= 1 has such a warm-up no longer than a segment and the premise on beta |k|^2 holds on
//     every chunk, the G CTAs of the head run their segments at once (segment 0 from the caller's initial state, the
//     last one writes the final state); segment 0, which has no warm-up, is then made longer and the others shorter
//     so that all G CTAs run about the same number of chunks, when the warm-ups at the moved boundaries allow it;
//   * otherwise the CTA of segment 0 runs the whole sequence serially and the others return at once.
// No host read, no data-dependent launch, no state passed between CTAs; results equal the serial chain's.
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_chain_t_device.cuh"
#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

constexpr int kMaxSeg = 8;

// One warp of a CTA: with segment 0 = chunks [0, L0) and segment s >= 1 = L1 chunks from L0 + (s - 1) L1 on, how many
// chunks of warm-up does segment s need (warm[s], 1 <= s < G)?  False if one of them has none within L1 chunks
// (L1 <= L0, so that many chunks always lie before a boundary).  meta: [NT][2] of this head.
__device__ __forceinline__ bool scan_warmups(const float* meta, int NT, int G, int L0, int L1, int lane, int* warm) {
    bool ok = true;
    for (int s = 1; s < G; ++s) {
        const int t0 = L0 + (s - 1) * L1;
        if (t0 >= NT) {
            if (lane == 0) warm[s] = 0;
            continue;
        }
        int p = 0;
        float carry = 0.f;
        for (int base = 0; base < L1 && p == 0; base += 32) {    // backwards from chunk t0 - 1, at most L1 chunks
            const int d = base + lane;
            float x = d < L1 ? meta[2 * (t0 - 1 - d)] : 0.f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float y = __shfl_up_sync(0xffffffffu, x, o);
                if (lane >= o) x += y;
            }
            x += carry;
            const unsigned below = __ballot_sync(0xffffffffu, d < L1 && x < kForgetLn);
            if (below) p = base + __ffs(below);                  // chunks [t0 - p, t0) make the state forget
            carry = __shfl_sync(0xffffffffu, x, 31);
        }
        if (p == 0) ok = false;                                  // no warm-up within a segment's length: no split
        if (lane == 0) warm[s] = p;
    }
    return ok;
}

// One warp of a CTA: can this head be run as G independent segments, and which ones?  Starts from equal segments of
// L chunks; when those work, segment 0 (which has no warm-up) is lengthened and the others shortened so that every
// CTA of the head runs about the same number of chunks, if the warm-ups at the moved boundaries allow it.
// Every CTA of the head computes the same answer from the same scalars.  Result: lens[0] = L0, lens[1] = L1, warm[].
__device__ __forceinline__ bool head_is_splittable(const float* meta, int NT, int G, int L, int lane, int* warm, int* lens) {
    float bmax = 0.f;
    for (int t = lane; t < NT; t += 32) bmax = fmaxf(bmax, meta[2 * t + 1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
    if (lane == 0) lens[0] = lens[1] = L;
    if (!(bmax <= 2.f)) return false;   // also for NaN and for the +inf that marks a gate out of range
    if (!scan_warmups(meta, NT, G, L, L, lane, warm)) return false;
    __syncwarp();
    int pmax = 0;
    for (int s = 1; s < G; ++s) pmax = max(pmax, warm[s]);
    // equal work: L0 = L1 + p with L0 + (G - 1) L1 = NT
    const int L1 = (NT - pmax + G - 1) / G, L0 = NT - (G - 1) * L1;
    if (pmax < 2 || L1 < 1 || L0 <= L || L0 < L1) return true;
    __shared__ int warm_moved[kMaxSeg];
    if (!scan_warmups(meta, NT, G, L0, L1, lane, warm_moved)) return true;
    __syncwarp();
    int p2 = 0;
    for (int s = 1; s < G; ++s) p2 = max(p2, warm_moved[s]);
    if (max(L0, L1 + p2) >= L + pmax) return true;   // nothing gained
    if (lane == 0) {
        for (int s = 1; s < G; ++s) warm[s] = warm_moved[s];
        lens[0] = L0;
        lens[1] = L1;
    }
    return true;
}

// SPLIT = false: one CTA per sequence.  SPLIT = true: blockIdx.z = segment.
template <bool SPLIT>
__global__ void __launch_bounds__(chain_t::kThreads, 1)
gdn_chain_t_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_t2, Problem p,
                   Workspace ws, int L) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);

    __shared__ __align__(8) uint64_t bars[chain_t::kNumBars];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int split_ok;
    __shared__ int warm[kMaxSeg];
    __shared__ int lens[2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hv = blockIdx.x, b = blockIdx.y;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const size_t seq = static_cast<size_t>(b) * p.Hv + hv;
    const chain_t::Bars cb{smem_u32(bars)};

    if (tid == 0) {
        chain_t::init_bars(bars);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, chain_t::kTmemCols);
        tmem_relinquish();
    }
    grid_dependency_wait();   // launched ahead of the end of the prepare kernel: nothing of the workspace is read above
    if (SPLIT && warp == 1) {
        const bool ok = head_is_splittable(ws.meta + seq * NT * 2, NT, ws.n_seg, L, lane, warm, lens);
        if (lane == 0) split_ok = ok ? 1 : 0;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    volatile int* abortp = &abort_flag;

    const float* h0 = p.h0 ? p.h0 + seq * kD * kD : nullptr;
    float* hT = p.hT ? p.hT + seq * kD * kD : nullptr;
    chain_t::Span sp{0, 0, 0, nullptr, nullptr};
    if (!SPLIT) {
        sp = chain_t::Span{0, NT, 0, h0, hT};
    } else {
        const int seg = static_cast<int>(blockIdx.z);
        const int t0 = seg == 0 ? 0 : lens[0] + (seg - 1) * lens[1];
        const int t1 = min(NT, seg == 0 ? lens[0] : t0 + lens[1]);
        if (!split_ok) {
            if (seg == 0) sp = chain_t::Span{0, NT, 0, h0, hT};
        } else if (t0 < NT) {
            if (seg == 0) sp = chain_t::Span{0, t1, 0, h0, t1 == NT ? hT : nullptr};
            else sp = chain_t::Span{t0 - warm[seg], t1, t0, nullptr, t1 == NT ? hT : nullptr};
        }
    }
    if (sp.t0 < sp.t1)
        chain_t::roles<false>(sm, sm_u32, tmem, cb, &tm_q, &tm_k, &tm_v, &tm_w, &tm_p, &tm_t2, p, ws, nullptr, abortp, sp, hv, b,
                              blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);

    tc_fence_before_sync();
    __syncthreads();
    if (*abortp) {   // let copies that may still be in flight land before the CTA's memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 100000ull) {}
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, chain_t::kTmemCols);
}

}  // namespace

int launch_chain_t(const Problem& p, const Workspace& ws, cudaStream_t stream) {
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tt2;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, nullptr, nullptr, 64)) return GDN_ERR_DRIVER;
    {   // T'' = T diag(beta): [tiles * 64][64] bf16 at the start of the U array
        const unsigned long long rows = static_cast<unsigned long long>(p.B) * p.Hv * ((p.S + kChunk - 1) / kChunk) * kChunk;
        const unsigned long long d[2] = {64, rows}, sb[1] = {128};
        const unsigned box[2] = {64, 64};
        if (encode_tma(&tt2, ws.U, 2, 2, d, sb, box, 128)) return GDN_ERR_DRIVER;
    }
    const uint32_t smem = chain_t::kBytes + 1024;
    const int NT = (p.S + kChunk - 1) / kChunk;
    auto go = [&](auto kernel, unsigned gz, int L) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return GDN_ERR_CUDA;
        // programmatic dependent launch: the CTAs may start (barriers, tensor memory) while the kernel before this one
        // in the stream drains; the kernel waits for that kernel's completion before it reads anything.
        // The value heads that share a qk head read the same K and Q tiles.  As a cluster of two CTAs they are
        // scheduled together and run in step, which keeps the second read of a tile close behind the first (with
        // many sequences the kernel is bound by HBM and L2 turns over every 20 microseconds); measured: 1 % off the
        // kernel with 2048 sequences, nothing lost elsewhere.  Nothing else of the cluster is used: no distributed
        // shared memory, no cluster barrier, every CTA does its own loads.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(p.Hv, p.B, gz);
        cfg.blockDim = dim3(chain_t::kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        const bool paired = (p.Hv / p.Hq) % 2 == 0 && p.Hv % 2 == 0 && p.dbg != 5;
        cfg.numAttrs = paired ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, tw, tp, tt2, p, ws, L);
        if (e != cudaSuccess && paired) {   // a context that cannot place the pairs: no clusters
            (void)cudaGetLastError();
            cfg.numAttrs = 1;
            e = cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, tw, tp, tt2, p, ws, L);
        }
        if (e != cudaSuccess) {             // ... or no dependent launch either: an ordinary launch (the kernel's wait is a no-op then)
            (void)cudaGetLastError();
            cfg.numAttrs = 0;
            e = cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, tw, tp, tt2, p, ws, L);
        }
        count_launch();
        return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
    };
    const int G = ws.n_seg;
    if (G <= 1 || G > kMaxSeg || !ws.meta) return go(gdn_chain_t_kernel<false>, 1, NT);
    return go(gdn_chain_t_kernel<true>, static_cast<unsigned>(G), (NT + G - 1) / G);
}

}  // namespace gdn
