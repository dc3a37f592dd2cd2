// "prepare": everything of a chunk that does not depend on the recurrent state, one CTA per
// (batch, value head, chunk), fully parallel over the sequence.
//
// For each 64-token chunk it produces, in the notation of the reference's torch definition
// (gdn_qsa_sm80/reference/gdn_chunk_ref.py:56-78):
//   gamma   inclusive cumsum of the log gate (warp shuffles), and from it the per-token factors
//           exp(gamma_C - gamma_i), scale*exp(gamma_i), exp(gamma_C)                  -> vec  [256] fp32
//   P     = tril(scale * exp(gamma_i - gamma_j) * Q K^T)          ("intra_chunk_attn")  -> P    [64][64]  bf16
//   T     = (I + tril(beta_i exp(gamma_i - gamma_j) K K^T, -1))^-1
//   W     = T (beta e^gamma K)                                   ("k_cumdecay")        -> W    [64][128] bf16
//   U     = T (beta V)                                           ("new_values")        -> U    [64][128] bf16
// K K^T, Q K^T, T [beta e^gamma K | beta V] run on tcgen05 with TMA-staged tiles; the decay mask is
// applied in fp32 while the raw products move from TMEM to registers.  The reference computes the
// same quantities in gdn_prepare_kernel (csrc/gdn_chunk/gdn_kernel.cu:343-710) at chunk 16 with the
// decay folded into the operands; here the pairwise factor exp(gamma_i - gamma_j) <= 1 is used, which
// stays finite at chunk 64.
//
// Persistent CTAs (two per SM: 106 KB of shared memory and 256 TMEM columns each) walk the tiles; the
// next tile's TMA loads and gate reads are issued as soon as the last UMMA of the current tile has
// finished, W and U leave through swizzled staging tiles and asynchronous TMA stores, and one CTA's
// tensor-core and memory latencies hide behind its neighbour's CUDA-core phases.
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "gdn_prep_device.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

// 71 KB per CTA so that three CTAs share an SM: every buffer is reused as soon as its contents are dead.
struct PSmem {
    static constexpr uint32_t KQ = 0;                    // [K;Q]: 2 k-halves x 128 rows x 128 B; V takes Q's place after Q K^T
    static constexpr uint32_t AS = KQ + 32768;           // A fp32 64 x 68, then the bf16 operand [T';T''], then the U staging tile
    static constexpr uint32_t TM = AS + 17408;           // T fp32 64 x 68, then the W staging tile
    static constexpr uint32_t YT = TM + 17408;           // merge temporaries
    static constexpr uint32_t kBytes = YT + 5120;        // 72704
    static constexpr uint32_t kDynamic = kBytes + 1024;
};
// 128 TMEM columns (three CTAs: 384 of the SM's 512): K K^T / Q K^T in the first 64, then W, then U through all 128
constexpr uint32_t kPrepTmemCols = 128;
constexpr int kPrepCtasPerSm = 3;

// WITH_U = false: for the transposed chain, which forms U^T = V^T T''^T itself from the raw V tile: no V load, no
// second product, no U tile; T'' = T diag(beta) (bf16, 64 x 64, row-major) goes to the workspace instead (tm_u then
// describes T''), and both T'' and P leave through swizzled tiles and TMA stores: T'' from the operand's rows 64-127,
// P from a tile in Q's place (rows stored one per thread straight to global memory cost a wavefront per lane).
template <bool GATE_F32, bool WITH_U>
__global__ void __launch_bounds__(128, kPrepCtasPerSm)
gdn_prepare_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_u, const __grid_constant__ CUtensorMap tm_p, Problem p,
                   Workspace ws, int NT, long long num_tiles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);
    __shared__ __align__(8) uint64_t bar_tma;
    __shared__ __align__(8) uint64_t bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) PrepScratch ps;

    const int tid = threadIdx.x, warp = tid >> 5;
    const float scale0 = rsqrtf(static_cast<float>(kD));
    const int i = tid & 63;

    // Persistent CTA: tiles L = blockIdx.x, blockIdx.x + gridDim.x, ...  L -> (b, chunk t, head hv) with the
    // head index fastest, so the value heads that share a qk head are prepared at about the same time.
    struct Tile { int b, t, hv, hq, s0; size_t ws_tile; };
    auto decode = [&](long long L) {
        Tile x;
        x.hv = static_cast<int>(L % p.Hv);
        x.t = static_cast<int>((L / p.Hv) % NT);
        x.b = static_cast<int>(L / (static_cast<long long>(p.Hv) * NT));
        x.hq = x.hv / (p.Hv / p.Hq);
        x.s0 = x.t * kChunk;
        x.ws_tile = (static_cast<size_t>(x.b) * p.Hv + x.hv) * NT + x.t;
        return x;
    };
    auto issue_loads = [&](const Tile& x) {   // one thread
        mbar_arrive_expect_tx(&bar_tma, 4 * 8192);
        tma_load_4d(sm + PSmem::KQ + 0, &tm_k, &bar_tma, 0, x.hq, x.s0, x.b);        // K, d 0-63   -> rows 0-63
        tma_load_4d(sm + PSmem::KQ + 16384, &tm_k, &bar_tma, 64, x.hq, x.s0, x.b);   // K, d 64-127
        tma_load_4d(sm + PSmem::KQ + 8192, &tm_q, &bar_tma, 0, x.hq, x.s0, x.b);     // Q           -> rows 64-127
        tma_load_4d(sm + PSmem::KQ + 24576, &tm_q, &bar_tma, 64, x.hq, x.s0, x.b);
    };
    auto issue_v = [&](const Tile& x) {       // one thread, once Q K^T is done: V (two 64-column groups) replaces Q
        mbar_arrive_expect_tx(&bar_tma, 2 * 8192);
        tma_load_4d(sm + PSmem::KQ + 8192, &tm_v, &bar_tma, 0, x.hv, x.s0, x.b);
        tma_load_4d(sm + PSmem::KQ + 24576, &tm_v, &bar_tma, 64, x.hv, x.s0, x.b);
    };

    // optional cycle accounting by thread 0 of CTA 0, summed over its tiles (slot 15 counts the tiles)
    const bool prof_on = GDN_DIAG(p.prof != nullptr && tid == 0 && blockIdx.x == 0);
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long prof_t = prof_on ? clock64() : 0;
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_acc[n] += now_ - prof_t;                  \
        prof_t = now_;                                 \
    }

    long long L = blockIdx.x;
    Tile cur = decode(L);
    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        fence_mbar_init();
        issue_loads(cur);
    }
    grid_launch_dependents();   // the chain kernel may set up its CTAs on SMs this grid has left
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kPrepTmemCols);
        tmem_relinquish();
    }
    float gv, bv;
    prep_load_gates<GATE_F32>(p.g, p.beta, static_cast<size_t>(cur.b) * p.S + cur.s0, cur.hv, p.Hv,
                              min(kChunk, p.S - cur.s0), gv, bv, PrepCtx::whole_cta(), p.gate_act != 0);
    float* As = reinterpret_cast<float*>(sm + PSmem::AS);
    float* Tm = reinterpret_cast<float*>(sm + PSmem::TM);
    float* Yt = reinterpret_cast<float*>(sm + PSmem::YT);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;
    uint32_t ph_tma = 0, ph_mma = 0;
    bool ok = true;
    long long tiles_done = 0;

    for (; L < num_tiles && ok; L += gridDim.x) {
        const size_t tile = cur.ws_tile;
        if (p.gate_act) prep_activate_gates(gv, bv);
        prep_gates(ps, gv, bv, scale0, ws.vec + tile * 256, PrepCtx::whole_cta(), false);
        __syncthreads();
        GDN_PHASE(0)

        ok = mbar_wait(&bar_tma, ph_tma, p.status, kDevTimeoutTma);
        ph_tma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        GDN_PHASE(1)

        if (tid == 0) {   // raw K K^T (lanes 0-63) and Q K^T (lanes 64-127)
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + PSmem::KQ + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                umma_bf16_ss(tmem, ad, ad, idesc, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        if (p.l2norm) {   // while the UMMAs run
            prep_l2norm_fold(ps, sm + PSmem::KQ, ws.vec + tile * 256);
            if (tid < kChunk) ps.ctab[0][tid] = ps.gam[tid] - __log2f(ps.rn[tid]);   // column table of the mask epilogue
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        // the previous tile's W/U stores must have finished reading their staging tiles (the T and A buffers) before
        // those are zeroed / overwritten below; waited for here rather than at the top of the loop, the gates, the
        // TMA wait and the first UMMAs have hidden most of that latency.  Q is dead now: V takes its place.
        if (tid == 0) {
            tma_store_wait_read();
            if (WITH_U) issue_v(cur);
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        GDN_PHASE(2)
        prep_zero_upper_blocks(Tm);   // the T buffer held the previous tile's W staging tile until the wait above

        tc_fence_after_sync();
        {   // mask epilogue (one exponential per element, shared with gdn_prepare_pair_kernel, so that both kernels
            // produce the same bits): thread = row i = TMEM lane
            const bool low_rows = (warp & 1) == 0;           // rows 0-31: columns 32-63 lie above the diagonal
            if (warp < 2) {   // A = tril(beta_i * decay * K K^T, -1), fp32, for the inverse
                const float ksq = prep_mask_row_A(ps, p.l2norm != 0, tmem_addr(tmem, lane_base, 0), i, low_rows, As, ws.meta != nullptr);
                if (ws.meta) {
                    const float bound = prep_bound_of_rows(ps, p.l2norm != 0, i, ksq);
                    if ((tid & 31) == 0) ps.wsum[warp] = bound;   // the cumsum's slots are free again by now
                }
            } else if (WITH_U) {   // P = tril(scale * decay * Q K^T), bf16, straight to the workspace (V is taking Q's place)
                prep_mask_row_P(ps, p.l2norm != 0, scale0, tmem_addr(tmem, lane_base, 0), i, low_rows,
                                ws.P + tile * (kChunk * kChunk) + static_cast<size_t>(i) * kChunk);
            } else {               // ... into a staging tile in the place of Q's first k-half (Q is dead, no V comes)
                uint4 pk[8];
                prep_mask_row_P_packed(ps, p.l2norm != 0, scale0, tmem_addr(tmem, lane_base, 0), i, low_rows, pk);
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)
                    *reinterpret_cast<uint4*>(sm + PSmem::KQ + 8192 + swz_chunk_offset<128>(i, ch)) = pk[ch];
                fence_proxy_async_smem();
            }
        }
        tc_fence_before_sync();
        __syncthreads();
        if (!WITH_U && tid == 0) {
            tma_store_2d(&tm_p, sm + PSmem::KQ + 8192, 0, static_cast<int>(tile * kChunk));
            tma_store_commit();
        }
        if (ws.meta && tid == 0) {
            ws.meta[2 * tile] = ps.gam[kChunk - 1] * (1.f / kLog2e);
            ws.meta[2 * tile + 1] = fmaxf(ps.wsum[0], ps.wsum[1]);
        }
        GDN_PHASE(3)

        prep_invert_unit_lower(As, Tm, Yt);
        GDN_PHASE(4)

        {   // [T diag(beta e^gamma) ; T diag(beta)] as one 128-row K-major operand
            const int which = tid >> 6;
            // without U, rows 64-127 are only the staging tile of T'' (their product rows are never read)
            prep_store_scaled_T_row(Tm, which == 0 ? ps.eg : ps.bet, i, sm + PSmem::AS, which * 64 + i);   // A is dead
        }
        fence_proxy_async_smem();
        __syncthreads();
        if (!WITH_U && tid == 0) {
            tma_store_2d(&tm_u, sm + PSmem::AS + 8192, 0, static_cast<int>(tile * kChunk));
            tma_store_commit();
        }
        if (WITH_U) {
            ok = mbar_wait(&bar_tma, ph_tma, p.status, kDevTimeoutTma);   // V has landed
            ph_tma ^= 1;
            ok = __syncthreads_and(ok);
            if (!ok) break;
        }
        GDN_PHASE(5)

        // W = T' K and U = T'' V go through the same 128 TMEM columns one after the other.  Both products use the
        // stacked operand [T';T''] (M = 128): rows 0-63 of the first are W, rows 64-127 of the second are U.
        constexpr uint32_t idesc_wu = umma_idesc_bf16(128, 128, MAJOR_K, MAJOR_MN);
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + PSmem::AS + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bk = umma_smem_desc(sm_u32 + PSmem::KQ + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tmem, ad, bk, idesc_wu, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (warp < 2) {   // W rows (lanes 0-63) -> bf16 -> swizzled staging tile in the T buffer (T fp32 is dead)
            uint32_t r[32];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, q4 * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                    pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                    pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                    pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                    *reinterpret_cast<uint4*>(sm + PSmem::TM + (q4 >> 1) * 8192 +
                                              swz_chunk_offset<128>(i, (q4 & 1) * 4 + ch)) = pk;
                }
            }
        }
        if (WITH_U) {
        tc_fence_before_sync();
        __syncthreads();          // W has left the accumulator
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + PSmem::AS + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bv_ = umma_smem_desc(sm_u32 + PSmem::KQ + 8192 + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tmem, ad, bv_, idesc_wu, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        }
        GDN_PHASE(6)

        // K, V and the [T';T''] operand are dead: start the next tile's loads and gate reads before the epilogue
        const long long Ln = L + gridDim.x;
        Tile nxt = cur;
        if (Ln < num_tiles) {
            nxt = decode(Ln);
            if (tid == 0) {
                if (!WITH_U) tma_store_wait_read();   // the P tile in Q's place has been read
                issue_loads(nxt);
            }
            prep_load_gates<GATE_F32>(p.g, p.beta, static_cast<size_t>(nxt.b) * p.S + nxt.s0, nxt.hv, p.Hv,
                                      min(kChunk, p.S - nxt.s0), gv, bv, PrepCtx::whole_cta(), p.gate_act != 0);
        }
        tc_fence_after_sync();
        if (WITH_U && warp >= 2) {   // U rows (lanes 64-127) -> staging tile in the A buffer (the operand there is dead)
            uint32_t r[32];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, q4 * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                    pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                    pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                    pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                    *reinterpret_cast<uint4*>(sm + PSmem::AS + (q4 >> 1) * 8192 +
                                              swz_chunk_offset<128>(i, (q4 & 1) * 4 + ch)) = pk;
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            const int row0 = static_cast<int>(tile * kChunk);
            tma_store_2d(&tm_w, sm + PSmem::TM, 0, row0);
            tma_store_2d(&tm_w, sm + PSmem::TM + 8192, 64, row0);
            if (WITH_U) {
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) tma_store_2d(&tm_u, sm + PSmem::AS + h2 * 8192, h2 * 64, row0);
            }
            tma_store_commit();
        }
        GDN_PHASE(7)
        cur = nxt;
        ++tiles_done;
    }
#undef GDN_PHASE
    if (prof_on) {
        for (int n = 0; n < 8; ++n) p.prof[n] = prof_acc[n];
        p.prof[15] = tiles_done;
    }
    if (tid == 0) tma_store_wait_all();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kPrepTmemCols);
}

}  // namespace

int launch_prepare(const Problem& p, const Workspace& ws, cudaStream_t stream, bool with_u) {
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tu;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, &tu, nullptr, 64)) return GDN_ERR_DRIVER;
    const int NT = (p.S + kChunk - 1) / kChunk;
    if (!with_u) {   // T'' = T diag(beta): [tiles * 64][64] bf16 at the start of the U array
        const unsigned long long rows = static_cast<unsigned long long>(p.B) * p.Hv * NT * kChunk;
        const unsigned long long d[2] = {64, rows}, sb[1] = {128};
        const unsigned box[2] = {64, 64};
        if (encode_tma(&tu, ws.U, 2, 2, d, sb, box, 128)) return GDN_ERR_DRIVER;
    }
    const long long tiles = static_cast<long long>(p.B) * p.Hv * NT;
    const long long max_ctas = static_cast<long long>(kPrepCtasPerSm) * sm_count();
    const unsigned grid = static_cast<unsigned>(tiles < max_ctas ? tiles : max_ctas);
    auto go = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PSmem::kDynamic) != cudaSuccess)
            return GDN_ERR_CUDA;
        kernel<<<grid, 128, PSmem::kDynamic, stream>>>(tq, tk, tv, tw, tu, tp, p, ws, NT, tiles);
        count_launch();
        return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
    };
    if (with_u) return p.gate_f32 ? go(gdn_prepare_kernel<true, true>) : go(gdn_prepare_kernel<false, true>);
    return p.gate_f32 ? go(gdn_prepare_kernel<true, false>) : go(gdn_prepare_kernel<false, false>);
}

}  // namespace gdn
