// "prepare" for the transposed chain, two value heads at a time.
//
// The value heads that share a qk head (the reference's head mapping, csrc/gdn_chunk/gdn_kernel.cu:385-387) share
// K, Q and therefore the raw products K K^T and Q K^T; only the gates differ.  One CTA of 256 threads prepares the
// chunk of BOTH heads of a pair: one K / Q load and one [K;Q] K^T product for the two, then per head (one half of
// the CTA each, in parallel) the decay mask, the 64 x 64 triangular inverse and T'' = T diag(beta), and finally ONE
// product [T'_a ; T'_b] K (M = 128, no wasted rows) that yields W of both heads.  U is not formed: the transposed
// chain computes U^T = V^T T''^T itself from the raw V tile.  Per head and chunk the workspace receives
//   W [64][128] bf16,  P [64][64] bf16,  T'' [64][64] bf16 (at the start of the U array),  the per-token factors and
//   the two scalars of the decay bound (sum of g, max beta |k|^2).
// W, P and T'' all leave through 128-byte-swizzled staging tiles and TMA stores (rows stored one per thread straight to
// global memory cost the LSU data pipe, this kernel's busiest unit, a wavefront per lane).
// Same math and the same device helpers as gdn_prepare_kernel (gdn_chunk_prepare_sm100.cu), which remains the
// producer for an odd number of value heads per qk head and for the kernels that read U from the workspace.
// Stands in for the reference's gdn_prepare_kernel (csrc/gdn_chunk/gdn_kernel.cu:343-710).
//
// Two CTAs per SM (101 KB of shared memory, 128 TMEM columns, 128 registers each): 16 warps whose phases overlap.
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "gdn_prep_device.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

struct QSmem {
    static constexpr uint32_t KQ = 0;                    // [K;Q]: 2 k-halves x 128 rows x 128 B (K rows 0-63, Q rows 64-127)
    static constexpr uint32_t YT = KQ + 8192;            // merge temporaries of head h at YT + h * 16384: Q's rows, dead after Q K^T
    static constexpr uint32_t AS = KQ + 32768;           // A fp32 64 x 68 of head h at AS + h * 17408 ...
    static constexpr uint32_t OP = AS;                   // ... then the stacked bf16 operand [T'_a ; T'_b] (16 KB) over head a's A,
                                                         //     and after the second product the P staging tiles of both heads there
    static constexpr uint32_t T2S = AS + 17408;          // ... and the T'' staging tiles of both heads (16 KB) over head b's A
    static constexpr uint32_t TM = AS + 2 * 17408;       // T fp32 64 x 68 of head h at TM + h * 17408 ...
    static constexpr uint32_t STG = TM;                  // ... then the W staging tiles of both heads (32 KB)
    static constexpr uint32_t kBytes = TM + 2 * 17408;   // 102400
    static constexpr uint32_t kDynamic = kBytes + 1024;
    static_assert(OP % 1024 == 0 && STG % 1024 == 0 && T2S % 1024 == 0, "UMMA / TMA tiles must be 1024-byte aligned");
};
constexpr uint32_t kPairTmemCols = 128;   // [K;Q] K^T in the first 64, then W of both heads through all 128
constexpr int kPairCtasPerSm = 2;

template <bool GATE_F32>
__global__ void __launch_bounds__(256, kPairCtasPerSm)
gdn_prepare_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_p,
                        const __grid_constant__ CUtensorMap tm_t2, Problem p, Workspace ws, int NT, long long num_items) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);
    __shared__ __align__(8) uint64_t bar_tma;
    __shared__ __align__(8) uint64_t bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) PrepScratch ps2[2];
    __shared__ float gates_b[2][kChunk];   // head b's log gate and update gate of the coming item, loaded by head a's half

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = tid >> 7;                       // which head of the pair this half of the CTA prepares
    const int htid = tid & 127, hwarp = htid >> 5, i = htid & 63;
    const PrepCtx ctx{htid, 1 + h};               // the half's own thread numbering and named barrier
    PrepScratch& ps = ps2[h];
    const float scale0 = rsqrtf(static_cast<float>(kD));
    const int rep = p.Hv / p.Hq, npairs = p.Hv / 2;
    float* As = reinterpret_cast<float*>(sm + QSmem::AS + h * 17408);
    float* Tm = reinterpret_cast<float*>(sm + QSmem::TM + h * 17408);
    float* Yt = reinterpret_cast<float*>(sm + QSmem::YT + h * 16384);
    uint8_t* kq = sm + QSmem::KQ;

    // Persistent CTA: items L = blockIdx.x, blockIdx.x + gridDim.x, ...  L -> (b, chunk t, pair of value heads), the
    // pair index fastest.
    struct Item { int b, t, hv, hq, s0; size_t tile; };
    auto decode = [&](long long L) {
        Item x;
        const int pr = static_cast<int>(L % npairs);
        x.t = static_cast<int>((L / npairs) % NT);
        x.b = static_cast<int>(L / (static_cast<long long>(npairs) * NT));
        x.hv = 2 * pr + h;
        x.hq = (2 * pr) / rep;
        x.s0 = x.t * kChunk;
        x.tile = (static_cast<size_t>(x.b) * p.Hv + x.hv) * NT + x.t;
        return x;
    };
    auto issue_loads = [&](const Item& x) {   // one thread
        mbar_arrive_expect_tx(&bar_tma, 4 * 8192);
        tma_load_4d(kq + 0, &tm_k, &bar_tma, 0, x.hq, x.s0, x.b);
        tma_load_4d(kq + 16384, &tm_k, &bar_tma, 64, x.hq, x.s0, x.b);
        tma_load_4d(kq + 8192, &tm_q, &bar_tma, 0, x.hq, x.s0, x.b);
        tma_load_4d(kq + 24576, &tm_q, &bar_tma, 64, x.hq, x.s0, x.b);
    };

    // optional cycle accounting (diagnostics builds) by thread 0 of CTA 0, summed over its items; slot 15 counts them.
    // Phases: 0 wait for K/Q, 1 first product + gates, 2 mask epilogue, 3 barrier + bound, 4 inverse, 5 T' / T'',
    // 6 second product, 7 W staging and stores.
    const bool prof_on = GDN_DIAG(p.prof != nullptr && tid == 0 && blockIdx.x == 0);
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long prof_t = prof_on ? clock64() : 0, prof_n = 0;
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_acc[n] += now_ - prof_t;                  \
        prof_t = now_;                                 \
    }

    long long L = blockIdx.x;
    Item cur = decode(L);
    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        fence_mbar_init();
        issue_loads(cur);
    }
    grid_launch_dependents();   // the chain kernel may set up its CTAs on SMs this grid has left
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kPairTmemCols);
        tmem_relinquish();
    }
    // The gates of the two heads of a pair lie side by side in memory: head a's half loads both with one 8-byte (fp32)
    // or 4-byte (bf16) access per token and hands head b's over through shared memory at the top of the item (a token
    // per lane, a row of heads apart: every access is a sector of its own, so two halves loading one head each
    // fetched every sector twice).  Padding tokens: zeros, or (raw gates) what prep_activate_gates maps to zeros.
    float gv, bv, gv_b = 0.f, bv_b = 0.f;
    auto load_gates_of_pair = [&](const Item& x) {
        if (h != 0 || htid >= kChunk) return;
        const float pad = p.gate_act ? -INFINITY : 0.f;
        gv = bv = gv_b = bv_b = pad;
        if (htid < min(kChunk, p.S - x.s0)) {
            const size_t idx = (static_cast<size_t>(x.b) * p.S + x.s0 + htid) * p.Hv + x.hv;   // x.hv: head a (even)
            if (GATE_F32) {
                const float2 g2 = *reinterpret_cast<const float2*>(static_cast<const float*>(p.g) + idx);
                const float2 b2 = *reinterpret_cast<const float2*>(static_cast<const float*>(p.beta) + idx);
                gv = g2.x; gv_b = g2.y; bv = b2.x; bv_b = b2.y;
            } else {
                const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(p.g) + idx));
                const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(p.beta) + idx));
                gv = g2.x; gv_b = g2.y; bv = b2.x; bv_b = b2.y;
            }
        }
    };
    auto hand_over_gates = [&]() {   // before the barrier at the top of the item they belong to
        if (h == 0 && htid < kChunk) {
            gates_b[0][htid] = gv_b;
            gates_b[1][htid] = bv_b;
        }
    };
    load_gates_of_pair(cur);
    hand_over_gates();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = static_cast<uint32_t>(hwarp) * 32u;   // (warp % 4) * 32: the warp's TMEM lane quadrant
    uint32_t ph_tma = 0, ph_mma = 0;
    bool ok = true;

    for (; L < num_items && ok; L += gridDim.x) {
        const size_t tile = cur.tile;
        ok = mbar_wait(&bar_tma, ph_tma, p.status, kDevTimeoutTma);
        ph_tma ^= 1;
        ok = __syncthreads_and(ok);   // also: every warp has left the previous item's accumulator
        if (!ok) break;
        if (h == 1 && htid < kChunk) {
            gv = gates_b[0][htid];
            bv = gates_b[1][htid];
        }
        GDN_PHASE(0)

        if (tid == 0) {   // raw K K^T (lanes 0-63) and Q K^T (lanes 64-127), shared by the two heads
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + QSmem::KQ + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                umma_bf16_ss(tmem, ad, ad, idesc, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        // the gate cumsum and the decay tables need nothing from the tiles: they run while the product does
        if (p.gate_act) prep_activate_gates(gv, bv);
        prep_gates(ps, gv, bv, scale0, ws.vec + tile * 256, ctx, false);
        ctx.sync();
        if (p.l2norm) {   // while the UMMAs run
            prep_l2norm_fold(ps, kq, ws.vec + tile * 256, ctx);
            if (htid < kChunk) ps.ctab[0][htid] = ps.gam[htid] - __log2f(ps.rn[htid]);   // column table of the mask epilogue
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        // the previous item's W stores must have finished reading their staging tiles (the T buffers) before the
        // inverse writes them again
        if (tid == 0) tma_store_wait_read();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        GDN_PHASE(1)

        tc_fence_after_sync();
        // Row i of P (warps 2, 3 of each half).  Rows written one per thread straight to global memory cost the LSU
        // data pipe a wavefront per lane and store (a third of the kernel's wavefronts when P and T'' left that
        // way); so P, like T'' and W, leaves through a swizzled staging tile and a TMA store.  No shared memory is
        // free for the tile before the second product has read its operand, hence the wait in registers.
        uint4 prow[8];
        {   // mask epilogue (one exponential per element, shared with gdn_prepare_kernel): thread = row i = TMEM lane
            const bool low_rows = (hwarp & 1) == 0;          // rows 0-31: columns 32-63 lie above the diagonal
            if (hwarp < 2) {   // A = tril(beta_i * decay * K K^T, -1), fp32, for the inverse
                const float ksq = prep_mask_row_A(ps, p.l2norm != 0, tmem_addr(tmem, lane_base, 0), i, low_rows, As, ws.meta != nullptr);
                if (ws.meta) {   // max over the chunk of beta_i |k_i|^2, +inf when a gate is outside beta >= 0, g <= 0
                    const float bound = prep_bound_of_rows(ps, p.l2norm != 0, i, ksq);
                    if (lane == 0) ps.wsum[hwarp] = bound;   // the cumsum's slots are free again by now
                }
                // the 32 x 32 diagonal block of T over this warp's own rows needs nobody else: no barrier, and it runs
                // while the other warps are still in their part of the mask epilogue
                __syncwarp();
                prep_invert_diag32(As, Tm, Yt + kDiagScratch * hwarp, hwarp, lane);
            } else {           // P = tril(scale * decay * Q K^T), bf16: the row waits in registers for its staging tile
                prep_mask_row_P_packed(ps, p.l2norm != 0, scale0, tmem_addr(tmem, lane_base, 0), i, low_rows, prow);
            }
        }
        GDN_PHASE(2)
        tc_fence_before_sync();
        ctx.sync();
        if (ws.meta && htid == 0) {
            ws.meta[2 * tile] = ps.gam[kChunk - 1] * (1.f / kLog2e);
            ws.meta[2 * tile + 1] = fmaxf(ps.wsum[0], ps.wsum[1]);
        }

        GDN_PHASE(3)
        prep_invert_level2(As, Tm, Yt, ctx);
        GDN_PHASE(4)

        // both heads are done with their A matrices (the stacked operand lies over head a's) and with the raw
        // products in tensor memory (W goes through the same columns)
        __syncthreads();
        // T' = T diag(beta e^gamma) (rows 64 h .. 64 h + 63 of the stacked operand) and T'' = T diag(beta) (as it is, for
        // the chain's V^T T''^T): every thread reads half a row of T once and writes both
        prep_store_T_half_row_tiles(Tm, ps.eg, ps.bet, i, htid >> 6, sm + QSmem::OP, h * 64 + i,
                                    sm + QSmem::T2S + h * 8192, i);
        fence_proxy_async_smem();
        __syncthreads();
        GDN_PHASE(5)

        if (tid == 0) {   // W of both heads: [T'_a ; T'_b] K
            tc_fence_after_sync();
            constexpr uint32_t idesc_w = umma_idesc_bf16(128, 128, MAJOR_K, MAJOR_MN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + QSmem::OP + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bk = umma_smem_desc(sm_u32 + QSmem::KQ + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tmem, ad, bk, idesc_w, ks > 0);
            }
            umma_commit(&bar_mma);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)   // T'' of both heads; tid 0 is in half 0: tile = head a's
                tma_store_2d(&tm_t2, sm + QSmem::T2S + hh * 8192, 0, static_cast<int>((tile + static_cast<size_t>(hh) * NT) * kChunk));
            tma_store_commit();
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();
        GDN_PHASE(6)

        // K, Q (the merge temporaries) and the operand are dead: the next item's loads and gate reads start now
        const long long Ln = L + gridDim.x;
        Item nxt = cur;
        if (Ln < num_items) {
            nxt = decode(Ln);
            if (tid == 0) issue_loads(nxt);
            load_gates_of_pair(nxt);
        }
        {   // W rows -> bf16 -> swizzled staging tiles in the T buffers (T fp32 is dead).  TMEM lanes 0-63 are head a's
            // rows, 64-127 head b's; warps 0-3 take columns 0-63, warps 4-7 columns 64-127.
            const int hh = hwarp >> 1, row = (hwarp & 1) * 32 + lane, cpart = warp >> 2;
            uint8_t* dst = sm + QSmem::STG + hh * 16384 + cpart * 8192;
            uint32_t r[32];
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, cpart * 64 + q2 * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                    pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                    pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                    pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                    *reinterpret_cast<uint4*>(dst + swz_chunk_offset<128>(row, q2 * 4 + ch)) = pk;
                }
            }
        }
        if (hwarp >= 2) {   // the P rows: staging tile of head h over the operand, which the second product has read
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
                *reinterpret_cast<uint4*>(sm + QSmem::OP + h * 8192 + swz_chunk_offset<128>(i, ch)) = prow[ch];
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int row0 = static_cast<int>((tile + static_cast<size_t>(hh) * NT) * kChunk);   // tid 0 is in half 0: tile = head a's
                tma_store_2d(&tm_w, sm + QSmem::STG + hh * 16384, 0, row0);
                tma_store_2d(&tm_w, sm + QSmem::STG + hh * 16384 + 8192, 64, row0);
                tma_store_2d(&tm_p, sm + QSmem::OP + hh * 8192, 0, row0);
            }
            tma_store_commit();
        }
        hand_over_gates();   // the next item's, loaded above: they have had the whole staging to arrive
        GDN_PHASE(7)
        ++prof_n;
        cur = nxt;
    }
#undef GDN_PHASE
    if (prof_on) {
        for (int n = 0; n < 8; ++n) p.prof[n] = prof_acc[n];
        p.prof[15] = prof_n;
    }
    if (tid == 0) tma_store_wait_all();
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kPairTmemCols);
}

}  // namespace

int launch_prepare_pair(const Problem& p, const Workspace& ws, cudaStream_t stream) {
    if (p.Hv % 2 || (p.Hv / p.Hq) % 2) return GDN_ERR_BAD_ARGUMENT;
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tt2;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, nullptr, nullptr, 64)) return GDN_ERR_DRIVER;
    const int NT = (p.S + kChunk - 1) / kChunk;
    {   // T'' = T diag(beta): [tiles * 64][64] bf16 at the start of the U array
        const unsigned long long rows = static_cast<unsigned long long>(p.B) * p.Hv * NT * kChunk;
        const unsigned long long d[2] = {64, rows}, sb[1] = {128};
        const unsigned box[2] = {64, 64};
        if (encode_tma(&tt2, ws.U, 2, 2, d, sb, box, 128)) return GDN_ERR_DRIVER;
    }
    const long long items = static_cast<long long>(p.B) * (p.Hv / 2) * NT;
    const long long max_ctas = static_cast<long long>(kPairCtasPerSm) * sm_count();
    const unsigned grid = static_cast<unsigned>(items < max_ctas ? items : max_ctas);
    auto go = [&](auto kernel) -> int {
        const uint32_t smem = p.dbg == 4 ? 200 * 1024 : QSmem::kDynamic;   // dbg 4 (experiment): one CTA per SM
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return GDN_ERR_CUDA;
        kernel<<<grid, 256, smem, stream>>>(tq, tk, tw, tp, tt2, p, ws, NT, items);
        count_launch();
        return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
    };
    return p.gate_f32 ? go(gdn_prepare_pair_kernel<true>) : go(gdn_prepare_pair_kernel<false>);
}

}  // namespace gdn
