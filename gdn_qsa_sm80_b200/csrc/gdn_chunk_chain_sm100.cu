// "chain": the serial part of gdn_chunk - the inter-chunk state recurrence and the outputs -
// reading what "prepare" left in the workspace.  One CTA per (batch, value head, NV-column slice
// of Dv); the Dv slices of a head never mix in the recurrence, so the split is exact.
//
// Per chunk t, with S the 128 x NV fp32 state slice (thread dk owns row dk in registers) and the
// notation of the reference's torch loop (gdn_qsa_sm80/reference/gdn_chunk_ref.py:90-94):
//   D3  [Q_t ; W_t] S          -> Q S (TMEM lanes 0-63), W S (lanes 64-127)
//       v_new = U_t - W S ;  v~ = exp(gamma_C - gamma_i) v_new                       (ref :91)
//   D5  K_t^T v~               -> S <- exp(gamma_C) S + K^T v~                         (ref :94)
//   D4  P_t v_new              -> O = scale exp(gamma_i) (Q S) + P v_new               (ref :92-93)
// The reference does the same work in gdn_recurrence_kernel phases P1/P3/P4/P6
// (csrc/gdn_chunk/gdn_kernel.cu:1027-1224) with mma.sync and a bf16 state; here the products are
// tcgen05 UMMAs with fp32 accumulators in TMEM and the state stays fp32.
//
// Roles: G = NV / 32 groups of four epilogue warps (warps 0 .. 4G-1; warp w works on TMEM lane quadrant w % 4 and on
// the 32 columns [32 (w / 4), +32) of the slice, so an epilogue costs the same whatever NV is); warp 2's first lane
// issues the UMMAs of the critical path (D3, D5); warp 4G is the TMA producer that keeps a ring of STAGES chunks
// (K, [Q;W], P, U slice, per-token factors) in flight; warp 4G+1's first lane issues D4, which nothing on the
// critical path waits for.  192 threads at NV = 32, 320 at NV = 64.  Only D3 -> v_new -> D5 ->
// state sits on the critical path: the output epilogue of chunk t-1 runs on warps 0-1 while
// warps 2-3 turn W S into v_new for chunk t, and accumulators are double-buffered so the next D3
// never waits for an output epilogue.  (A UMMA with N <= 64 occupies the tensor pipe for about 40
// cycles whatever N is, and issuing from several warps does not raise that rate, so what counts on
// the critical path is the number of UMMA instructions: 8 for D3, 4 for D5.)
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

template <int NV, int STAGES>
struct CSmem {
    static constexpr uint32_t kRowBytes = NV * 2;
    static constexpr uint32_t kSwz = NV == 64 ? SWZ_128B : SWZ_64B;
    // one stage
    static constexpr uint32_t KT = 0;                       // K: 2 dk-halves x 64 rows x 128 B
    static constexpr uint32_t QW = KT + 16384;              // [Q;W]: 2 k-halves x 128 rows x 128 B
    static constexpr uint32_t PB = QW + 32768;              // P: 64 rows x 128 B; the 64 rows after it are don't-care
    static constexpr uint32_t UB = PB + 8192;               // U slice bf16: 64 rows x kRowBytes
    static constexpr uint32_t VEC = UB + 64 * NV * 2;       // 256 floats
    static constexpr uint32_t kStage = VEC + 1024;
    static constexpr uint32_t kStageTx = 16384 + 16384 + 16384 + 8192 + 64 * NV * 2 + 1024;
    // after the ring
    static constexpr uint32_t VN = STAGES * kStage;         // v_new  bf16 64 rows x kRowBytes
    static constexpr uint32_t VS = VN + 64 * kRowBytes;     // v~
    static constexpr uint32_t SB = VS + 64 * kRowBytes;     // bf16 copy of the state, 128 rows x kRowBytes
    static constexpr uint32_t kBytes = SB + 128 * kRowBytes;
    static constexpr uint32_t kDynamic = kBytes + 1024;
    static_assert(kStage % 1024 == 0 && VN % 1024 == 0, "tiles must stay 1024-byte aligned");
    // the 64 don't-care rows of the P operand (8 KB after PB) run into U, the factors and whatever follows the stage:
    // always inside the allocation, because VN/VS/SB follow the last stage
    static_assert(UB - PB == 8192, "P tile is 8 KB");
};

constexpr int kDevTimeoutChainFull = 0x201;
constexpr int kDevTimeoutChainEmpty = 0x202;
constexpr int kDevTimeoutChainD3 = 0x203;
constexpr int kDevTimeoutChainKV = 0x204;
constexpr int kDevTimeoutChainPV = 0x205;
constexpr int kDevTimeoutChainVN = 0x206;

// 32 fp32 values -> bf16 -> columns [32 cg, 32 cg + 32) of row `row` of a swizzled tile with NV columns
template <int NV>
__device__ __forceinline__ void store_row_bf16(uint8_t* tile, uint32_t row, const float* x, int cg) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint4 pk;
        pk.x = pack_bf16x2(x[8 * ch + 0], x[8 * ch + 1]);
        pk.y = pack_bf16x2(x[8 * ch + 2], x[8 * ch + 3]);
        pk.z = pack_bf16x2(x[8 * ch + 4], x[8 * ch + 5]);
        pk.w = pack_bf16x2(x[8 * ch + 6], x[8 * ch + 7]);
        *reinterpret_cast<uint4*>(tile + swz_chunk_offset<NV * 2>(row, cg * 4 + ch)) = pk;
    }
}

template <int NV, int STAGES>
__global__ void __launch_bounds__((NV / 32 * 4 + 2) * 32, 1)
gdn_chain_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_p,
                 const __grid_constant__ CUtensorMap tm_u, Problem p, Workspace ws) {
    using L = CSmem<NV, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_d3, bar_kv;
    __shared__ __align__(8) uint64_t bar_pv[2];
    __shared__ __align__(8) uint64_t bar_vn;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
    const int hq = hv / (p.Hv / p.Hq);
    const int dv0 = split * NV;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const size_t tile0 = (static_cast<size_t>(b) * p.Hv + hv) * NT;

    constexpr uint32_t kTmemCols = NV == 32 ? 256 : 512;
    constexpr uint32_t kColD3 = 0;            // 2 x NV: Q S | W S, double-buffered
    constexpr uint32_t kColPV = 2 * NV;       // 2 x NV: P v_new, double-buffered
    constexpr uint32_t kColKV = 4 * NV;       // NV: K^T v~

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 2);   // D5 seen complete by a chain thread + D4 complete (commit)
        }
        mbar_init(&bar_vn, 1);
        mbar_init(&bar_d3, 1);
        mbar_init(&bar_kv, 1);
        mbar_init(&bar_pv[0], 1);
        mbar_init(&bar_pv[1], 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    volatile int* abortp = &abort_flag;

    constexpr int kGroups = NV / 32;               // epilogue warp groups, 32 columns each
    constexpr int kEpiWarps = 4 * kGroups;
    if (warp == kEpiWarps) {
        // ------------------------------- TMA producer -----------------------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_p); tma_prefetch_desc(&tm_u);
            for (int t = 0; t < NT; ++t) {
                const int s = t % STAGES;
                if (t >= STAGES &&
                    !mbar_wait_abortable(&bar_empty[s], ((t / STAGES) - 1) & 1, p.status, kDevTimeoutChainEmpty, abortp))
                    break;
                uint8_t* st = sm + s * L::kStage;
                const int s0 = t * kChunk;
                const int row0 = static_cast<int>((tile0 + t) * kChunk);
                mbar_arrive_expect_tx(&bar_full[s], L::kStageTx);
                tma_load_4d(st + L::KT + 0, &tm_k, &bar_full[s], 0, hq, s0, b);
                tma_load_4d(st + L::KT + 8192, &tm_k, &bar_full[s], 64, hq, s0, b);
                tma_load_4d(st + L::QW + 0, &tm_q, &bar_full[s], 0, hq, s0, b);
                tma_load_4d(st + L::QW + 16384, &tm_q, &bar_full[s], 64, hq, s0, b);
                tma_load_2d(st + L::QW + 8192, &tm_w, &bar_full[s], 0, row0);
                tma_load_2d(st + L::QW + 24576, &tm_w, &bar_full[s], 64, row0);
                tma_load_2d(st + L::PB, &tm_p, &bar_full[s], 0, row0);
                tma_load_2d(st + L::UB, &tm_u, &bar_full[s], dv0, row0);
                bulk_load_1d(st + L::VEC, ws.vec + (tile0 + t) * 256, 1024, &bar_full[s]);
            }
        }
    } else if (warp == kEpiWarps + 1) {
        // ------------------------------- off-critical-path UMMA issuer: D4 = P v_new -----------------
        if (lane == 0) {
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
            for (int t = 0; t < NT; ++t) {
                const int s = t % STAGES;
                if (!mbar_wait_abortable(&bar_vn, t & 1, p.status, kDevTimeoutChainVN, abortp)) break;
                tc_fence_after_sync();
                const uint32_t sb = sm_u32 + s * L::kStage;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t ad = umma_smem_desc(sb + L::PB + ks * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = umma_smem_desc(sm_u32 + L::VN + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, L::kSwz);
                    umma_bf16_ss(tmem + kColPV + (t & 1) * NV, ad, bd, idesc_pv, ks > 0);
                }
                umma_commit(&bar_pv[t & 1]);
                umma_commit(&bar_empty[s]);    // second arrival: the P tile of this stage has been consumed
            }
        }
    } else {
        // ------------------------------- chain warps ---------------------------------------------------
        const int quad = warp & 3, cg = warp >> 2;     // TMEM lane quadrant; column group of the slice
        const int row = quad * 32 + lane;              // state row (dk) this thread owns: 0..127
        const uint32_t lane_base = static_cast<uint32_t>(quad) * 32u;
        const uint32_t col0 = static_cast<uint32_t>(cg) * 32u;
        const bool issuer = (tid == 64);               // group 0, quadrant 2
        const int i = row & 63;           // token row handled in the v_new / output epilogues
        float st[32];
        const size_t st_off = ((static_cast<size_t>(b) * p.Hv + hv) * kD + row) * kD + dv0 + col0;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float4 x = p.h0 ? *reinterpret_cast<const float4*>(p.h0 + st_off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            st[c] = x.x; st[c + 1] = x.y; st[c + 2] = x.z; st[c + 3] = x.w;
        }
        store_row_bf16<NV>(sm + L::SB, row, st, cg);
        fence_proxy_async_smem();

        // per-token factors of the current chunk, read from the stage before its D3 is issued
        float f_tok = 0.f, f_tok_prev = 0.f, dC = 0.f;
        auto load_factors = [&](int t) {
            const float* vec = reinterpret_cast<const float*>(sm + (t % STAGES) * L::kStage + L::VEC);
            f_tok_prev = f_tok;
            f_tok = (quad < 2) ? vec[kChunk + i] : vec[i];     // quadrants 0-1: scale e^gamma_i ; 2-3: e^{gamma_C-gamma_i}
            dC = vec[2 * kChunk];
        };
        const uint64_t sb_desc0 = umma_smem_desc(sm_u32 + L::SB, 16384, 8 * L::kRowBytes, L::kSwz);
        const uint64_t vs_desc0 = umma_smem_desc(sm_u32 + L::VS, 16384, 8 * L::kRowBytes, L::kSwz);
        auto issue_d3 = [&](int t) {
            const uint32_t sb = sm_u32 + (t % STAGES) * L::kStage;
            constexpr uint32_t idesc = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
            // descriptors differ only in the start-address field (bytes >> 4 in the low bits)
            const uint64_t a0 = umma_smem_desc(sb + L::QW, 16, 1024, SWZ_128B);
            const uint32_t d = tmem + kColD3 + (t & 1) * NV;
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_bf16_ss(d, a0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), sb_desc0 + ((ks * 16 * L::kRowBytes) >> 4),
                             idesc, ks > 0);
            umma_commit(&bar_d3);
        };
        auto out_epilogue = [&](int t, float qf) {   // rows of chunk t: O = qf * (Q S) + P v_new
            const int s = t * kChunk + i;
            uint32_t a[32], c2[32];
            {
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColD3 + (t & 1) * NV + col0), a);
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColPV + (t & 1) * NV + col0), c2);
                tmem_ld_wait();
                if (s < p.S) {
                    __nv_bfloat16* dst = p.out + ((static_cast<size_t>(b) * p.S + s) * p.Hv + hv) * kD + dv0 + col0;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(fmaf(qf, __uint_as_float(a[8 * ch + 0]), __uint_as_float(c2[8 * ch + 0])),
                                           fmaf(qf, __uint_as_float(a[8 * ch + 1]), __uint_as_float(c2[8 * ch + 1])));
                        pk.y = pack_bf16x2(fmaf(qf, __uint_as_float(a[8 * ch + 2]), __uint_as_float(c2[8 * ch + 2])),
                                           fmaf(qf, __uint_as_float(a[8 * ch + 3]), __uint_as_float(c2[8 * ch + 3])));
                        pk.z = pack_bf16x2(fmaf(qf, __uint_as_float(a[8 * ch + 4]), __uint_as_float(c2[8 * ch + 4])),
                                           fmaf(qf, __uint_as_float(a[8 * ch + 5]), __uint_as_float(c2[8 * ch + 5])));
                        pk.w = pack_bf16x2(fmaf(qf, __uint_as_float(a[8 * ch + 6]), __uint_as_float(c2[8 * ch + 6])),
                                           fmaf(qf, __uint_as_float(a[8 * ch + 7]), __uint_as_float(c2[8 * ch + 7])));
                        *reinterpret_cast<uint4*>(dst + 8 * ch) = pk;
                    }
                }
            }
        };

        // optional cycle accounting by the UMMA-issuing thread of CTA (0,0,0), summed over chunks
        const bool prof_on = GDN_DIAG(p.prof != nullptr && issuer && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
        long long prof_acc[6] = {0, 0, 0, 0, 0, 0};
        long long prof_t = prof_on ? clock64() : 0;
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_acc[n] += now_ - prof_t;                  \
        prof_t = now_;                                 \
    }

        bool ok = mbar_wait_abortable(&bar_full[0], 0, p.status, kDevTimeoutChainFull, abortp);
        if (ok) load_factors(0);
        tc_fence_before_sync();
        named_bar_sync(2, 128 * kGroups);
        if (issuer && ok) issue_d3(0);

        if (prof_on) prof_t = clock64();
        for (int t = 0; t < NT; ++t) {
            const int s = t % STAGES;
            uint8_t* stg = sm + s * L::kStage;
            if (quad >= 2) {
                // ---- v_new = U - W S, and its decay-scaled copy -------------------------------------------
                float x[32], y[32];
                // U does not depend on the state: fetch it while D3 is still in flight
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const uint4 uv = *reinterpret_cast<const uint4*>(stg + L::UB + swz_chunk_offset<NV * 2>(i, cg * 4 + ch));
                    const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {     // bf16 pair -> two fp32
                        x[8 * ch + 2 * e] = __uint_as_float(uw[e] << 16);
                        x[8 * ch + 2 * e + 1] = __uint_as_float(uw[e] & 0xffff0000u);
                    }
                }
                ok = mbar_wait_abortable(&bar_d3, t & 1, p.status, kDevTimeoutChainD3, abortp) && ok;
                tc_fence_after_sync();
                GDN_PHASE(0)
                {
                    uint32_t w[32];
                    tmem_ld_x32(tmem_addr(tmem, lane_base, kColD3 + (t & 1) * NV + col0), w);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float vn = x[c] - __uint_as_float(w[c]);
                        x[c] = vn;
                        y[c] = vn * f_tok;
                    }
                }
                if (t > 0)   // D4 of the previous chunk must have finished reading v_new
                    ok = mbar_wait_abortable(&bar_pv[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, kDevTimeoutChainPV, abortp) && ok;
                store_row_bf16<NV>(sm + L::VN, i, x, cg);
                store_row_bf16<NV>(sm + L::VS, i, y, cg);
                fence_proxy_async_smem();
                tc_fence_before_sync();
                named_bar_sync(1, 64 * kGroups);
                GDN_PHASE(1)
                if (issuer && ok) {
                    constexpr uint32_t idesc_kv = umma_idesc_bf16(128, NV, MAJOR_MN, MAJOR_MN);
                    const uint64_t k0 = umma_smem_desc(sm_u32 + s * L::kStage + L::KT, 8192, 1024, SWZ_128B);
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_bf16_ss(tmem + kColKV, k0 + ((ks * 2048) >> 4), vs_desc0 + ((ks * 16 * L::kRowBytes) >> 4),
                                     idesc_kv, ks > 0);
                    umma_commit(&bar_kv);
                    mbar_arrive(&bar_vn);          // v_new is in shared memory: warp 5 may issue D4
                }
                GDN_PHASE(2)
            } else if (t > 0) {
                // ---- output rows of the previous chunk, off the critical path ---------------------------------
                ok = mbar_wait_abortable(&bar_pv[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, kDevTimeoutChainPV, abortp) && ok;
                tc_fence_after_sync();
                out_epilogue(t - 1, f_tok_prev);
            }
            // ---- state rows: S <- exp(gamma_C) S + K^T v~ ------------------------------------------------------
            ok = mbar_wait_abortable(&bar_kv, t & 1, p.status, kDevTimeoutChainKV, abortp) && ok;
            tc_fence_after_sync();
            if (tid == 0 && ok) mbar_arrive(&bar_empty[s]);   // first arrival: D3 and D5 of this stage are complete
            GDN_PHASE(3)
            {
                uint32_t r[32];
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColKV + col0), r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) st[c] = fmaf(dC, st[c], __uint_as_float(r[c]));
                store_row_bf16<NV>(sm + L::SB, row, st, cg);
            }
            fence_proxy_async_smem();
            if (t + 1 < NT) {
                ok = mbar_wait_abortable(&bar_full[(t + 1) % STAGES], ((t + 1) / STAGES) & 1, p.status, kDevTimeoutChainFull, abortp) && ok;
                if (ok) load_factors(t + 1);
                else f_tok_prev = f_tok;
            } else {
                f_tok_prev = f_tok;
            }
            tc_fence_before_sync();
            named_bar_sync(2, 128 * kGroups);
            GDN_PHASE(4)
            if (issuer && ok && t + 1 < NT) issue_d3(t + 1);
            GDN_PHASE(5)
        }
#undef GDN_PHASE
        if (prof_on)
            for (int n = 0; n < 6; ++n) p.prof[8 + n] = prof_acc[n];
        if (quad < 2 && NT > 0) {   // output rows of the last chunk
            ok = mbar_wait_abortable(&bar_pv[(NT - 1) & 1], ((NT - 1) >> 1) & 1, p.status, kDevTimeoutChainPV, abortp) && ok;
            tc_fence_after_sync();
            out_epilogue(NT - 1, f_tok_prev);
        }
        if (ok && p.hT) {
#pragma unroll
            for (int c = 0; c < 32; c += 4)
                *reinterpret_cast<float4*>(p.hT + st_off + c) = make_float4(st[c], st[c + 1], st[c + 2], st[c + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abortp) {   // give copies that may still be in flight time to land before the CTA's memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 100000ull) {}
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

template <int NV, int STAGES>
int launch_chain_nv(const Problem& p, const Workspace& ws, cudaStream_t stream) {
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tu;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, nullptr, &tu, NV)) return GDN_ERR_DRIVER;
    using L = CSmem<NV, STAGES>;
    auto kernel = gdn_chain_kernel<NV, STAGES>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) != cudaSuccess)
        return GDN_ERR_CUDA;
    const dim3 grid(kD / NV, p.Hv, p.B), block((NV / 32 * 4 + 2) * 32);
    kernel<<<grid, block, L::kDynamic, stream>>>(tq, tk, tw, tp, tu, p, ws);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
}

}  // namespace

int launch_chain(const Problem& p, const Workspace& ws, int nv, cudaStream_t stream) {
    if (nv == 32) return launch_chain_nv<32, 3>(p, ws, stream);
    if (nv == 64) return launch_chain_nv<64, 2>(p, ws, stream);
    return GDN_ERR_BAD_ARGUMENT;
}

}  // namespace gdn
