// Device-side roles of the "transposed" chain: the serial state recurrence and the outputs of one whole value
// head per CTA, with every state-dependent operand held in tensor memory instead of shared memory.
//
// All products are formed transposed, so that the quantities the recurrence rewrites every chunk (the bf16 copy of
// the state, v_new and its decay-scaled copy) are A operands, which tcgen05.mma may read from tensor memory, and
// the B operands are tiles exactly as TMA loaded them.  With S^T the [dv x dk] state (thread = one dv row, fp32
// registers), per 64-token chunk (notation of gdn_qsa_sm80/reference/gdn_chunk_ref.py:90-94):
//   E0   ACC_V   = V^T T''^T            (A = the raw V tile read MN-major, B = T'' = T diag(beta) as prepared) = U^T
//   E1   ACC_V  -= S^T W^T              (A = bf16 S^T in TMEM, negated; B = the W tile as loaded) -> v_new^T   (ref :91)
//   E1'  ACC_QS  = S^T Q^T              (same A, not negated; B = the Q tile; nothing on the critical path waits for it)
//   E2   ACC_S  = v~^T K                (A = bf16 v~^T in TMEM, B = K as loaded, MN-major)
//        S^T <- exp(gamma_C) S^T + ACC_S                                                                   (ref :94)
//   E3   ACC_PV = v_new^T P^T           (A = bf16 v_new^T in TMEM, B = P as loaded)
//        O^T = scale exp(gamma_i) (S^T Q^T) + ACC_PV  (column factors)                                   (ref :92-93)
// 28 UMMA instructions per chunk, of which the 8 of E1 and the 4 of E2 are on the critical path.  What the critical
// warps hand over is ordered by who waits for it: the decay-scaled v~^T first (E2), the plain v_new^T behind a barrier
// of its own (E3, an output product), each half of the state's bf16 copy as soon as that half is updated.
// Nothing the recurrence produces is written to shared memory, no generic-to-async proxy fence sits on the critical
// path, and one CTA carries all 128 value columns of a head, so every workspace tile is read once per head.
// The reference keeps its state in registers for the same reason (csrc/gdn_chunk/gdn_kernel.cu:1581-1606).
//
// Roles (14 warps): warps 0-7 "critical" (warp w: TMEM lane quadrant w % 4, column half w / 4): v_new and state
// epilogues; warps 8-11 output epilogue (one per lane quadrant); warp 12 lane 0 TMA producer; warp 13 lane 0 issues
// every UMMA.  Every wait is bounded and abortable.
#pragma once

#include <cuda.h>

#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace chain_t {

constexpr int kStages = 2;
constexpr int kVecSlots = 4;
constexpr int kThreads = 14 * 32;
// one stage of the ring (every tile 1024-byte aligned; two 64-column halves of 64 rows x 128 B each)
// [W;Q]: two dk-halves of 128 rows x 128 B, rows 0-63 W, rows 64-127 Q
constexpr uint32_t KT = 0, WQ = 16384, VT = 49152, PT = 65536, T2 = 73728, kStage = 81920;
constexpr uint32_t kStageTx = kStage + 1024;              // the stage plus its slot of per-token factors
constexpr uint32_t VEC = kStages * kStage;                // kVecSlots x 256 floats
constexpr uint32_t kBytes = VEC + kVecSlots * 1024;
static_assert(kStage % 1024 == 0, "tiles must stay 1024-byte aligned");

// tensor-memory columns (32-bit) of one chain CTA
constexpr uint32_t ACC_S = 0;      // 128: v~^T K
constexpr uint32_t ACC_VQ = 128;   // 128: v_new^T (64) | S^T Q^T (64)
constexpr uint32_t ACC_PV = 256;   // 64: v_new^T P^T
constexpr uint32_t A_S = 320;      // 64: bf16 S^T (128 dk)
constexpr uint32_t A_VN = 384;     // 32: bf16 v_new^T (64 tokens)
constexpr uint32_t A_VS = 416;     // 32: bf16 v~^T
constexpr uint32_t kTmemCols = 512;

constexpr int kTimeoutFull = 0x401, kTimeoutEmpty = 0x402, kTimeoutV = 0x403, kTimeoutVN = 0x404, kTimeoutS = 0x405,
              kTimeoutState = 0x406, kTimeoutO = 0x407, kTimeoutQsDone = 0x408, kTimeoutFlag = 0x409, kTimeoutPvDone = 0x40a, kTimeoutVNP = 0x40b;

// The CTA's barriers: kNumBars consecutive 8-byte mbarriers in shared memory, addressed by their shared-window address.
enum : uint32_t { B_FULL = 0, B_EMPTY = kStages, B_V = 2 * kStages, B_Q, B_VN, B_VNP, B_S, B_STATE, B_O, B_QSDONE, B_PVDONE, kNumBars };
struct Bars {
    uint32_t base;                     // shared-window address of barrier 0
    __device__ __forceinline__ uint32_t operator()(uint32_t i) const { return base + 8u * i; }
};

__device__ __forceinline__ void init_bars(uint64_t* bars) {   // one thread
    for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars[B_FULL + s], 1);
        mbar_init(&bars[B_EMPTY + s], 5);   // the commit behind the chunk's last UMMA + the four output warps (see there)
    }
    mbar_init(&bars[B_V], 1);
    mbar_init(&bars[B_Q], 1);
    mbar_init(&bars[B_VN], 8);
    mbar_init(&bars[B_VNP], 8);
    mbar_init(&bars[B_S], 1);
    mbar_init(&bars[B_STATE], 8);
    mbar_init(&bars[B_O], 1);
    mbar_init(&bars[B_QSDONE], 4);
    mbar_init(&bars[B_PVDONE], 4);
}

__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait for a tile flag written by another CTA of the same launch.
__device__ __forceinline__ bool wait_tile_flag(const int* flag, int* status, volatile int* abort_flag) {
    if (*abort_flag) return false;
    if (ld_acquire_gpu_s32(flag) != 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (ld_acquire_gpu_s32(flag) != 0) return true;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            atomicCAS(status, 0, kTimeoutFlag);
            *abort_flag = 1;
            return false;
        }
    }
}

// The stretch of chunks [t0, t1) of one (batch, value head) a CTA runs, the state it starts from (a 128 x 128 fp32
// matrix, [dk][dv]; null = zeros) and where the state it ends with goes (null = nowhere).  Outputs are stored from
// chunk t_store on: chunks [t0, t_store) only bring the state up to date (the warm-up of a segment).
struct Span {
    int t0, t1, t_store;
    const float* s_in;
    float* s_out;
};

// `sm`: the CTA's 1024-byte aligned dynamic shared memory (chain region first); `tmem`: base of kTmemCols columns.
// tm_v: the value tensor (64 x 64 boxes); tm_t2: T'' [tiles * 64][64] (64 x 64 boxes).  flags: per-tile "prepared"
// flags when WAIT_FLAGS.
template <bool WAIT_FLAGS>
__device__ __forceinline__ void roles(uint8_t* sm, uint32_t sm_u32, uint32_t tmem, const Bars& cb, const CUtensorMap* tm_q,
                                      const CUtensorMap* tm_k, const CUtensorMap* tm_v, const CUtensorMap* tm_w,
                                      const CUtensorMap* tm_p, const CUtensorMap* tm_t2, const Problem& p, const Workspace& ws, const int* flags,
                                      volatile int* abortp, const Span& sp, int hv, int b, bool prof_cta) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = hv / (p.Hv / p.Hq);
    const int NT = (p.S + kChunk - 1) / kChunk;
    const int t0 = sp.t0, t1 = sp.t1;
    const size_t tile0 = (static_cast<size_t>(b) * p.Hv + hv) * NT;
    // experiment: absolute time stamps of the events of chunk 50 of one CTA (prof buffer of >= 128 slots)
#ifdef GDN_DIAGNOSTICS
    const bool tl_on = p.prof != nullptr && prof_cta && p.dbg >= 100 && lane == 0;
#define GDN_TL(idx) if (tl_on && t == t0 + 20) p.prof[idx] = clock64();
#else
#define GDN_TL(idx)
#endif

    if (warp == 12) {
        if (lane != 0) return;
        // ------------------------------- TMA producer ----------------------------------------------------------
        for (int t = t0; t < t1; ++t) {
            const int n = t - t0, s = n % kStages;
            if (WAIT_FLAGS) {
                if (!wait_tile_flag(flags + tile0 + t, p.status, abortp)) break;   // chunk t has been prepared
                asm volatile("fence.proxy.async;" ::: "memory");   // order the TMA reads after the acquire
            }
            if (n >= kStages && !mbar_wait_abortable_a(cb(B_EMPTY + s), ((n / kStages) - 1) & 1, p.status, kTimeoutEmpty, abortp))
                break;
            const uint32_t st = sm_u32 + s * kStage, fb = cb(B_FULL + s);
            const int s0 = t * kChunk;
            const int row0 = static_cast<int>((tile0 + t) * kChunk);
            mbar_arrive_expect_tx_a(fb, kStageTx);
            tma_load_2d_a(st + WQ, tm_w, fb, 0, row0);
            tma_load_2d_a(st + WQ + 16384, tm_w, fb, 64, row0);
            tma_load_2d_a(st + T2, tm_t2, fb, 0, row0);
            tma_load_4d_a(st + VT, tm_v, fb, 0, hv, s0, b);
            tma_load_4d_a(st + VT + 8192, tm_v, fb, 64, hv, s0, b);
            bulk_load_1d_a(sm_u32 + VEC + (n % kVecSlots) * 1024, ws.vec + (tile0 + t) * 256, 1024, fb);
            tma_load_4d_a(st + KT, tm_k, fb, 0, hq, s0, b);
            tma_load_4d_a(st + KT + 8192, tm_k, fb, 64, hq, s0, b);
            tma_load_2d_a(st + PT, tm_p, fb, 0, row0);
            tma_load_4d_a(st + WQ + 8192, tm_q, fb, 0, hq, s0, b);
            tma_load_4d_a(st + WQ + 24576, tm_q, fb, 64, hq, s0, b);
        }
        return;
    }
    if (warp == 13) {
        if (lane != 0) return;
        // ------------------------------- UMMA issuer --------------------------------------------------------------
        constexpr uint32_t idesc_e0 = umma_idesc_bf16(128, 64, MAJOR_MN, MAJOR_K);
        constexpr uint32_t idesc_e1 = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K, 1);    // negated A
        constexpr uint32_t idesc_e2 = umma_idesc_bf16(128, 128, MAJOR_K, MAJOR_MN);
        constexpr uint32_t idesc_e3 = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K);
        const bool prof = GDN_DIAG(p.prof != nullptr && prof_cta);
        long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long ct = prof ? clock64() : 0;
#define GDN_TPHASE(n)                                  \
    if (prof) {                                        \
        const long long now_ = clock64();              \
        acc[n] += now_ - ct;                           \
        ct = now_;                                     \
    }
        for (int t = t0; t < t1; ++t) {
            const int n = t - t0, s = n % kStages;
            const uint32_t sb = sm_u32 + s * kStage;
            if (!mbar_wait_abortable_a(cb(B_FULL + s), (n / kStages) & 1, p.status, kTimeoutFull, abortp)) break;
            GDN_TL(0)
            // the output warps have taken chunk t-1's S^T Q^T out of ACC_VQ (its v_new part was read before bar vn)
            if (n > 0 && !mbar_wait_abortable_a(cb(B_QSDONE), (n - 1) & 1, p.status, kTimeoutQsDone, abortp)) break;
            tc_fence_after_sync();
            GDN_TPHASE(0)
            GDN_TL(1)
            {   // E0: ACC_V = V^T T''^T
                const uint64_t a0 = umma_smem_desc(sb + VT, 8192, 1024, SWZ_128B);
                const uint64_t b0 = umma_smem_desc(sb + T2, 16, 1024, SWZ_128B);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_bf16_ss(tmem + ACC_VQ, a0 + ((ks * 2048) >> 4), b0 + ((ks * 32) >> 4), idesc_e0, ks > 0);
            }
            GDN_TPHASE(1)
            GDN_TL(2)
            if (!mbar_wait_abortable_a(cb(B_STATE), n & 1, p.status, kTimeoutState, abortp)) break;
            tc_fence_after_sync();
            GDN_TPHASE(2)
            GDN_TL(3)
            {   // E1: ACC_V -= S^T W^T (the critical one), then E1': ACC_QS = S^T Q^T
                const uint64_t w0 = umma_smem_desc(sb + WQ, 16, 1024, SWZ_128B);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_bf16_ts(tmem + ACC_VQ, tmem + A_S + ks * 8, w0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), idesc_e1, 1);
                umma_commit_a(cb(B_V));
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_bf16_ts(tmem + ACC_VQ + 64, tmem + A_S + ks * 8, w0 + (((ks >> 2) * 16384 + 8192 + (ks & 3) * 32) >> 4), idesc_e3, ks > 0);
                umma_commit_a(cb(B_Q));
            }
            GDN_TPHASE(3)
            GDN_TL(4)
            if (!mbar_wait_abortable_a(cb(B_VN), n & 1, p.status, kTimeoutVN, abortp)) break;
            tc_fence_after_sync();
            GDN_TPHASE(4)
            GDN_TL(5)
            {   // E2: ACC_S = v~^T K
                const uint64_t k0 = umma_smem_desc(sb + KT, 8192, 1024, SWZ_128B);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_bf16_ts(tmem + ACC_S, tmem + A_VS + ks * 8, k0 + ((ks * 2048) >> 4), idesc_e2, ks > 0);
                umma_commit_a(cb(B_S));
            }
            GDN_TPHASE(5)
            GDN_TL(6)
            if (n > 0 && !mbar_wait_abortable_a(cb(B_PVDONE), (n - 1) & 1, p.status, kTimeoutPvDone, abortp)) break;
            if (!mbar_wait_abortable_a(cb(B_VNP), n & 1, p.status, kTimeoutVNP, abortp)) break;   // the plain bf16 v_new^T is in place
            tc_fence_after_sync();
            GDN_TPHASE(6)
            GDN_TL(7)
            {   // E3: ACC_PV = v_new^T P^T
                const uint64_t p0 = umma_smem_desc(sb + PT, 16, 1024, SWZ_128B);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_bf16_ts(tmem + ACC_PV, tmem + A_VN + ks * 8, p0 + ((ks * 32) >> 4), idesc_e3, ks > 0);
                umma_commit_a(cb(B_O));
                umma_commit_a(cb(B_EMPTY + s));
            }
            GDN_TPHASE(7)
            GDN_TL(8)
        }
#undef GDN_TPHASE
        if (prof && p.dbg < 100) {
            for (int n = 0; n < 8; ++n) p.prof[8 + n] = acc[n];
        }
        return;
    }

    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad) * 32u;
    const int dv = quad * 32 + lane;                      // the value column (= TMEM lane) this thread owns

    if (warp >= 8) {
        // ------------------------------- output epilogue (warps 8-11) ----------------------------------------------
        const bool oprof = GDN_DIAG(p.prof != nullptr && prof_cta && tid == 256);
        long long oacc[3] = {0, 0, 0};
        long long oct = oprof ? clock64() : 0;
#define GDN_OPHASE(n)                                  \
    if (oprof) {                                       \
        const long long now_ = clock64();              \
        oacc[n] += now_ - oct;                         \
        oct = now_;                                    \
    }
        for (int t = t0; t < t1; ++t) {
            const int n = t - t0, s = n % kStages;
            // The stage's factors are read with ordinary loads, so this warp must see the stage's barrier complete
            // itself.  Nothing else orders this warp against the ring, so it also holds the stage until it has looked:
            // otherwise the barrier could complete a second time (chunk t + 2) before the warp tests the parity of chunk t.
            bool ok = mbar_wait_abortable_a(cb(B_FULL + s), (n / kStages) & 1, p.status, kTimeoutFull, abortp);
            __syncwarp();
            if (lane == 0) mbar_arrive_a(cb(B_EMPTY + s));
            ok = mbar_wait_abortable_a(cb(B_Q), n & 1, p.status, kTimeoutV, abortp) && ok;
            if (!ok) break;
            tc_fence_after_sync();
            GDN_OPHASE(0)
            GDN_TL(50 + warp - 8)
            const float* qf = reinterpret_cast<const float*>(sm + VEC + (n % kVecSlots) * 1024) + kChunk;   // scale e^gamma_i
            uint32_t o[64];                               // (S^T Q^T)[dv][j], taken as soon as it exists
            {
                uint32_t (&o0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&o[0]);
                uint32_t (&o1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&o[32]);
                tmem_ld_x32(tmem_addr(tmem, lane_base, ACC_VQ + 64), o0);
                tmem_ld_x32(tmem_addr(tmem, lane_base, ACC_VQ + 96), o1);
                tmem_ld_wait();
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(cb(B_QSDONE));
            GDN_TL(54 + warp - 8)
            ok = mbar_wait_abortable_a(cb(B_O), n & 1, p.status, kTimeoutO, abortp);
            if (!ok) break;
            tc_fence_after_sync();
            GDN_OPHASE(1)
            GDN_TL(58 + warp - 8)
            __nv_bfloat16* dst = p.out + ((static_cast<size_t>(b) * p.S + t * kChunk) * p.Hv + hv) * kD + dv;
            const size_t row_stride = static_cast<size_t>(p.Hv) * kD;
            const int valid = t >= sp.t_store ? min(kChunk, p.S - t * kChunk) : 0;   // warm-up chunks store nothing
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                uint32_t c[32];
                tmem_ld_x32(tmem_addr(tmem, lane_base, ACC_PV + 32 * h2), c);
                tmem_ld_wait();
                if (h2 == 1) {   // the accumulator is in registers: the next chunk may overwrite it
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_a(cb(B_PVDONE));
                    GDN_TL(62 + warp - 8)
                }
                // O^T[dv][j] = scale e^gamma_j (S^T Q^T) + v_new^T P^T: a warp stores 64 contiguous bytes of row j
                __nv_bfloat16* drow = dst + static_cast<size_t>(32 * h2) * row_stride;
                if (valid == kChunk) {          // whole chunk (the common case): no per-row test
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 f = *reinterpret_cast<const float4*>(qf + 32 * h2 + j);
                        const float fq[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            *drow = __float2bfloat16(fmaf(fq[u], __uint_as_float(o[32 * h2 + j + u]), __uint_as_float(c[j + u])));
                            drow += row_stride;
                        }
                    }
                } else if (valid > 32 * h2) {   // ragged tail
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (32 * h2 + j < valid)
                            *drow = __float2bfloat16(fmaf(qf[32 * h2 + j], __uint_as_float(o[32 * h2 + j]), __uint_as_float(c[j])));
                        drow += row_stride;
                    }
                }
            }
            GDN_OPHASE(2)
            GDN_TL(66 + warp - 8)
        }
#undef GDN_OPHASE
        if (oprof && p.dbg < 100)
            for (int n = 0; n < 3; ++n) p.prof[5 + n] = oacc[n];
        return;
    }

    // ------------------------------- critical warps 0-7: v_new and state epilogues -----------------------------------
    const int hf = warp >> 2;                             // which half of the columns of each accumulator
    float st[64];                                         // S^T[dv][64 hf .. 64 hf + 63]
    const size_t st_off = static_cast<size_t>(64 * hf) * kD + dv;
#pragma unroll
    for (int c = 0; c < 64; ++c) st[c] = sp.s_in ? sp.s_in[st_off + static_cast<size_t>(c) * kD] : 0.f;
    auto publish_state = [&]() {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            uint32_t pk[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) pk[c] = pack_bf16x2(st[32 * h2 + 2 * c], st[32 * h2 + 2 * c + 1]);
            tmem_st_x16(tmem_addr(tmem, lane_base, A_S + 32 * hf + 16 * h2), pk);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_a(cb(B_STATE));
    };
    publish_state();

    // optional cycle accounting by one critical thread of one CTA, summed over chunks
    const bool cprof = GDN_DIAG(p.prof != nullptr && prof_cta && tid == 0);
    long long cacc[5] = {0, 0, 0, 0, 0};
    long long cct = cprof ? clock64() : 0;
#define GDN_CPHASE(n)                                  \
    if (cprof) {                                       \
        const long long now_ = clock64();              \
        cacc[n] += now_ - cct;                         \
        cct = now_;                                    \
    }
    bool ok = true;
    for (int t = t0; t < t1 && ok; ++t) {
        const int n = t - t0, s = n % kStages;
        ok = mbar_wait_abortable_a(cb(B_FULL + s), (n / kStages) & 1, p.status, kTimeoutFull, abortp);
        GDN_CPHASE(0)
        const float* vec = reinterpret_cast<const float*>(sm + VEC + (n % kVecSlots) * 1024);
        const float dC = ok ? vec[2 * kChunk] : 0.f;      // exp(gamma_C); read now, the slot may be reloaded later
        ok = mbar_wait_abortable_a(cb(B_V), n & 1, p.status, kTimeoutV, abortp) && ok;
        if (!ok) break;
        tc_fence_after_sync();
        GDN_CPHASE(1)
        GDN_TL(10 + warp)
        {   // v~^T, then v_new^T, of tokens [32 hf, +32) -> bf16 A operands.  E2 (the state's next term) waits for the
            // scaled copy only; the plain copy, which only the output product E3 reads, follows behind a barrier of its own.
            uint32_t a0[16], a1[16];
            tmem_ld_x16(tmem_addr(tmem, lane_base, ACC_VQ + 32 * hf), a0);
            tmem_ld_x16(tmem_addr(tmem, lane_base, ACC_VQ + 32 * hf + 16), a1);
            tmem_ld_wait();
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                uint32_t ps[8];
#pragma unroll
                for (int c = 0; c < 8; c += 2) {
                    const float4 f = *reinterpret_cast<const float4*>(vec + 32 * hf + 16 * h2 + 2 * c);   // exp(gamma_C - gamma_j)
                    const float x0 = __uint_as_float(h2 ? a1[2 * c] : a0[2 * c]), x1 = __uint_as_float(h2 ? a1[2 * c + 1] : a0[2 * c + 1]);
                    const float x2 = __uint_as_float(h2 ? a1[2 * c + 2] : a0[2 * c + 2]), x3 = __uint_as_float(h2 ? a1[2 * c + 3] : a0[2 * c + 3]);
                    ps[c] = pack_bf16x2(x0 * f.x, x1 * f.y);
                    ps[c + 1] = pack_bf16x2(x2 * f.z, x3 * f.w);
                }
                tmem_st_x8(tmem_addr(tmem, lane_base, A_VS + 16 * hf + 8 * h2), ps);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(cb(B_VN));
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                uint32_t pn[8];
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    pn[c] = pack_bf16x2(__uint_as_float(h2 ? a1[2 * c] : a0[2 * c]), __uint_as_float(h2 ? a1[2 * c + 1] : a0[2 * c + 1]));
                tmem_st_x8(tmem_addr(tmem, lane_base, A_VN + 16 * hf + 8 * h2), pn);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(cb(B_VNP));
        }
        GDN_CPHASE(2)
        GDN_TL(20 + warp)
        ok = mbar_wait_abortable_a(cb(B_S), n & 1, p.status, kTimeoutS, abortp);
        if (!ok) break;
        tc_fence_after_sync();
        GDN_CPHASE(3)
        GDN_TL(30 + warp)
        const bool more = t + 1 < t1;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {   // S^T <- exp(gamma_C) S^T + v~^T K, 32 columns at a time
            uint32_t r[32];
            tmem_ld_x32(tmem_addr(tmem, lane_base, ACC_S + 64 * hf + 32 * h2), r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) st[32 * h2 + c] = fmaf(dC, st[32 * h2 + c], __uint_as_float(r[c]));
            if (more) {                    // its bf16 copy goes out while the other half is loaded
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) pk[c] = pack_bf16x2(st[32 * h2 + 2 * c], st[32 * h2 + 2 * c + 1]);
                tmem_st_x16(tmem_addr(tmem, lane_base, A_S + 32 * hf + 16 * h2), pk);
            }
        }
        if (more) {
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(cb(B_STATE));
        }
        GDN_CPHASE(4)
        GDN_TL(40 + warp)
    }
#undef GDN_CPHASE
    if (cprof && p.dbg < 100)
        for (int n = 0; n < 5; ++n) p.prof[n] = cacc[n];
    if (ok && sp.s_out) {
#pragma unroll
        for (int c = 0; c < 64; ++c) sp.s_out[st_off + static_cast<size_t>(c) * kD] = st[c];
    }
}

#undef GDN_TL
}  // namespace chain_t
}  // namespace gdn
