// Single-launch gdn_chunk forward for problems with few independent sequences (4 * B * Hv <= number of SMs).
//
// The four 32-column CTAs of a (batch, value head) pair run the serial chain exactly as gdn_chain_kernel does,
// and share the state-independent work among themselves: CTA j prepares chunks j, j+4, j+8, ... of its head
// (the same steps as gdn_prepare_kernel, by a second warpgroup), writes W, U, P and the per-token factors to the
// workspace in global memory and publishes a per-tile flag; the TMA producer of every CTA of that head waits for
// the flag of chunk t before it loads chunk t's tiles.  Each chunk is prepared once (no redundancy across the
// column split) while the chain of earlier chunks is running, so the prepare work hides behind the chain's
// latency instead of preceding it as a separate kernel.  The workspace is consumed microseconds after it is
// produced and stays in L2.
//
// All CTAs must be resident together (one CTA per SM because of its shared memory; the host checks
// grid <= number of SMs).  Waiting is on flags written inside the same launch; every wait is bounded and a wait
// that runs out sets the status word and drains the CTA.
//
// Warps: 0-3 chain epilogues (warp 2 lane 0 issues D3/D5), 4 lane 0 TMA producer, 5 lane 0 issues D4,
// 6 lane 0 stores and publishes the prepared tiles, 7 idle, 8-11 prepare group (warp w of it owns TMEM lane quadrant w % 4, like the chain warps).
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "gdn_prep_device.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

constexpr int NV = 32;
constexpr int STAGES = 2;
struct XSmem {
    static constexpr uint32_t kRowBytes = NV * 2;
    // chain ring, one stage:
    static constexpr uint32_t KT = 0, QW = 16384, PB = 49152, UB = 57344, VEC = 61440, kStage = 62464;
    static constexpr uint32_t kStageTx = 16384 + 16384 + 16384 + 8192 + 4096 + 1024;
    static constexpr uint32_t VN = STAGES * kStage;      // v_new bf16, 2 buffers x 64 rows x 64 B (chunk parity)
    static constexpr uint32_t VS = VN + 8192;            // decay-scaled v_new
    static constexpr uint32_t SB = VS + 4096;            // bf16 state, 128 rows x 64 B
    // prepare group:
    static constexpr uint32_t PKQ = SB + 8192;           // [K;Q] stack; V replaces Q once Q K^T is done
    static constexpr uint32_t PAS = PKQ + 32768;         // A fp32 64x68, later the bf16 [T';T''] operand
    static constexpr uint32_t PTM = PAS + 17408;         // T fp32 64x68
    static constexpr uint32_t PYT = PTM + 17408;         // merge temporaries
    static constexpr uint32_t kBytes = PYT + 5120;
    static constexpr uint32_t kDynamic = kBytes + 1024;
    static_assert(PKQ % 1024 == 0 && PAS % 1024 == 0, "operand tiles must be 1024-byte aligned");
};
constexpr uint32_t kColD3 = 0, kColPV = 64, kColKV = 128, kColPrep = 256;

constexpr int kTimeoutFull = 0x301, kTimeoutEmpty = 0x302, kTimeoutD3 = 0x303, kTimeoutKV = 0x304, kTimeoutPV = 0x305,
              kTimeoutVN = 0x306, kTimeoutFlag = 0x307, kTimeoutPrepTma = 0x308, kTimeoutPrepMma = 0x309;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded wait for a tile flag written by another CTA of this launch.
__device__ __forceinline__ bool wait_flag(const int* flag, int* status, volatile int* abort_flag) {
    if (*abort_flag) return false;
    if (ld_acquire_gpu(flag) != 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (ld_acquire_gpu(flag) != 0) return true;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            atomicCAS(status, 0, kTimeoutFlag);
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void store_row32_bf16(uint8_t* tile, uint32_t row, const float* x) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint4 pk;
        pk.x = pack_bf16x2(x[8 * ch + 0], x[8 * ch + 1]);
        pk.y = pack_bf16x2(x[8 * ch + 2], x[8 * ch + 3]);
        pk.z = pack_bf16x2(x[8 * ch + 4], x[8 * ch + 5]);
        pk.w = pack_bf16x2(x[8 * ch + 6], x[8 * ch + 7]);
        *reinterpret_cast<uint4*>(tile + swz_chunk_offset<64>(row, ch)) = pk;
    }
}

// ------------------------------------------------------------------------------------------------------
// prepare group (128 threads, ptid 0..127): tiles t = split, split+4, ... of this CTA's head
// ------------------------------------------------------------------------------------------------------
template <bool GATE_F32>
__device__ __forceinline__ void coop_prepare_role(uint8_t* sm, uint32_t sm_u32, uint32_t tmem, int ptid, const CUtensorMap* tm_q,
                                                  const CUtensorMap* tm_k, const CUtensorMap* tm_v, const Problem& p,
                                                  const Workspace& ws, int* flags, PrepScratch& ps, uint64_t* bar_ptma,
                                                  uint64_t* bar_pmma, uint64_t* bar_ready, uint64_t* bar_free, volatile int* abortp, int split, int hv, int b, int hq,
                                                  int NT, size_t tile0) {
    const PrepCtx ctx{ptid, 3};
    const int pwarp = ptid >> 5, i = ptid & 63;
    const uint32_t lane_base = static_cast<uint32_t>(pwarp) * 32u;
    const float scale = rsqrtf(static_cast<float>(kD));
    float* As = reinterpret_cast<float*>(sm + XSmem::PAS);
    float* Tm = reinterpret_cast<float*>(sm + XSmem::PTM);
    float* Yt = reinterpret_cast<float*>(sm + XSmem::PYT);
    uint8_t* kq = sm + XSmem::PKQ;
    const uint32_t kq_u32 = sm_u32 + XSmem::PKQ, ts_u32 = sm_u32 + XSmem::PAS;
    const uint32_t tm_prep = tmem + kColPrep;
    uint32_t ph_tma = 0, ph_mma = 0;

    auto issue_kq = [&](int t) {   // one thread
        mbar_arrive_expect_tx(bar_ptma, 4 * 8192);
        tma_load_4d(kq + 0, tm_k, bar_ptma, 0, hq, t * kChunk, b);
        tma_load_4d(kq + 16384, tm_k, bar_ptma, 64, hq, t * kChunk, b);
        tma_load_4d(kq + 8192, tm_q, bar_ptma, 0, hq, t * kChunk, b);
        tma_load_4d(kq + 24576, tm_q, bar_ptma, 64, hq, t * kChunk, b);
    };
    // optional cycle accounting by thread 0 of the prepare group of CTA (0,0,0), summed over its tiles
    const bool prof_on = p.prof != nullptr && ptid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long prof_t = prof_on ? clock64() : 0, prof_n = 0;
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_acc[n] += now_ - prof_t;                  \
        prof_t = now_;                                 \
    }
    int t = split;
    float gv = 0.f, bv = 0.f;
    if (t < NT) {
        if (ptid == 0) issue_kq(t);
        prep_load_gates<GATE_F32>(p.g, p.beta, static_cast<size_t>(b) * p.S + t * kChunk, hv, p.Hv,
                                  min(kChunk, p.S - t * kChunk), gv, bv, ctx);
    }
    uint32_t ph_free = 0;
    for (; t < NT; t += 4) {
        const size_t tile = tile0 + t;
        prep_gates(ps, gv, bv, scale, ws.vec + tile * 256, ctx);
        ctx.sync();
        GDN_PHASE(0)
        mbar_wait_abortable(bar_ptma, ph_tma, p.status, kTimeoutPrepTma, abortp);
        ph_tma ^= 1;
        GDN_PHASE(1)
        if (ptid == 0) {   // raw K K^T (lanes 0-63) and Q K^T (lanes 64-127)
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ad = umma_smem_desc(kq_u32 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                umma_bf16_ss(tm_prep, ad, ad, idesc, ks > 0);
            }
            umma_commit(bar_pmma);
        }
        mbar_wait_abortable(bar_pmma, ph_mma, p.status, kTimeoutPrepMma, abortp);
        ph_mma ^= 1;
        tc_fence_after_sync();
        GDN_PHASE(2)
        if (ptid == 0) {   // Q is no longer needed: V takes its place (two 64-column groups, 16 KB apart)
            mbar_arrive_expect_tx(bar_ptma, 2 * 8192);
            tma_load_4d(kq + 8192, tm_v, bar_ptma, 0, hv, t * kChunk, b);
            tma_load_4d(kq + 24576, tm_v, bar_ptma, 64, hv, t * kChunk, b);
        }
        // next tile's gates: a strided global read, issued a whole tile ahead so its latency never shows
        // (this tile's values were consumed by prep_gates above)
        if (t + 4 < NT)
            prep_load_gates<GATE_F32>(p.g, p.beta, static_cast<size_t>(b) * p.S + (t + 4) * kChunk, hv, p.Hv,
                                      min(kChunk, p.S - (t + 4) * kChunk), gv, bv, ctx);
        if (t != split) {   // the previous tile's W / U staging tiles (the A and T buffers) have been read by its TMA stores
            mbar_wait_abortable(bar_free, ph_free, p.status, kTimeoutPrepTma, abortp);
            ph_free ^= 1;
        }
        prep_zero_upper_blocks(Tm, ctx);
        {
            float ri, diag[16];
            prep_row_setup(ps, i, ri, diag);
            uint32_t r[32];
            float f[32];
            if (pwarp < 2) {
                const float bi = ps.bet[i];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, half * 32), r);
                    prep_row_factors(ps, i, half, ri, diag, f);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float4 o;
                        o.x = (half * 32 + c + 0 < i) ? bi * f[c + 0] * __uint_as_float(r[c + 0]) : 0.f;
                        o.y = (half * 32 + c + 1 < i) ? bi * f[c + 1] * __uint_as_float(r[c + 1]) : 0.f;
                        o.z = (half * 32 + c + 2 < i) ? bi * f[c + 2] * __uint_as_float(r[c + 2]) : 0.f;
                        o.w = (half * 32 + c + 3 < i) ? bi * f[c + 3] * __uint_as_float(r[c + 3]) : 0.f;
                        *reinterpret_cast<float4*>(As + i * kSolveStride + half * 32 + c) = o;
                    }
                }
            } else {
                __nv_bfloat16* prow = ws.P + tile * (kChunk * kChunk) + static_cast<size_t>(i) * kChunk;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, half * 32), r);
                    prep_row_factors(ps, i, half, ri, diag, f);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(scale * f[8 * ch + 0] * __uint_as_float(r[8 * ch + 0]), scale * f[8 * ch + 1] * __uint_as_float(r[8 * ch + 1]));
                        pk.y = pack_bf16x2(scale * f[8 * ch + 2] * __uint_as_float(r[8 * ch + 2]), scale * f[8 * ch + 3] * __uint_as_float(r[8 * ch + 3]));
                        pk.z = pack_bf16x2(scale * f[8 * ch + 4] * __uint_as_float(r[8 * ch + 4]), scale * f[8 * ch + 5] * __uint_as_float(r[8 * ch + 5]));
                        pk.w = pack_bf16x2(scale * f[8 * ch + 6] * __uint_as_float(r[8 * ch + 6]), scale * f[8 * ch + 7] * __uint_as_float(r[8 * ch + 7]));
                        *reinterpret_cast<uint4*>(prow + half * 32 + 8 * ch) = pk;
                    }
                }
            }
        }
        tc_fence_before_sync();
        ctx.sync();
        GDN_PHASE(3)
        prep_invert_unit_lower(As, Tm, Yt, ctx);
        GDN_PHASE(4)
        {   // A is dead: its buffer receives the bf16 operand [T diag(beta e^gamma) ; T diag(beta)]
            const int which = ptid >> 6;
            prep_store_scaled_T_row(Tm, which == 0 ? ps.eg : ps.bet, i, sm + XSmem::PAS, which * 64 + i);
        }
        fence_proxy_async_smem();
        ctx.sync();
        mbar_wait_abortable(bar_ptma, ph_tma, p.status, kTimeoutPrepTma, abortp);   // V has landed
        ph_tma ^= 1;
        GDN_PHASE(5)
        if (ptid == 0) {   // W = T' K (lanes 0-63, 128 columns), U = T'' V (lanes 64-127, next 128 columns)
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, 128, MAJOR_K, MAJOR_MN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(ts_u32 + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bk = umma_smem_desc(kq_u32 + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tm_prep, ad, bk, idesc, ks > 0);
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(ts_u32 + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bv_ = umma_smem_desc(kq_u32 + 8192 + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tm_prep + 128, ad, bv_, idesc, ks > 0);
            }
            umma_commit(bar_pmma);
        }
        mbar_wait_abortable(bar_pmma, ph_mma, p.status, kTimeoutPrepMma, abortp);
        ph_mma ^= 1;
        tc_fence_after_sync();
        GDN_PHASE(6)
        // the tile's K/Q/V buffer is free: next tile's K and Q
        const int tn = t + 4;
        if (tn < NT && ptid == 0) issue_kq(tn);
        // W and U (bf16) leave through swizzled staging tiles and TMA stores: W in the A buffer, U in the T buffer
        // (both dead once the last UMMA of the tile has finished)
        {
            uint32_t r[32];
            if (pwarp < 2) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, q4 * 32), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                        pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                        pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                        pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                        *reinterpret_cast<uint4*>(sm + XSmem::PAS + (q4 >> 1) * 8192 + swz_chunk_offset<128>(i, (q4 & 1) * 4 + ch)) = pk;
                    }
                }
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, 128 + q4 * 32), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                        pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                        pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                        pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                        *reinterpret_cast<uint4*>(sm + XSmem::PTM + (q4 >> 1) * 8192 + swz_chunk_offset<128>(i, (q4 & 1) * 4 + ch)) = pk;
                    }
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        ctx.sync();
        // hand the staging tiles to the publisher thread (warp 6): it stores them, frees them and raises the flag
        if (ptid == 0) mbar_arrive(bar_ready);
        GDN_PHASE(7)
        ++prof_n;
    }
#undef GDN_PHASE
    if (prof_on) {
        for (int n = 0; n < 8; ++n) p.prof[n] = prof_acc[n];
        p.prof[15] = prof_n;
    }
}

template <bool GATE_F32>
__global__ void __launch_bounds__(384, 1)
gdn_coop_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_u,
                const __grid_constant__ CUtensorMap tm_us, Problem p, Workspace ws,
                int* flags, int skip_prepare) {
    using L = XSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_d3, bar_kv, bar_vn, bar_ptma, bar_pmma, bar_ready, bar_free;
    __shared__ __align__(8) uint64_t bar_pv[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) PrepScratch ps;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
    const int hq = hv / (p.Hv / p.Hq);
    const int dv0 = split * NV;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const size_t tile0 = (static_cast<size_t>(b) * p.Hv + hv) * NT;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 2);
        }
        mbar_init(&bar_d3, 1);
        mbar_init(&bar_kv, 1);
        mbar_init(&bar_vn, 1);
        mbar_init(&bar_pv[0], 1);
        mbar_init(&bar_pv[1], 1);
        mbar_init(&bar_ptma, 1);
        mbar_init(&bar_pmma, 1);
        mbar_init(&bar_ready, 1);
        mbar_init(&bar_free, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    volatile int* abortp = &abort_flag;

    if (warp >= 8) {
        if (!skip_prepare)
        coop_prepare_role<GATE_F32>(sm, sm_u32, tmem, tid - 256, &tm_q, &tm_k, &tm_v, p, ws, flags, ps, &bar_ptma, &bar_pmma,
                                    &bar_ready, &bar_free, abortp, split, hv, b, hq, NT, tile0);
    } else if (warp >= 4) {
        if (warp == 4 && lane == 0) {
            // ------------------------------- TMA producer of the chain ------------------------------------
            for (int t = 0; t < NT; ++t) {
                const int s = t % STAGES;
                // first the flag (an L2 round trip, usually long since raised), then the stage: the flag read
                // overlaps the time the stage is still in use
                if (!wait_flag(flags + tile0 + t, p.status, abortp)) break;   // chunk t has been prepared (any CTA of this head)
                fence_proxy_async_all();     // the workspace was written by another SM; order the TMA reads after the acquire
                if (t >= STAGES &&
                    !mbar_wait_abortable(&bar_empty[s], ((t / STAGES) - 1) & 1, p.status, kTimeoutEmpty, abortp))
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
        } else if (warp == 6 && lane == 0 && !skip_prepare) {
            // ------------------------------- publisher of this CTA's prepared tiles ------------------------
            // Stores W and U from the staging tiles, frees the tiles, and raises the tile's flag once the stores
            // are complete; doing this on its own thread keeps the ~3 us write latency off the prepare group.
            uint32_t ph = 0;
            for (int t = split; t < NT; t += 4) {
                if (!mbar_wait_abortable(&bar_ready, ph, p.status, kTimeoutPrepMma, abortp)) break;
                ph ^= 1;
                const size_t tile = tile0 + t;
                const int row0 = static_cast<int>(tile * kChunk);
                tma_store_2d(&tm_w, sm + L::PAS, 0, row0);
                tma_store_2d(&tm_w, sm + L::PAS + 8192, 64, row0);
                tma_store_2d(&tm_us, sm + L::PTM, 0, row0);
                tma_store_2d(&tm_us, sm + L::PTM + 8192, 64, row0);
                tma_store_commit();
                tma_store_wait_read();
                mbar_arrive(&bar_free);
                tma_store_wait_all();
                fence_proxy_async_all();
                __threadfence();         // cumulative: also covers the group's P / factor stores ordered before bar_ready
                if (!*abortp) st_release_gpu(flags + tile, 1);
            }
        } else if (warp == 5 && lane == 0) {
            // ------------------------------- D4 = P v_new, off the critical path --------------------------
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
            for (int t = 0; t < NT; ++t) {
                const int s = t % STAGES;
                if (!mbar_wait_abortable(&bar_vn, t & 1, p.status, kTimeoutVN, abortp)) break;
                tc_fence_after_sync();
                const uint32_t sb = sm_u32 + s * L::kStage;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t ad = umma_smem_desc(sb + L::PB + ks * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = umma_smem_desc(sm_u32 + L::VN + (t & 1) * 4096 + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, SWZ_64B);
                    umma_bf16_ss(tmem + kColPV + (t & 1) * NV, ad, bd, idesc_pv, ks > 0);
                }
                umma_commit(&bar_pv[t & 1]);
                umma_commit(&bar_empty[s]);
            }
        }
    } else {
        // ------------------------------- chain warps (as in gdn_chain_kernel) ------------------------------
        const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;
        const bool issuer = (tid == 64);
        const int i = tid & 63;
        float st[NV];
        const size_t st_off = ((static_cast<size_t>(b) * p.Hv + hv) * kD + tid) * kD + dv0;
#pragma unroll
        for (int c = 0; c < NV; c += 4) {
            const float4 x = p.h0 ? *reinterpret_cast<const float4*>(p.h0 + st_off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            st[c] = x.x; st[c + 1] = x.y; st[c + 2] = x.z; st[c + 3] = x.w;
        }
        store_row32_bf16(sm + L::SB, tid, st);
        fence_proxy_async_smem();

        float f_tok = 0.f, f_tok_prev = 0.f, dC = 0.f;
        auto load_factors = [&](int t) {
            const float* vec = reinterpret_cast<const float*>(sm + (t % STAGES) * L::kStage + L::VEC);
            f_tok_prev = f_tok;
            f_tok = (warp < 2) ? vec[kChunk + i] : vec[i];
            dC = vec[2 * kChunk];
        };
        const uint64_t sb_desc0 = umma_smem_desc(sm_u32 + L::SB, 16384, 8 * L::kRowBytes, SWZ_64B);
        const uint64_t vs_desc0 = umma_smem_desc(sm_u32 + L::VS, 16384, 8 * L::kRowBytes, SWZ_64B);
        auto issue_d3 = [&](int t) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
            const uint64_t a0 = umma_smem_desc(sm_u32 + (t % STAGES) * L::kStage + L::QW, 16, 1024, SWZ_128B);
            const uint32_t d = tmem + kColD3 + (t & 1) * NV;
            tc_fence_after_sync();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_bf16_ss(d, a0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), sb_desc0 + ((ks * 16 * L::kRowBytes) >> 4),
                             idesc, ks > 0);
            umma_commit(&bar_d3);
        };
        auto out_epilogue = [&](int t, float qf) {
            const int s = t * kChunk + i;
            uint32_t a[32], c2[32];
            tmem_ld_x32(tmem_addr(tmem, lane_base, kColD3 + (t & 1) * NV), a);
            tmem_ld_x32(tmem_addr(tmem, lane_base, kColPV + (t & 1) * NV), c2);
            tmem_ld_wait();
            if (s < p.S) {
                __nv_bfloat16* dst = p.out + ((static_cast<size_t>(b) * p.S + s) * p.Hv + hv) * kD + dv0;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    float o[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) o[u] = fmaf(qf, __uint_as_float(a[8 * ch + u]), __uint_as_float(c2[8 * ch + u]));
                    uint4 pk;
                    pk.x = pack_bf16x2(o[0], o[1]); pk.y = pack_bf16x2(o[2], o[3]);
                    pk.z = pack_bf16x2(o[4], o[5]); pk.w = pack_bf16x2(o[6], o[7]);
                    *reinterpret_cast<uint4*>(dst + 8 * ch) = pk;
                }
            }
        };

        const bool cprof = p.prof != nullptr && issuer && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        long long cacc[7] = {0, 0, 0, 0, 0, 0, 0};
        long long ct = 0;
#define GDN_CPHASE(n)                                  \
    if (cprof) {                                       \
        const long long now_ = clock64();              \
        cacc[n] += now_ - ct;                          \
        ct = now_;                                     \
    }
        bool ok = mbar_wait_abortable(&bar_full[0], 0, p.status, kTimeoutFull, abortp);
        if (ok) load_factors(0);
        tc_fence_before_sync();
        named_bar_sync(2, 128);
        if (issuer && ok) issue_d3(0);

        if (cprof) ct = clock64();
        for (int t = 0; t < NT; ++t) {
            const int s = t % STAGES;
            uint8_t* stg = sm + s * L::kStage;
            if (warp >= 2) {
                uint32_t w[32];
                float x[NV], y[NV], u[32];
                // U does not depend on the state: fetch it while D3 is still in flight
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const uint4 uv = *reinterpret_cast<const uint4*>(stg + L::UB + swz_chunk_offset<64>(i, ch));
                    const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {     // bf16 pair -> two fp32
                        u[8 * ch + 2 * e] = __uint_as_float(uw[e] << 16);
                        u[8 * ch + 2 * e + 1] = __uint_as_float(uw[e] & 0xffff0000u);
                    }
                }
                ok = mbar_wait_abortable(&bar_d3, t & 1, p.status, kTimeoutD3, abortp) && ok;
                tc_fence_after_sync();
                GDN_CPHASE(0)
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColD3 + (t & 1) * NV), w);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float vn = u[c] - __uint_as_float(w[c]);
                    x[c] = vn;
                    y[c] = vn * f_tok;
                }
                if (t > 1)   // v_new is double-buffered: only D4 of chunk t-2 must have finished reading this buffer
                    ok = mbar_wait_abortable(&bar_pv[t & 1], ((t - 2) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
                store_row32_bf16(sm + L::VN + (t & 1) * 4096, i, x);
                store_row32_bf16(sm + L::VS, i, y);
                fence_proxy_async_smem();
                tc_fence_before_sync();
                named_bar_sync(1, 64);
                GDN_CPHASE(1)
                if (issuer && ok) {
                    constexpr uint32_t idesc_kv = umma_idesc_bf16(128, NV, MAJOR_MN, MAJOR_MN);
                    const uint64_t k0 = umma_smem_desc(sm_u32 + s * L::kStage + L::KT, 8192, 1024, SWZ_128B);
                    tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_bf16_ss(tmem + kColKV, k0 + ((ks * 2048) >> 4), vs_desc0 + ((ks * 16 * L::kRowBytes) >> 4),
                                     idesc_kv, ks > 0);
                    umma_commit(&bar_kv);
                }
                GDN_CPHASE(2)
            } else if (t > 0) {
                ok = mbar_wait_abortable(&bar_pv[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
                tc_fence_after_sync();
                out_epilogue(t - 1, f_tok_prev);
            }
            ok = mbar_wait_abortable(&bar_kv, t & 1, p.status, kTimeoutKV, abortp) && ok;
            tc_fence_after_sync();
            if (tid == 0 && ok) {
                mbar_arrive(&bar_empty[s]);
                mbar_arrive(&bar_vn);      // D5 is complete: warp 5 may now issue D4 without delaying the critical path
            }
            GDN_CPHASE(3)
            {
                uint32_t r[32];
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColKV), r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) st[c] = fmaf(dC, st[c], __uint_as_float(r[c]));
                store_row32_bf16(sm + L::SB, tid, st);
            }
            fence_proxy_async_smem();
            GDN_CPHASE(4)
            if (t + 1 < NT) {
                ok = mbar_wait_abortable(&bar_full[(t + 1) % STAGES], ((t + 1) / STAGES) & 1, p.status, kTimeoutFull, abortp) && ok;
                if (ok) load_factors(t + 1);
                else f_tok_prev = f_tok;
            } else {
                f_tok_prev = f_tok;
            }
            tc_fence_before_sync();
            named_bar_sync(2, 128);
            GDN_CPHASE(5)
            if (issuer && ok && t + 1 < NT) issue_d3(t + 1);
            GDN_CPHASE(6)
        }
#undef GDN_CPHASE
        if (cprof)
            for (int n = 0; n < 7; ++n) p.prof[8 + n] = cacc[n];
        if (warp < 2 && NT > 0) {
            ok = mbar_wait_abortable(&bar_pv[(NT - 1) & 1], ((NT - 1) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
            tc_fence_after_sync();
            out_epilogue(NT - 1, f_tok_prev);
        }
        if (ok && p.hT) {
#pragma unroll
            for (int c = 0; c < NV; c += 4)
                *reinterpret_cast<float4*>(p.hT + st_off + c) = make_float4(st[c], st[c + 1], st[c + 2], st[c + 3]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abortp) {   // let copies that may still be in flight land before the CTA's memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 100000ull) {}
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace

bool coop_supported(const Problem& p) {
    return static_cast<long long>(p.B) * p.Hv * (kD / NV) <= sm_count() && p.B <= 65535 && p.Hv <= 65535;
}

int launch_coop(const Problem& p, const Workspace& ws, int* flags, size_t flag_bytes, cudaStream_t stream, bool skip_prepare) {
    if (!coop_supported(p)) return GDN_ERR_BAD_ARGUMENT;
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tu, tus;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, &tus, &tu, NV)) return GDN_ERR_DRIVER;
    if (cudaMemsetAsync(flags, skip_prepare ? 1 : 0, flag_bytes, stream) != cudaSuccess) return GDN_ERR_CUDA;
    auto go = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, XSmem::kDynamic) != cudaSuccess)
            return GDN_ERR_CUDA;
        const dim3 grid(kD / NV, p.Hv, p.B), block(384);
        kernel<<<grid, block, XSmem::kDynamic, stream>>>(tq, tk, tv, tw, tp, tu, tus, p, ws, flags, skip_prepare ? 1 : 0);
        count_launch();
        return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
    };
    return p.gate_f32 ? go(gdn_coop_kernel<true>) : go(gdn_coop_kernel<false>);
}

}  // namespace gdn
