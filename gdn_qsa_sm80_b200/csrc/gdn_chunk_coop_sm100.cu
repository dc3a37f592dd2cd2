// Single-launch gdn_chunk forward for problems with few independent sequences.
//
// One launch contains two kinds of roles that talk through the workspace in global memory:
//   * chain roles run the serial state recurrence and the outputs exactly as gdn_chain_kernel does (one CTA per
//     (batch, value head, NV-column slice of Dv));
//   * prepare groups (128 threads) compute the state-independent quantities of a chunk exactly as
//     gdn_prepare_kernel does (W, U, P, per-token factors), stage W/U in shared memory, and hand them to a
//     publisher thread that stores them by TMA, waits for the stores to complete and raises a per-tile flag
//     (st.release.gpu); the chain's TMA producer polls that flag (ld.acquire.gpu) before it loads chunk t.
// Every chunk is prepared once, while the chains of earlier chunks are running, so the prepare work hides behind
// the chain's latency instead of preceding it as a separate kernel, and the workspace is consumed from L2
// microseconds after it is written.
//
// Roles: NV = 32.  Every CTA is a chain CTA (4 per head) plus one prepare group that prepares every fourth chunk
// of its own head.  12 warps: 0-3 chain epilogues (warp 2 lane 0 issues D3/D5), 4 TMA producer, 5 issues D4,
// 6 publisher, 8-11 prepare group.  Needs 4*B*Hv <= #SMs.  Used for short sequences (up to 1024 tokens); longer ones
// and larger batches take the prepare kernel and the transposed chain.
//
// All CTAs must be resident together (one CTA per SM because of its shared memory): the kernel is launched
// cooperatively, so the runtime refuses a grid that cannot be resident at once and schedules it as a whole.
// Waiting is on flags written inside the same launch; every wait is bounded and a wait that runs out sets the
// status word and drains the CTA.
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "gdn_prep_device.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

constexpr int STAGES = 2;

// one prepare group's shared memory (offsets inside its region)
constexpr uint32_t PKQ = 0;                   // [K;Q] stack; V replaces Q once Q K^T is done
constexpr uint32_t PAS = PKQ + 32768;         // A fp32 64x68, then the bf16 [T';T''] operand, then the W staging tile
constexpr uint32_t PTM = PAS + 17408;         // T fp32 64x68, then the U staging tile
constexpr uint32_t PYT = PTM + 17408;         // merge temporaries
constexpr uint32_t kPrepBytes = PYT + 5120;   // 72704 = 71 KB

template <int NV>
struct XSmem {
    static constexpr uint32_t kRowBytes = NV * 2;
    static constexpr uint32_t kSwz = NV == 64 ? SWZ_128B : SWZ_64B;
    // chain ring, one stage:
    static constexpr uint32_t KT = 0, QW = 16384, PB = 49152, UB = 57344, VEC = UB + 64 * kRowBytes, kStage = VEC + 1024;
    static constexpr uint32_t kStageTx = 16384 + 16384 + 16384 + 8192 + 64 * kRowBytes + 1024;
    static constexpr uint32_t VN = STAGES * kStage;              // v_new bf16, 2 buffers (chunk parity) x 64 rows
    static constexpr uint32_t VS = VN + 2 * 64 * kRowBytes;      // decay-scaled v_new
    static constexpr uint32_t SB = VS + 64 * kRowBytes;          // bf16 state, 128 rows
    static constexpr uint32_t kChainBytes = SB + 128 * kRowBytes;
    static_assert(kStage % 1024 == 0 && kChainBytes % 1024 == 0 && kPrepBytes % 1024 == 0, "tiles must stay 1024-byte aligned");
};

constexpr int kTimeoutFull = 0x301, kTimeoutEmpty = 0x302, kTimeoutD3 = 0x303, kTimeoutKV = 0x304, kTimeoutPV = 0x305,
              kTimeoutVN = 0x306, kTimeoutFlag = 0x307, kTimeoutPrepTma = 0x308, kTimeoutPrepMma = 0x309,
              kTimeoutPrepFree = 0x30a, kTimeoutPrepReady = 0x30b;

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

// Which tiles a prepare group (and its publisher) walks.
//   per_head: chunks first, first + stride, ... of one fixed (b, hv)
//   otherwise: linear index L = first, first + stride, ... < BH * NT, chunk-major: L -> (chunk L / BH, head L % BH)
struct TileSched {
    long long first, stride;
    int per_head, b, hv, NT, BH, Hv;
    __device__ __forceinline__ bool get(long long n, int& b_, int& hv_, int& t_) const {
        const long long L = first + n * stride;
        if (per_head) {
            b_ = b; hv_ = hv; t_ = static_cast<int>(L);
            return L < NT;
        }
        if (L >= static_cast<long long>(BH) * NT) return false;
        const int head = static_cast<int>(L % BH);
        t_ = static_cast<int>(L / BH);
        b_ = head / Hv;
        hv_ = head % Hv;
        return true;
    }
};

// Resources of one prepare group.
struct PrepRes {
    uint8_t* sm;          // base of its shared-memory region (generic pointer) ...
    uint32_t sm_u32;      // ... and the same as a shared-window address
    uint32_t tmem;        // first of its 256 TMEM columns
    int bar_id;           // named barrier of its 128 threads
    uint64_t *tma, *mma, *ready, *free_;
    PrepScratch* ps;
};

// ------------------------------------------------------------------------------------------------------
// prepare group (128 threads, ptid 0..127)
// ------------------------------------------------------------------------------------------------------
template <bool GATE_F32>
__device__ __forceinline__ void prepare_role(const PrepRes& r, int ptid, const CUtensorMap* tm_q, const CUtensorMap* tm_k,
                                             const CUtensorMap* tm_v, const Problem& p, const Workspace& ws,
                                             const TileSched& sched, volatile int* abortp, bool prof_cta) {
    const PrepCtx ctx{ptid, r.bar_id};
    PrepScratch& ps = *r.ps;
    const int pwarp = ptid >> 5, i = ptid & 63;
    const uint32_t lane_base = static_cast<uint32_t>(pwarp) * 32u;
    const float scale0 = rsqrtf(static_cast<float>(kD));
    const int NT = sched.NT, rep = p.Hv / p.Hq;
    float* As = reinterpret_cast<float*>(r.sm + PAS);
    float* Tm = reinterpret_cast<float*>(r.sm + PTM);
    float* Yt = reinterpret_cast<float*>(r.sm + PYT);
    uint8_t* kq = r.sm + PKQ;
    const uint32_t kq_u32 = r.sm_u32 + PKQ, ts_u32 = r.sm_u32 + PAS;
    const uint32_t tm_prep = r.tmem;
    uint32_t ph_tma = 0, ph_mma = 0, ph_free = 0;

    auto issue_kq = [&](int b, int hv, int t) {   // one thread
        const int hq = hv / rep;
        mbar_arrive_expect_tx(r.tma, 4 * 8192);
        tma_load_4d(kq + 0, tm_k, r.tma, 0, hq, t * kChunk, b);
        tma_load_4d(kq + 16384, tm_k, r.tma, 64, hq, t * kChunk, b);
        tma_load_4d(kq + 8192, tm_q, r.tma, 0, hq, t * kChunk, b);
        tma_load_4d(kq + 24576, tm_q, r.tma, 64, hq, t * kChunk, b);
    };
    auto load_gates = [&](int b, int hv, int t, float& gv, float& bv) {
        prep_load_gates<GATE_F32>(p.g, p.beta, static_cast<size_t>(b) * p.S + t * kChunk, hv, p.Hv,
                                  min(kChunk, p.S - t * kChunk), gv, bv, ctx, p.gate_act != 0);
    };
    // optional cycle accounting by thread 0 of one prepare group, summed over its tiles
    const bool prof_on = GDN_DIAG(p.prof != nullptr && ptid == 0 && prof_cta);
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long prof_t = prof_on ? clock64() : 0, prof_n = 0;
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_acc[n] += now_ - prof_t;                  \
        prof_t = now_;                                 \
    }
    int b, hv, t;
    float gv = 0.f, bv = 0.f;
    bool have = sched.get(0, b, hv, t);
    if (have) {
        if (ptid == 0) issue_kq(b, hv, t);
        load_gates(b, hv, t, gv, bv);
    }
    for (long long n = 0; have; ++n) {
        const size_t tile = (static_cast<size_t>(b) * p.Hv + hv) * NT + t;
        int bn, hvn, tn;
        const bool have_next = sched.get(n + 1, bn, hvn, tn);
        if (p.gate_act) prep_activate_gates(gv, bv);
        prep_gates(ps, gv, bv, scale0, ws.vec + tile * 256, ctx);
        ctx.sync();
        GDN_PHASE(0)
        mbar_wait_abortable(r.tma, ph_tma, p.status, kTimeoutPrepTma, abortp);
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
            umma_commit(r.mma);
        }
        if (p.l2norm) prep_l2norm_fold(ps, kq, ws.vec + tile * 256, ctx);   // while the UMMAs run
        mbar_wait_abortable(r.mma, ph_mma, p.status, kTimeoutPrepMma, abortp);
        ph_mma ^= 1;
        tc_fence_after_sync();
        GDN_PHASE(2)
        if (ptid == 0) {   // Q is no longer needed: V takes its place (two 64-column groups, 16 KB apart)
            mbar_arrive_expect_tx(r.tma, 2 * 8192);
            tma_load_4d(kq + 8192, tm_v, r.tma, 0, hv, t * kChunk, b);
            tma_load_4d(kq + 24576, tm_v, r.tma, 64, hv, t * kChunk, b);
        }
        // next tile's gates: a strided global read, issued a whole tile ahead so its latency never shows
        // (this tile's values were consumed by prep_gates above)
        if (have_next) load_gates(bn, hvn, tn, gv, bv);
        if (n > 0) {   // the previous tile's W / U staging tiles (the A and T buffers) have been read by its TMA stores
            mbar_wait_abortable(r.free_, ph_free, p.status, kTimeoutPrepFree, abortp);
            ph_free ^= 1;
        }
        prep_zero_upper_blocks(Tm, ctx);
        {
            float ri, diag[16];
            if (p.l2norm) prep_row_setup_l2(ps, i, ri, diag);
            else prep_row_setup(ps, i, ri, diag);
            const float scale = p.l2norm ? scale0 * ps.rn[kChunk + i] : scale0;   // row factor of P
            uint32_t rr[32];
            float f[32];
            if (pwarp < 2) {
                const float bi = p.l2norm ? ps.bet[i] * ps.rn[i] : ps.bet[i];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, half * 32), rr);
                    prep_row_factors(ps, i, half, ri, diag, f);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float4 o;
                        o.x = (half * 32 + c + 0 < i) ? bi * f[c + 0] * __uint_as_float(rr[c + 0]) : 0.f;
                        o.y = (half * 32 + c + 1 < i) ? bi * f[c + 1] * __uint_as_float(rr[c + 1]) : 0.f;
                        o.z = (half * 32 + c + 2 < i) ? bi * f[c + 2] * __uint_as_float(rr[c + 2]) : 0.f;
                        o.w = (half * 32 + c + 3 < i) ? bi * f[c + 3] * __uint_as_float(rr[c + 3]) : 0.f;
                        *reinterpret_cast<float4*>(As + i * kSolveStride + half * 32 + c) = o;
                    }
                }
            } else {
                __nv_bfloat16* prow = ws.P + tile * (kChunk * kChunk) + static_cast<size_t>(i) * kChunk;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tm_prep, lane_base, half * 32), rr);
                    prep_row_factors(ps, i, half, ri, diag, f);
                    tmem_ld_wait();
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(scale * f[8 * ch + 0] * __uint_as_float(rr[8 * ch + 0]), scale * f[8 * ch + 1] * __uint_as_float(rr[8 * ch + 1]));
                        pk.y = pack_bf16x2(scale * f[8 * ch + 2] * __uint_as_float(rr[8 * ch + 2]), scale * f[8 * ch + 3] * __uint_as_float(rr[8 * ch + 3]));
                        pk.z = pack_bf16x2(scale * f[8 * ch + 4] * __uint_as_float(rr[8 * ch + 4]), scale * f[8 * ch + 5] * __uint_as_float(rr[8 * ch + 5]));
                        pk.w = pack_bf16x2(scale * f[8 * ch + 6] * __uint_as_float(rr[8 * ch + 6]), scale * f[8 * ch + 7] * __uint_as_float(rr[8 * ch + 7]));
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
            prep_store_scaled_T_row(Tm, which == 0 ? ps.eg : ps.bet, i, r.sm + PAS, which * 64 + i);
        }
        fence_proxy_async_smem();
        ctx.sync();
        mbar_wait_abortable(r.tma, ph_tma, p.status, kTimeoutPrepTma, abortp);   // V has landed
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
            umma_commit(r.mma);
        }
        mbar_wait_abortable(r.mma, ph_mma, p.status, kTimeoutPrepMma, abortp);
        ph_mma ^= 1;
        tc_fence_after_sync();
        GDN_PHASE(6)
        // the tile's K/Q/V buffer is free: next tile's K and Q
        if (have_next && ptid == 0) issue_kq(bn, hvn, tn);
        // W and U (bf16) leave through swizzled staging tiles and TMA stores: W in the A buffer, U in the T buffer
        // (both dead once the last UMMA of the tile has finished)
        {
            uint32_t rr[32];
            uint8_t* dst = r.sm + (pwarp < 2 ? PAS : PTM);
            const uint32_t col0 = pwarp < 2 ? 0u : 128u;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                tmem_ld_x32(tmem_addr(tm_prep, lane_base, col0 + q4 * 32), rr);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16x2(__uint_as_float(rr[8 * ch + 0]), __uint_as_float(rr[8 * ch + 1]));
                    pk.y = pack_bf16x2(__uint_as_float(rr[8 * ch + 2]), __uint_as_float(rr[8 * ch + 3]));
                    pk.z = pack_bf16x2(__uint_as_float(rr[8 * ch + 4]), __uint_as_float(rr[8 * ch + 5]));
                    pk.w = pack_bf16x2(__uint_as_float(rr[8 * ch + 6]), __uint_as_float(rr[8 * ch + 7]));
                    *reinterpret_cast<uint4*>(dst + (q4 >> 1) * 8192 + swz_chunk_offset<128>(i, (q4 & 1) * 4 + ch)) = pk;
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        ctx.sync();
        // hand the staging tiles to the publisher thread: it stores them, frees them and raises the flag
        if (ptid == 0) mbar_arrive(r.ready);
        GDN_PHASE(7)
        ++prof_n;
        have = have_next;
        b = bn; hv = hvn; t = tn;
    }
#undef GDN_PHASE
    if (prof_on) {
        for (int n = 0; n < 8; ++n) p.prof[n] = prof_acc[n];
        p.prof[15] = prof_n;
    }
}

// Publisher of one prepare group (one thread): stores W and U from the staging tiles, frees the tiles, and raises the
// tile's flag once the stores are complete; on its own thread the ~3 us write latency stays off the prepare group.
__device__ __forceinline__ void publisher_role(const PrepRes& r, const CUtensorMap* tm_w, const CUtensorMap* tm_us,
                                               const Problem& p, int* flags, const TileSched& sched, volatile int* abortp) {
    uint32_t ph = 0;
    int b, hv, t;
    for (long long n = 0; sched.get(n, b, hv, t); ++n) {
        if (!mbar_wait_abortable(r.ready, ph, p.status, kTimeoutPrepReady, abortp)) break;
        ph ^= 1;
        const size_t tile = (static_cast<size_t>(b) * p.Hv + hv) * sched.NT + t;
        const int row0 = static_cast<int>(tile * kChunk);
        tma_store_2d(tm_w, r.sm + PAS, 0, row0);
        tma_store_2d(tm_w, r.sm + PAS + 8192, 64, row0);
        tma_store_2d(tm_us, r.sm + PTM, 0, row0);
        tma_store_2d(tm_us, r.sm + PTM + 8192, 64, row0);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(r.free_);
        tma_store_wait_all();
        fence_proxy_async_all();
        __threadfence();         // cumulative: also covers the group's P / factor stores ordered before `ready`
        if (!*abortp) st_release_gpu(flags + tile, 1);
    }
}

// ------------------------------------------------------------------------------------------------------
// chain roles of one CTA: G = NV / 32 groups of four epilogue warps (warps 0 .. 4G-1; warp w works on TMEM lane
// quadrant w % 4 and on columns [32 (w / 4), +32) of the slice; warp 2 lane 0 issues D3 / D5), warp 4G lane 0 TMA
// producer, warp 4G+1 lane 0 issues D4.  `sm` is the CTA's (1024-byte aligned) dynamic shared memory, chain region first.
// ------------------------------------------------------------------------------------------------------
struct ChainBars {
    uint64_t *full, *empty;   // [STAGES] each
    uint64_t *d3, *kv, *vn, *pv;   // pv: [2]
};

template <int NV>
__device__ __forceinline__ void chain_roles(uint8_t* sm, uint32_t sm_u32, uint32_t tmem, const ChainBars& cb,
                                            const CUtensorMap* tm_q, const CUtensorMap* tm_k, const CUtensorMap* tm_w,
                                            const CUtensorMap* tm_p, const CUtensorMap* tm_u, const Problem& p,
                                            const Workspace& ws, const int* flags, volatile int* abortp, int split, int hv,
                                            int b, bool prof_cta) {
    using L = XSmem<NV>;
    constexpr uint32_t kColD3 = 0, kColPV = 2 * NV, kColKV = 4 * NV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hq = hv / (p.Hv / p.Hq);
    const int dv0 = split * NV;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const size_t tile0 = (static_cast<size_t>(b) * p.Hv + hv) * NT;

    constexpr int kGroups = NV / 32, kEpiWarps = 4 * kGroups;
    if (warp == kEpiWarps) {
        if (lane != 0) return;
        // ------------------------------- TMA producer ------------------------------------------------------
        for (int t = 0; t < NT; ++t) {
            const int s = t % STAGES;
            // first the flag (an L2 round trip, usually long since raised), then the stage: the flag read overlaps
            // the time the stage is still in use
            if (!wait_flag(flags + tile0 + t, p.status, abortp)) break;   // chunk t has been prepared
            fence_proxy_async_all();     // the workspace was written by another SM; order the TMA reads after the acquire
            if (t >= STAGES && !mbar_wait_abortable(&cb.empty[s], ((t / STAGES) - 1) & 1, p.status, kTimeoutEmpty, abortp))
                break;
            uint8_t* st = sm + s * L::kStage;
            const int s0 = t * kChunk;
            const int row0 = static_cast<int>((tile0 + t) * kChunk);
            mbar_arrive_expect_tx(&cb.full[s], L::kStageTx);
            tma_load_4d(st + L::KT + 0, tm_k, &cb.full[s], 0, hq, s0, b);
            tma_load_4d(st + L::KT + 8192, tm_k, &cb.full[s], 64, hq, s0, b);
            tma_load_4d(st + L::QW + 0, tm_q, &cb.full[s], 0, hq, s0, b);
            tma_load_4d(st + L::QW + 16384, tm_q, &cb.full[s], 64, hq, s0, b);
            tma_load_2d(st + L::QW + 8192, tm_w, &cb.full[s], 0, row0);
            tma_load_2d(st + L::QW + 24576, tm_w, &cb.full[s], 64, row0);
            tma_load_2d(st + L::PB, tm_p, &cb.full[s], 0, row0);
            tma_load_2d(st + L::UB, tm_u, &cb.full[s], dv0, row0);
            bulk_load_1d(st + L::VEC, ws.vec + (tile0 + t) * 256, 1024, &cb.full[s]);
        }
        return;
    }
    if (warp == kEpiWarps + 1) {
        if (lane != 0) return;
        // ------------------------------- D4 = P v_new, off the critical path ---------------------------------
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
        for (int t = 0; t < NT; ++t) {
            const int s = t % STAGES;
            if (!mbar_wait_abortable(cb.vn, t & 1, p.status, kTimeoutVN, abortp)) break;
            tc_fence_after_sync();
            const uint32_t sb = sm_u32 + s * L::kStage;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sb + L::PB + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bd = umma_smem_desc(sm_u32 + L::VN + (t & 1) * 64 * L::kRowBytes + ks * 16 * L::kRowBytes, 16384,
                                                   8 * L::kRowBytes, L::kSwz);
                umma_bf16_ss(tmem + kColPV + (t & 1) * NV, ad, bd, idesc_pv, ks > 0);
            }
            umma_commit(&cb.pv[t & 1]);
            umma_commit(&cb.empty[s]);    // second arrival: the P tile of this stage has been consumed
        }
        return;
    }
    // ------------------------------- epilogue warps -----------------------------------------------------------
    const int quad = warp & 3, cg = warp >> 2;          // TMEM lane quadrant; column group of the slice
    const int row = quad * 32 + lane;                   // state row (dk) this thread owns: 0..127
    const uint32_t lane_base = static_cast<uint32_t>(quad) * 32u;
    const uint32_t col0 = static_cast<uint32_t>(cg) * 32u;
    const bool issuer = (tid == 64);                    // group 0, quadrant 2
    const int i = row & 63;
    float st[32];
    const size_t st_off = ((static_cast<size_t>(b) * p.Hv + hv) * kD + row) * kD + dv0 + col0;
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
        const float4 x = p.h0 ? *reinterpret_cast<const float4*>(p.h0 + st_off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        st[c] = x.x; st[c + 1] = x.y; st[c + 2] = x.z; st[c + 3] = x.w;
    }
    store_row_bf16<NV>(sm + L::SB, row, st, cg);
    fence_proxy_async_smem();

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
        constexpr uint32_t idesc = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
        const uint64_t a0 = umma_smem_desc(sm_u32 + (t % STAGES) * L::kStage + L::QW, 16, 1024, SWZ_128B);
        const uint32_t d = tmem + kColD3 + (t & 1) * NV;
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
            umma_bf16_ss(d, a0 + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), sb_desc0 + ((ks * 16 * L::kRowBytes) >> 4), idesc, ks > 0);
        umma_commit(cb.d3);
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
                    float o[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) o[u] = fmaf(qf, __uint_as_float(a[8 * ch + u]), __uint_as_float(c2[8 * ch + u]));
                    uint4 pk;
                    pk.x = pack_bf16x2(o[0], o[1]); pk.y = pack_bf16x2(o[2], o[3]);
                    pk.z = pack_bf16x2(o[4], o[5]); pk.w = pack_bf16x2(o[6], o[7]);
                    *reinterpret_cast<uint4*>(dst + 8 * ch) = pk;
                }
            }
        }
    };

    // optional cycle accounting by the UMMA-issuing thread of one chain CTA, summed over chunks
    const bool cprof = GDN_DIAG(p.prof != nullptr && issuer && prof_cta);
    long long cacc[7] = {0, 0, 0, 0, 0, 0, 0};
    long long ct = 0;
#define GDN_CPHASE(n)                                  \
    if (cprof) {                                       \
        const long long now_ = clock64();              \
        cacc[n] += now_ - ct;                          \
        ct = now_;                                     \
    }
    bool ok = mbar_wait_abortable(&cb.full[0], 0, p.status, kTimeoutFull, abortp);
    if (ok) load_factors(0);
    tc_fence_before_sync();
    named_bar_sync(2, 128 * kGroups);
    if (issuer && ok) issue_d3(0);

    if (cprof) ct = clock64();
    for (int t = 0; t < NT; ++t) {
        const int s = t % STAGES;
        uint8_t* stg = sm + s * L::kStage;
        if (quad >= 2) {
            // ---- v_new = U - W S, and its decay-scaled copy ---------------------------------------------------
            float u[32];
            // U does not depend on the state: fetch it while D3 is still in flight
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                const uint4 uv = *reinterpret_cast<const uint4*>(stg + L::UB + swz_chunk_offset<NV * 2>(i, cg * 4 + ch));
                const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {     // bf16 pair -> two fp32
                    u[8 * ch + 2 * e] = __uint_as_float(uw[e] << 16);
                    u[8 * ch + 2 * e + 1] = __uint_as_float(uw[e] & 0xffff0000u);
                }
            }
            ok = mbar_wait_abortable(cb.d3, t & 1, p.status, kTimeoutD3, abortp) && ok;
            tc_fence_after_sync();
            GDN_CPHASE(0)
            float y[32];
            {
                uint32_t w[32];
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColD3 + (t & 1) * NV + col0), w);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float vn = u[c] - __uint_as_float(w[c]);
                    u[c] = vn;
                    y[c] = vn * f_tok;
                }
            }
            if (t > 1)   // v_new is double-buffered: only D4 of chunk t-2 must have finished reading this buffer
                ok = mbar_wait_abortable(&cb.pv[t & 1], ((t - 2) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
            store_row_bf16<NV>(sm + L::VN + (t & 1) * 64 * L::kRowBytes, i, u, cg);
            store_row_bf16<NV>(sm + L::VS, i, y, cg);
            fence_proxy_async_smem();
            tc_fence_before_sync();
            named_bar_sync(1, 64 * kGroups);
            GDN_CPHASE(1)
            if (issuer && ok) {
                constexpr uint32_t idesc_kv = umma_idesc_bf16(128, NV, MAJOR_MN, MAJOR_MN);
                const uint64_t k0 = umma_smem_desc(sm_u32 + s * L::kStage + L::KT, 8192, 1024, SWZ_128B);
                tc_fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_bf16_ss(tmem + kColKV, k0 + ((ks * 2048) >> 4), vs_desc0 + ((ks * 16 * L::kRowBytes) >> 4), idesc_kv, ks > 0);
                umma_commit(cb.kv);
            }
            GDN_CPHASE(2)
        } else if (t > 0) {
            // ---- output rows of the previous chunk, off the critical path --------------------------------------
            ok = mbar_wait_abortable(&cb.pv[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
            tc_fence_after_sync();
            out_epilogue(t - 1, f_tok_prev);
        }
        // ---- state rows: S <- exp(gamma_C) S + K^T v~ -----------------------------------------------------------
        ok = mbar_wait_abortable(cb.kv, t & 1, p.status, kTimeoutKV, abortp) && ok;
        tc_fence_after_sync();
        if (tid == 0 && ok) {
            mbar_arrive(&cb.empty[s]);   // first arrival: D3 and D5 of this stage are complete
            mbar_arrive(cb.vn);          // D5 is complete: warp 5 may issue D4 without delaying the critical path
        }
        GDN_CPHASE(3)
        {
            uint32_t r[32];
            tmem_ld_x32(tmem_addr(tmem, lane_base, kColKV + col0), r);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) st[c] = fmaf(dC, st[c], __uint_as_float(r[c]));
        }
        store_row_bf16<NV>(sm + L::SB, row, st, cg);
        fence_proxy_async_smem();
        GDN_CPHASE(4)
        if (t + 1 < NT) {
            ok = mbar_wait_abortable(&cb.full[(t + 1) % STAGES], ((t + 1) / STAGES) & 1, p.status, kTimeoutFull, abortp) && ok;
            if (ok) load_factors(t + 1);
            else f_tok_prev = f_tok;
        } else {
            f_tok_prev = f_tok;
        }
        tc_fence_before_sync();
        named_bar_sync(2, 128 * kGroups);
        GDN_CPHASE(5)
        if (issuer && ok && t + 1 < NT) issue_d3(t + 1);
        GDN_CPHASE(6)
    }
#undef GDN_CPHASE
    if (cprof)
        for (int n = 0; n < 7; ++n) p.prof[8 + n] = cacc[n];
    if (quad < 2 && NT > 0) {   // output rows of the last chunk
        ok = mbar_wait_abortable(&cb.pv[(NT - 1) & 1], ((NT - 1) >> 1) & 1, p.status, kTimeoutPV, abortp) && ok;
        tc_fence_after_sync();
        out_epilogue(NT - 1, f_tok_prev);
    }
    if (ok && p.hT) {
#pragma unroll
        for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(p.hT + st_off + c) = make_float4(st[c], st[c + 1], st[c + 2], st[c + 3]);
    }
}

template <int NV, bool GATE_F32>
__global__ void __launch_bounds__(384, 1)
gdn_coop_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_u,
                const __grid_constant__ CUtensorMap tm_us, Problem p, Workspace ws, int* flags, int skip_prepare) {
    using L = XSmem<NV>;
    constexpr int kSplits = kD / NV;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);

    __shared__ __align__(8) uint64_t bar_full[STAGES];
    __shared__ __align__(8) uint64_t bar_empty[STAGES];
    __shared__ __align__(8) uint64_t bar_d3, bar_kv, bar_vn;
    __shared__ __align__(8) uint64_t bar_pv[2];
    __shared__ __align__(8) uint64_t bar_prep[1][4];   // the prepare group's barriers: tma, mma, ready, free
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ __align__(16) PrepScratch ps[1];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const int bid = blockIdx.x;
    const int head = bid / kSplits, split = bid % kSplits;
    const int hv = head % p.Hv, b = head / p.Hv;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 2);   // D5 seen complete by a chain thread + D4 complete (commit)
        }
        mbar_init(&bar_d3, 1);
        mbar_init(&bar_kv, 1);
        mbar_init(&bar_vn, 1);
        mbar_init(&bar_pv[0], 1);
        mbar_init(&bar_pv[1], 1);
        for (int k = 0; k < 4; ++k) mbar_init(&bar_prep[0][k], 1);
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

    auto prep_res = [&](int gi, uint32_t region_off, uint32_t tmem_col) {
        PrepRes r;
        r.sm = sm + region_off;
        r.sm_u32 = sm_u32 + region_off;
        r.tmem = tmem + tmem_col;
        r.bar_id = 3 + gi;
        r.tma = &bar_prep[gi][0]; r.mma = &bar_prep[gi][1]; r.ready = &bar_prep[gi][2]; r.free_ = &bar_prep[gi][3];
        r.ps = &ps[gi];
        return r;
    };

    // every CTA: chain roles on warps 0-5, publisher on warp 6, one prepare group on warps 8-11
    if (warp < 4 * (NV / 32) + 2) {
        ChainBars cb{bar_full, bar_empty, &bar_d3, &bar_kv, &bar_vn, bar_pv};
        chain_roles<NV>(sm, sm_u32, tmem, cb, &tm_q, &tm_k, &tm_w, &tm_p, &tm_u, p, ws, flags, abortp, split, hv, b, bid == 0);
    } else if (!skip_prepare && (warp == 6 || warp >= 8)) {
        const PrepRes r = prep_res(0, L::kChainBytes, 256);
        const TileSched sched{split, kSplits, 1, b, hv, NT, p.B * p.Hv, p.Hv};
        if (warp >= 8) prepare_role<GATE_F32>(r, tid - 256, &tm_q, &tm_k, &tm_v, p, ws, sched, abortp, bid == 0);
        else if (lane == 0) publisher_role(r, &tm_w, &tm_us, p, flags, sched, abortp);
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

template <int NV>
int launch_coop_t(const Problem& p, const Workspace& ws, int* flags, size_t flag_bytes, cudaStream_t stream, bool skip_prepare) {
    alignas(64) CUtensorMap tq, tk, tv, tw, tp, tu, tus;
    if (encode_qkv_maps(p, &tq, &tk, &tv, 64)) return GDN_ERR_DRIVER;
    if (encode_workspace_maps(p, ws, &tw, &tp, &tus, &tu, NV)) return GDN_ERR_DRIVER;
    // p.dbg == 7 (test hook): chain roles only AND no flag raised, so that every chain CTA's wait for its first tile
    // runs into the time limit, reports through the status word and returns
    if (cudaMemsetAsync(flags, (skip_prepare && p.dbg != 7) ? 1 : 0, flag_bytes, stream) != cudaSuccess) return GDN_ERR_CUDA;
    using L = XSmem<NV>;
    const int grid = p.B * p.Hv * (kD / NV);
    const uint32_t smem = L::kChainBytes + kPrepBytes + 1024;
    auto go = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return GDN_ERR_CUDA;
        // Cooperative launch: the CTAs wait on flags raised by other CTAs of the same grid, so all of them must be
        // resident together.  The runtime checks that against the occupancy of this context and refuses the launch
        // (nothing runs) when the grid does not fit, instead of letting part of it spin until the wait limit.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(384);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, tw, tp, tu, tus, p, ws, flags, skip_prepare ? 1 : 0);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return GDN_ERR_CUDA;
        }
        count_launch();
        return GDN_OK;
    };
    return p.gate_f32 ? go(gdn_coop_kernel<NV, true>) : go(gdn_coop_kernel<NV, false>);
}

}  // namespace

// four chain CTAs per head, each with a prepare group
bool coop_supported(const Problem& p) {
    return static_cast<long long>(p.B) * p.Hv * 4 <= sm_count();
}

int launch_coop(const Problem& p, const Workspace& ws, int* flags, size_t flag_bytes, cudaStream_t stream, bool skip_prepare) {
    if (!coop_supported(p)) return GDN_ERR_BAD_ARGUMENT;
    return launch_coop_t<32>(p, ws, flags, flag_bytes, stream, skip_prepare);
}

}  // namespace gdn
