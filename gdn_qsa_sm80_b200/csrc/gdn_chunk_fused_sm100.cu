// Fused gdn_chunk forward for sm_100a: TMA-staged 64-token chunks, every dense product on
// tcgen05 (UMMA) with fp32 accumulators in TMEM, the recurrent state in fp32 registers.
//
// One CTA owns one (batch, value head, NV-column slice of Dv) and walks the chunks in order.
// The Dv slices of a head are independent (the state update never mixes value columns), so the
// column split is exact; it is the lever that gives B*Hv*(128/NV) CTAs when B*Hv is small.
//
// Per chunk (C = 64 tokens, gamma = inclusive cumsum of the log gate g inside the chunk), in the
// notation of the reference's torch definition (gdn_qsa_sm80/reference/gdn_chunk_ref.py:56-94):
//   D1  [K;Q] K^T                        -> raw K K^T (lanes 0-63) and Q K^T (lanes 64-127)
//       fp32 epilogue: A = tril(beta_i e^{gamma_i-gamma_j} K K^T, -1),  P = tril(scale e^{gamma_i-gamma_j} Q K^T)
//       (the pairwise factor is <= 1, so nothing overflows at chunk 64; ref :69-74)
//   T = (I + A)^-1 by blocked substitution in fp32 (ref :77-78 solve_triangular)
//   D2  [T diag(beta e^gamma) ; T diag(beta)] [K | V]  -> W (lanes 0-63), U (lanes 64-127)
//   D3  [Q ; W] S                        -> Q S (lanes 0-63), W S (lanes 64-127)       (ref :91-92)
//       v_new = U - W S ; also v~ = e^{gamma_C - gamma_i} v_new
//   D4  P v_new ;  O = scale e^{gamma_i} (Q S) + P v_new                               (ref :93)
//   D5  K^T v~  ;  S <- e^{gamma_C} S + K^T v~                                         (ref :94)
// Stacking two 64-row operands into one M = 128 UMMA keeps every accumulator in the plain
// "row i -> TMEM lane i" layout.  Raw TMA tiles are used as K-major operands (contraction over
// the head dimension) and as MN-major operands (contraction over tokens) without any transpose.
//
// This translation unit is the synchronous version: the CTA's 128 threads step through the
// phases together; one elected thread issues the UMMAs.
#include <cuda.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {

namespace {

constexpr int kAsStride = 68;   // fp32 row stride of the 64x64 solve matrices (16-byte aligned, conflict-free)

// Shared-memory map (bytes from a 1024-byte aligned base).
template <int NV>
struct Smem {
    static constexpr uint32_t kRowBytes = NV * 2;                 // bytes per row of NV-wide bf16 tiles
    static constexpr uint32_t kSwz = NV == 64 ? SWZ_128B : SWZ_64B;
    static constexpr uint32_t KQ = 0;                             // [K;Q]: 2 k-halves x 128 rows x 128 B
    static constexpr uint32_t QW = KQ + 32768;                    // [Q;W]: same shape
    static constexpr uint32_t TS = QW + 32768;                    // [T';T'']: 128 rows x 128 B
    static constexpr uint32_t PB = TS + 16384;                    // P: 64 rows x 128 B (+64 don't-care rows = AS)
    static constexpr uint32_t AS = PB + 8192;                     // A  fp32 64 x 68
    static constexpr uint32_t TM = AS + 17408;                    // T  fp32 64 x 68
    static constexpr uint32_t YT = TM + 17408;                    // solve temporaries, 1024 fp32
    static constexpr uint32_t VT = YT + 4096;                     // V tile: 64 rows x kRowBytes
    static constexpr uint32_t VN = VT + 64 * kRowBytes;           // v_new
    static constexpr uint32_t VS = VN + 64 * kRowBytes;           // v~ (decay-scaled v_new)
    static constexpr uint32_t SB = VS + 64 * kRowBytes;           // bf16 state: 128 rows x kRowBytes
    static constexpr uint32_t kBytes = SB + 128 * kRowBytes;
    static constexpr uint32_t kDynamic = kBytes + 1024;           // slack for manual alignment
};

// TMEM columns (fp32, 128 lanes each)
constexpr uint32_t kColD1 = 0;     // 64 : K K^T | Q K^T
constexpr uint32_t kColW = 64;     // 128: W (lanes 0-63)
constexpr uint32_t kColU = 192;    // NV : U (lanes 64-127)
constexpr uint32_t kColQS = 256;   // NV : Q S (lanes 0-63) / W S (lanes 64-127)
constexpr uint32_t kColPV = 320;   // NV : P v_new (lanes 0-63)
constexpr uint32_t kColKV = 384;   // NV : K^T v~ (all lanes)
constexpr uint32_t kTmemCols = 512;
constexpr int kProfSlots = 16;

template <int NV>
__device__ __forceinline__ void store_row_bf16(uint8_t* tile, uint32_t row, const float* x) {
#pragma unroll
    for (int ch = 0; ch < NV / 8; ++ch) {
        uint4 pk;
        pk.x = pack_bf16x2(x[8 * ch + 0], x[8 * ch + 1]);
        pk.y = pack_bf16x2(x[8 * ch + 2], x[8 * ch + 3]);
        pk.z = pack_bf16x2(x[8 * ch + 4], x[8 * ch + 5]);
        pk.w = pack_bf16x2(x[8 * ch + 6], x[8 * ch + 7]);
        *reinterpret_cast<uint4*>(tile + swz_chunk_offset<NV * 2>(row, ch)) = pk;
    }
}

template <bool GATE_F32>
__device__ __forceinline__ float load_gate(const void* p, size_t idx) {
    if (GATE_F32) return static_cast<const float*>(p)[idx];
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

template <int NV, bool GATE_F32>
__global__ void __launch_bounds__(128, 1)
gdn_chunk_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, Problem p) {
    using L = Smem<NV>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u32 = smem_u32(sm);

    __shared__ __align__(8) uint64_t bar_tma;
    __shared__ __align__(8) uint64_t bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ float gam_s[kChunk];     // gamma * log2(e)
    __shared__ float bet_s[kChunk];
    __shared__ float wsum_s[2];
    __shared__ long long prof_s[kProfSlots];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
    const int hq = hv / (p.Hv / p.Hq);
    const int dv0 = split * NV;
    const int NT = (p.S + kChunk - 1) / kChunk;
    const float scale = rsqrtf(static_cast<float>(kD));

    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        fence_mbar_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;   // this warp's TMEM lanes

    // recurrent state: thread `tid` owns row dk = tid, columns dv0 .. dv0+NV-1, in fp32
    float st[NV];
    const size_t st_off = ((static_cast<size_t>(b) * p.Hv + hv) * kD + tid) * kD + dv0;
#pragma unroll
    for (int c = 0; c < NV; c += 4) {
        float4 x = p.h0 ? *reinterpret_cast<const float4*>(p.h0 + st_off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        st[c] = x.x; st[c + 1] = x.y; st[c + 2] = x.z; st[c + 3] = x.w;
    }
    store_row_bf16<NV>(sm + L::SB, tid, st);
    fence_proxy_async_smem();
    __syncthreads();

    float* As = reinterpret_cast<float*>(sm + L::AS);
    float* Tm = reinterpret_cast<float*>(sm + L::TM);
    float* Yt = reinterpret_cast<float*>(sm + L::YT);

    uint32_t ph_tma = 0, ph_mma = 0;
    bool ok = true;

    // optional per-phase cycle accounting by one thread of CTA (0,0,0)
    const bool prof_on = p.prof != nullptr && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    long long prof_t = 0;
    if (prof_on) {
        for (int i = 0; i < kProfSlots; ++i) prof_s[i] = 0;
        prof_t = clock64();
    }
#define GDN_PHASE(n)                                   \
    if (prof_on) {                                     \
        const long long now_ = clock64();              \
        prof_s[n] += now_ - prof_t;                    \
        prof_t = now_;                                 \
    }

    for (int t = 0; t < NT && ok; ++t) {
        const int s0 = t * kChunk;
        // ---- stage the chunk's tiles --------------------------------------------------------------
        if (tid == 0) {
            mbar_arrive_expect_tx(&bar_tma, 6 * 8192 + 64 * L::kRowBytes);
            tma_load_4d(sm + L::KQ + 0, &tm_k, &bar_tma, 0, hq, s0, b);        // K, d 0-63   -> rows 0-63
            tma_load_4d(sm + L::KQ + 16384, &tm_k, &bar_tma, 64, hq, s0, b);   // K, d 64-127
            tma_load_4d(sm + L::KQ + 8192, &tm_q, &bar_tma, 0, hq, s0, b);     // Q           -> rows 64-127
            tma_load_4d(sm + L::KQ + 24576, &tm_q, &bar_tma, 64, hq, s0, b);
            tma_load_4d(sm + L::QW + 0, &tm_q, &bar_tma, 0, hq, s0, b);        // Q again     -> rows 0-63 of [Q;W]
            tma_load_4d(sm + L::QW + 16384, &tm_q, &bar_tma, 64, hq, s0, b);
            tma_load_4d(sm + L::VT, &tm_v, &bar_tma, dv0, hv, s0, b);          // V slice
        }
        // ---- gates: inclusive cumsum of g over the chunk by warp shuffles ---------------------------
        float gsum = 0.f, bv = 0.f;
        if (tid < kChunk) {
            const int s = s0 + tid;
            float gv = 0.f;
            if (s < p.S) {
                const size_t idx = (static_cast<size_t>(b) * p.S + s) * p.Hv + hv;
                gv = load_gate<GATE_F32>(p.g, idx);
                bv = load_gate<GATE_F32>(p.beta, idx);
            }
            gsum = gv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float y = __shfl_up_sync(0xffffffffu, gsum, o);
                if (lane >= o) gsum += y;
            }
            if (lane == 31) wsum_s[warp] = gsum;
        }
        __syncthreads();
        if (tid < kChunk) {
            if (warp == 1) gsum += wsum_s[0];
            gam_s[tid] = gsum * kLog2e;
            bet_s[tid] = bv;
        }
        // zero the T matrix while the loads are in flight
        for (int e = tid; e < kChunk * kAsStride; e += 128) Tm[e] = 0.f;
        __syncthreads();

        ok = mbar_wait(&bar_tma, ph_tma, p.status, kDevTimeoutTma);
        ph_tma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;

        GDN_PHASE(0)
        // ---- D1 = [K;Q] K^T --------------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, 64, MAJOR_K, MAJOR_K);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t a = sm_u32 + L::KQ + (ks >> 2) * 16384 + (ks & 3) * 32;
                const uint64_t ad = umma_smem_desc(a, 16, 1024, SWZ_128B);
                umma_bf16_ss(tmem + kColD1, ad, ad, idesc, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        GDN_PHASE(1)
        // ---- mask epilogue: A (fp32, for the solve) and P (bf16 operand) -----------------------------
        {
            const int i = tid & 63;
            const float gi = gam_s[i];
            uint32_t r[32];
            if (warp < 2) {
                const float bi = bet_s[i];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tmem, lane_base, kColD1 + half * 32), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float4 o;
                        float* op = reinterpret_cast<float*>(&o);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int j = half * 32 + c + u;
                            const float m = exp2f(gi - gam_s[j]);
                            op[u] = (j < i) ? bi * m * __uint_as_float(r[c + u]) : 0.f;
                        }
                        *reinterpret_cast<float4*>(As + i * kAsStride + half * 32 + c) = o;
                    }
                }
            } else {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    tmem_ld_x32(tmem_addr(tmem, lane_base, kColD1 + half * 32), r);
                    tmem_ld_wait();
                    float x[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int j = half * 32 + c;
                        const float m = exp2f(gi - gam_s[j]);
                        x[c] = (j <= i) ? scale * m * __uint_as_float(r[c]) : 0.f;
                    }
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 pk;
                        pk.x = pack_bf16x2(x[8 * ch + 0], x[8 * ch + 1]);
                        pk.y = pack_bf16x2(x[8 * ch + 2], x[8 * ch + 3]);
                        pk.z = pack_bf16x2(x[8 * ch + 4], x[8 * ch + 5]);
                        pk.w = pack_bf16x2(x[8 * ch + 6], x[8 * ch + 7]);
                        *reinterpret_cast<uint4*>(sm + L::PB + swz_chunk_offset<128>(i, half * 4 + ch)) = pk;
                    }
                }
            }
        }
        tc_fence_before_sync();
        __syncthreads();

        GDN_PHASE(2)
        // ---- T = (I + A)^-1, blocked: 16x16 diagonal blocks by substitution, then two merge levels ----
        if (tid < 64) {
            const int blk = tid >> 4, c = tid & 15;
            const float* a = As + (16 * blk) * kAsStride + 16 * blk;
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = (i == c) ? 1.f : 0.f;
#pragma unroll
            for (int i = 1; i < 16; ++i) {
                float acc = x[i];
#pragma unroll
                for (int j = 0; j < i; ++j) acc = fmaf(-a[i * kAsStride + j], x[j], acc);
                x[i] = acc;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) Tm[(16 * blk + i) * kAsStride + 16 * blk + c] = x[i];
        }
        __syncthreads();
        GDN_PHASE(3)
        {   // level 1: within each 32x32 diagonal block, X21 = -X22 (A21 X11)
            const int pr = tid >> 6, i = (tid >> 2) & 15, c0 = (tid & 3) * 4;
            const float* a21 = As + (32 * pr + 16 + i) * kAsStride + 32 * pr;
            float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const float av = a21[k];
                const float4 x = *reinterpret_cast<const float4*>(Tm + (32 * pr + k) * kAsStride + 32 * pr + c0);
                y[0] = fmaf(av, x.x, y[0]); y[1] = fmaf(av, x.y, y[1]);
                y[2] = fmaf(av, x.z, y[2]); y[3] = fmaf(av, x.w, y[3]);
            }
            *reinterpret_cast<float4*>(Yt + pr * 256 + i * 16 + c0) = make_float4(y[0], y[1], y[2], y[3]);
            __syncthreads();
            const float* x22 = Tm + (32 * pr + 16 + i) * kAsStride + 32 * pr + 16;
            float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const float tv = x22[k];
                const float4 yv = *reinterpret_cast<const float4*>(Yt + pr * 256 + k * 16 + c0);
                z[0] = fmaf(tv, yv.x, z[0]); z[1] = fmaf(tv, yv.y, z[1]);
                z[2] = fmaf(tv, yv.z, z[2]); z[3] = fmaf(tv, yv.w, z[3]);
            }
            __syncthreads();   // every read of the diagonal blocks of this level is done
            *reinterpret_cast<float4*>(Tm + (32 * pr + 16 + i) * kAsStride + 32 * pr + c0) =
                make_float4(-z[0], -z[1], -z[2], -z[3]);
        }
        __syncthreads();
        GDN_PHASE(4)
        {   // level 2: X[32:64, 0:32] = -T[32:64,32:64] (A[32:64,0:32] T[0:32,0:32])
            const int i = tid >> 2, c0 = (tid & 3) * 8;
            const float* all = As + (32 + i) * kAsStride;
            float y[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) y[u] = 0.f;
#pragma unroll 8
            for (int k = 0; k < 32; ++k) {
                const float av = all[k];
                const float4 x0 = *reinterpret_cast<const float4*>(Tm + k * kAsStride + c0);
                const float4 x1 = *reinterpret_cast<const float4*>(Tm + k * kAsStride + c0 + 4);
                y[0] = fmaf(av, x0.x, y[0]); y[1] = fmaf(av, x0.y, y[1]);
                y[2] = fmaf(av, x0.z, y[2]); y[3] = fmaf(av, x0.w, y[3]);
                y[4] = fmaf(av, x1.x, y[4]); y[5] = fmaf(av, x1.y, y[5]);
                y[6] = fmaf(av, x1.z, y[6]); y[7] = fmaf(av, x1.w, y[7]);
            }
            *reinterpret_cast<float4*>(Yt + i * 32 + c0) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(Yt + i * 32 + c0 + 4) = make_float4(y[4], y[5], y[6], y[7]);
            __syncthreads();
            const float* thi = Tm + (32 + i) * kAsStride + 32;
            float z[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) z[u] = 0.f;
#pragma unroll 8
            for (int k = 0; k < 32; ++k) {
                const float tv = thi[k];
                const float4 y0 = *reinterpret_cast<const float4*>(Yt + k * 32 + c0);
                const float4 y1 = *reinterpret_cast<const float4*>(Yt + k * 32 + c0 + 4);
                z[0] = fmaf(tv, y0.x, z[0]); z[1] = fmaf(tv, y0.y, z[1]);
                z[2] = fmaf(tv, y0.z, z[2]); z[3] = fmaf(tv, y0.w, z[3]);
                z[4] = fmaf(tv, y1.x, z[4]); z[5] = fmaf(tv, y1.y, z[5]);
                z[6] = fmaf(tv, y1.z, z[6]); z[7] = fmaf(tv, y1.w, z[7]);
            }
            *reinterpret_cast<float4*>(Tm + (32 + i) * kAsStride + c0) = make_float4(-z[0], -z[1], -z[2], -z[3]);
            *reinterpret_cast<float4*>(Tm + (32 + i) * kAsStride + c0 + 4) = make_float4(-z[4], -z[5], -z[6], -z[7]);
        }
        __syncthreads();
        GDN_PHASE(5)
        {   // T' = T diag(beta e^gamma) (rows 0-63), T'' = T diag(beta) (rows 64-127), bf16, K-major operand
            const int i = tid & 63, which = tid >> 6;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                float x[8];
                const float4 t0 = *reinterpret_cast<const float4*>(Tm + i * kAsStride + ch * 8);
                const float4 t1 = *reinterpret_cast<const float4*>(Tm + i * kAsStride + ch * 8 + 4);
                const float tv[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int j = ch * 8 + u;
                    float f = bet_s[j];
                    if (which == 0) f *= exp2f(gam_s[j]);
                    x[u] = tv[u] * f;
                }
                uint4 pk;
                pk.x = pack_bf16x2(x[0], x[1]); pk.y = pack_bf16x2(x[2], x[3]);
                pk.z = pack_bf16x2(x[4], x[5]); pk.w = pack_bf16x2(x[6], x[7]);
                *reinterpret_cast<uint4*>(sm + L::TS + swz_chunk_offset<128>(which * 64 + i, ch)) = pk;
            }
        }
        fence_proxy_async_smem();
        __syncthreads();

        GDN_PHASE(6)
        // ---- D2 = [T';T''] [K | V] -------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
            constexpr uint32_t idesc_w = umma_idesc_bf16(128, 128, MAJOR_K, MAJOR_MN);
            constexpr uint32_t idesc_u = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + L::TS + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bk = umma_smem_desc(sm_u32 + L::KQ + ks * 2048, 16384, 1024, SWZ_128B);
                umma_bf16_ss(tmem + kColW, ad, bk, idesc_w, ks > 0);
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + L::TS + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bv_ = umma_smem_desc(sm_u32 + L::VT + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, L::kSwz);
                umma_bf16_ss(tmem + kColU, ad, bv_, idesc_u, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        GDN_PHASE(7)
        // ---- W: TMEM fp32 -> bf16 rows 64-127 of the [Q;W] operand ----------------------------------
        if (warp < 2) {
            uint32_t r[32];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColW + q4 * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16x2(__uint_as_float(r[8 * ch + 0]), __uint_as_float(r[8 * ch + 1]));
                    pk.y = pack_bf16x2(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
                    pk.z = pack_bf16x2(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
                    pk.w = pack_bf16x2(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
                    *reinterpret_cast<uint4*>(sm + L::QW + (q4 >> 1) * 16384 +
                                              swz_chunk_offset<128>(64 + tid, (q4 & 1) * 4 + ch)) = pk;
                }
            }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();

        GDN_PHASE(8)
        // ---- D3 = [Q;W] S ----------------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
            constexpr uint32_t idesc = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + L::QW + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                const uint64_t bd = umma_smem_desc(sm_u32 + L::SB + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, L::kSwz);
                umma_bf16_ss(tmem + kColQS, ad, bd, idesc, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        GDN_PHASE(9)
        // ---- v_new = U - W S (token rows on lanes 64-127) ---------------------------------------------
        if (warp >= 2) {
            const int i = tid - 64;
            const float kd = exp2f(gam_s[kChunk - 1] - gam_s[i]);
            uint32_t u[32], w[32];
            float x[NV], y[NV];
#pragma unroll
            for (int part = 0; part < NV / 32; ++part) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColU + part * 32), u);
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColQS + part * 32), w);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float vn = __uint_as_float(u[c]) - __uint_as_float(w[c]);
                    x[part * 32 + c] = vn;
                    y[part * 32 + c] = vn * kd;
                }
            }
            store_row_bf16<NV>(sm + L::VN, i, x);
            store_row_bf16<NV>(sm + L::VS, i, y);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();

        GDN_PHASE(10)
        // ---- D4 = P v_new ; D5 = K^T v~ ----------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after_sync();
            constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NV, MAJOR_K, MAJOR_MN);
            constexpr uint32_t idesc_kv = umma_idesc_bf16(128, NV, MAJOR_MN, MAJOR_MN);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + L::PB + ks * 32, 16, 1024, SWZ_128B);
                const uint64_t bd = umma_smem_desc(sm_u32 + L::VN + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, L::kSwz);
                umma_bf16_ss(tmem + kColPV, ad, bd, idesc_pv, ks > 0);
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint64_t ad = umma_smem_desc(sm_u32 + L::KQ + ks * 2048, 16384, 1024, SWZ_128B);
                const uint64_t bd = umma_smem_desc(sm_u32 + L::VS + ks * 16 * L::kRowBytes, 16384, 8 * L::kRowBytes, L::kSwz);
                umma_bf16_ss(tmem + kColKV, ad, bd, idesc_kv, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, ph_mma, p.status, kDevTimeoutMma);
        ph_mma ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        GDN_PHASE(11)
        // ---- O rows (lanes 0-63) ------------------------------------------------------------------------
        if (warp < 2) {
            const int i = tid, s = s0 + i;
            const float qf = scale * exp2f(gam_s[i]);
            uint32_t a[32], c2[32];
#pragma unroll
            for (int part = 0; part < NV / 32; ++part) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColQS + part * 32), a);
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColPV + part * 32), c2);
                tmem_ld_wait();
                if (s < p.S) {
                    __nv_bfloat16* dst = p.out + ((static_cast<size_t>(b) * p.S + s) * p.Hv + hv) * kD + dv0 + part * 32;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        float o[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            o[u] = fmaf(qf, __uint_as_float(a[8 * ch + u]), __uint_as_float(c2[8 * ch + u]));
                        uint4 pk;
                        pk.x = pack_bf16x2(o[0], o[1]); pk.y = pack_bf16x2(o[2], o[3]);
                        pk.z = pack_bf16x2(o[4], o[5]); pk.w = pack_bf16x2(o[6], o[7]);
                        *reinterpret_cast<uint4*>(dst + 8 * ch) = pk;
                    }
                }
            }
        }
        // ---- state rows (all lanes): S <- e^{gamma_C} S + K^T v~ ---------------------------------------
        {
            const float dC = exp2f(gam_s[kChunk - 1]);
            uint32_t r[32];
#pragma unroll
            for (int part = 0; part < NV / 32; ++part) {
                tmem_ld_x32(tmem_addr(tmem, lane_base, kColKV + part * 32), r);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) st[part * 32 + c] = fmaf(dC, st[part * 32 + c], __uint_as_float(r[c]));
            }
            store_row_bf16<NV>(sm + L::SB, tid, st);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        GDN_PHASE(12)
    }
#undef GDN_PHASE
    if (prof_on)
        for (int i = 0; i < kProfSlots; ++i) p.prof[i] = prof_s[i];

    if (ok && p.hT) {
#pragma unroll
        for (int c = 0; c < NV; c += 4)
            *reinterpret_cast<float4*>(p.hT + st_off + c) = make_float4(st[c], st[c + 1], st[c + 2], st[c + 3]);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

template <int NV>
int launch_nv(const Problem& p, cudaStream_t stream) {
    alignas(64) CUtensorMap tq, tk, tv;
    const unsigned long long dq[4] = {static_cast<unsigned long long>(kD), static_cast<unsigned long long>(p.Hq),
                                      static_cast<unsigned long long>(p.S), static_cast<unsigned long long>(p.B)};
    const unsigned long long sq[3] = {kD * 2ull, static_cast<unsigned long long>(p.Hq) * kD * 2ull,
                                      static_cast<unsigned long long>(p.S) * p.Hq * kD * 2ull};
    const unsigned long long dvv[4] = {static_cast<unsigned long long>(kD), static_cast<unsigned long long>(p.Hv),
                                       static_cast<unsigned long long>(p.S), static_cast<unsigned long long>(p.B)};
    const unsigned long long sv[3] = {kD * 2ull, static_cast<unsigned long long>(p.Hv) * kD * 2ull,
                                      static_cast<unsigned long long>(p.S) * p.Hv * kD * 2ull};
    const unsigned box_qk[4] = {64, 1, 64, 1};
    const unsigned box_v[4] = {static_cast<unsigned>(NV), 1, 64, 1};
    if (encode_tma_bf16(&tq, p.q, 4, dq, sq, box_qk, 128)) return GDN_ERR_DRIVER;
    if (encode_tma_bf16(&tk, p.k, 4, dq, sq, box_qk, 128)) return GDN_ERR_DRIVER;
    if (encode_tma_bf16(&tv, p.v, 4, dvv, sv, box_v, NV * 2)) return GDN_ERR_DRIVER;

    using L = Smem<NV>;
    auto gate_launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return GDN_ERR_CUDA;
        const dim3 grid(kD / NV, p.Hv, p.B), block(128);
        kernel<<<grid, block, L::kDynamic, stream>>>(tq, tk, tv, p);
        count_launch();
        return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
    };
    if (p.gate_f32) return gate_launch(gdn_chunk_fused_kernel<NV, true>);
    return gate_launch(gdn_chunk_fused_kernel<NV, false>);
}

}  // namespace

int launch_fused(const Problem& p, int nv, cudaStream_t stream) {
    if (nv == 64) return launch_nv<64>(p, stream);
    if (nv == 32) return launch_nv<32>(p, stream);
    return GDN_ERR_BAD_ARGUMENT;
}

}  // namespace gdn
