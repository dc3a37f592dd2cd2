// Device-side building blocks of the state-independent ("prepare") part of a chunk, shared by the
// kernels that need it: gate cumsum and decay tables, the masked K K^T / Q K^T epilogue, and the
// 64x64 unit-lower-triangular inverse T = (I + A)^-1.
//
// All functions are executed by the same 128 threads (4 warps) and communicate through the
// PrepScratch block in shared memory; callers place __syncthreads() where the comments say so.
#pragma once

#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {

constexpr int kSolveStride = 68;   // fp32 row stride of the 64x64 solve matrices: 16-byte aligned rows,
                                   // and 68 = 4 (mod 32) spreads rows over banks for row-wise and fragment reads
// row strides of the temporaries of merge levels 1 (16 columns) and 2 (32 columns): 40 = 8 (mod 32) keeps both the
// B-fragment reads (bank 8 t + g) and the accumulator-fragment stores of a half-warp off each other's banks
constexpr int kY1Stride = 40;
constexpr int kY2Stride = 40;
constexpr int kDiagScratch = 16 * kY1Stride;   // floats of scratch one warp needs in prep_invert_diag32
static_assert(2 * kDiagScratch <= 32 * kY2Stride, "the two warps' scratch must fit the buffer sized for merge level 2");

struct alignas(16) PrepScratch {
    float gam[kChunk];        // gamma_j * log2(e): inclusive cumsum of the log gate inside the chunk
    float bet[kChunk];        // beta_j (0 for padding tokens)
    float eg[kChunk];         // beta_j * exp(gamma_j)
    float ctab[3][kChunk];    // ctab[I-1][j] = exp(gamma_{16 I} - gamma_j) for j < 16 I  (always <= 1)
    float rn[2 * kChunk];     // optional in-kernel L2 normalisation: 1/|k_j| (0..63) and 1/|q_i| (64..127), else unused
    float wsum[2];
};

// Which 128 threads run the prepare steps: the whole CTA (thread index = threadIdx.x, __syncthreads) or a
// 128-thread group inside a larger CTA (its own thread numbering and a named barrier).
struct PrepCtx {
    int tid;
    int bar;   // 0 = __syncthreads(), otherwise the id of a 128-thread named barrier
    __device__ __forceinline__ static PrepCtx whole_cta() { return PrepCtx{static_cast<int>(threadIdx.x), 0}; }
    __device__ __forceinline__ void sync() const {
        if (bar == 0) __syncthreads();
        else named_bar_sync(static_cast<uint32_t>(bar), 128);
    }
};

template <bool GATE_F32>
__device__ __forceinline__ float prep_load_gate(const void* p, size_t idx) {
    if (GATE_F32) return static_cast<const float*>(p)[idx];
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

// Loads the log gate and the update gate of token `tid` of a chunk (threads 0-63; zeros for padding).
template <bool GATE_F32>
__device__ __forceinline__ void prep_load_gates(const void* g, const void* beta, size_t tok0, int hv, int Hv,
                                                int valid, float& gv, float& bv,
                                                PrepCtx ctx = PrepCtx::whole_cta(), bool raw_gates = false) {
    const int tid = ctx.tid;
    // padding: zeros, or (raw gates) the values prep_activate_gates maps to zeros
    gv = raw_gates ? -INFINITY : 0.f;
    bv = gv;
    if (tid < valid) {
        const size_t idx = (tok0 + tid) * Hv + hv;
        gv = prep_load_gate<GATE_F32>(g, idx);
        bv = prep_load_gate<GATE_F32>(beta, idx);
    }
}

// Gate activations inside the kernel: g = -softplus(raw), beta = sigmoid(raw), the way a GDN layer derives its gates
// (an extension; the reference takes finished gates).  -inf maps to g = 0, beta = 0 (padding).  Applied where the
// values are consumed, not where they are loaded, so the load stays a tile ahead.
__device__ __forceinline__ void prep_activate_gates(float& gv, float& bv) {
    gv = gv > 20.f ? -gv : -log1pf(__expf(gv));
    bv = 1.f / (1.f + __expf(-bv));
}

// Gate cumsum over the chunk by warp shuffles (threads 0-63 hold one token each: gv, bv) and the decay tables.
// Contains two barriers of the group; a third one is needed before the tables are read.
// If vec_out != nullptr, also writes the per-token factors a later kernel needs:
//   vec_out[i] = exp(gamma_C - gamma_i), vec_out[64+i] = scale * exp(gamma_i), vec_out[128] = exp(gamma_C).
// tables = false skips the block decay tables (ctab) for callers whose mask epilogue does not use them.
__device__ __forceinline__ void prep_gates(PrepScratch& ps, float gv, float bv, float scale, float* vec_out,
                                           PrepCtx ctx = PrepCtx::whole_cta(), bool tables = true) {
    const int tid = ctx.tid, warp = tid >> 5, lane = tid & 31;
    float gsum = 0.f;
    if (tid < kChunk) {
        gsum = gv;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, gsum, o);
            if (lane >= o) gsum += y;
        }
        if (lane == 31) ps.wsum[warp] = gsum;
    }
    ctx.sync();
    if (tid < kChunk) {
        if (warp == 1) gsum += ps.wsum[0];
        ps.gam[tid] = gsum * kLog2e;
        ps.bet[tid] = bv;
    }
    ctx.sync();
    if (tid < kChunk) {
        const float gi = ps.gam[tid], gC = ps.gam[kChunk - 1];
        const float e = exp2f(gi);
        ps.eg[tid] = bv * e;
        if (vec_out) {
            vec_out[tid] = exp2f(gC - gi);
            vec_out[kChunk + tid] = scale * e;
            if (tid == 0) vec_out[2 * kChunk] = exp2f(gC);
        }
    }
    if (tables && tid < 96) {   // 16 + 32 + 48 table entries
        const int I = tid < 16 ? 1 : (tid < 48 ? 2 : 3);
        const int j = tid - (I == 1 ? 0 : (I == 2 ? 16 : 48));
        ps.ctab[I - 1][j] = exp2f(ps.gam[16 * I] - ps.gam[j]);
    }
}

// Pairwise decay factors of row i for the 32 columns [32*half, 32*half+32):
//   f[c] = exp(gamma_i - gamma_j) for j <= i, 0 above the diagonal.
// Off-diagonal 16-blocks use exp(gamma_i - gamma_ref) * exp(gamma_ref - gamma_j) with ref = first token
// of row i's block (both factors <= 1, so nothing overflows); the diagonal block uses direct exponentials.
__device__ __forceinline__ void prep_row_factors(const PrepScratch& ps, int i, int half, float ri,
                                                 const float (&diag)[16], float (&f)[32]) {
    const int I = i >> 4;
    const float* ct = ps.ctab[I > 0 ? I - 1 : 0];
#pragma unroll
    for (int J2 = 0; J2 < 2; ++J2) {
        const int J = half * 2 + J2;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 c4 = *reinterpret_cast<const float4*>(ct + 16 * J + 4 * q);
            const float cv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int jj = 4 * q + u;
                f[16 * J2 + jj] = (J < I) ? ri * cv[u] : ((J == I) ? diag[jj] : 0.f);
            }
        }
    }
}

// In-kernel L2 normalisation of q and k (the reference's torch definition has it as use_qk_l2norm_in_kernel,
// gdn_qsa_sm80/reference/gdn_chunk_ref.py:15-17, :43-45: x * rsqrt(sum x^2 + 1e-6)).  Nothing is rewritten in the
// tiles: the inverse norms are folded into factors that exist anyway.  With rk_j = 1/|k_j|, rq_i = 1/|q_i|:
//   K K^T, Q K^T columns  -> the decay tables (ctab here, the diagonal factors in prep_row_setup_l2)
//   rows of A / P         -> beta_i rk_i and scale rq_i (callers)
//   W = T (beta e^gamma K)-> eg_j rk_j
//   K^T v~ and (Q S) later-> the per-token factors in vec_out: exp(gamma_C-gamma_i) rk_i and scale exp(gamma_i) rq_i
// `kq` is the [K;Q] stack (two k-halves of 128 rows x 128 bytes, 128-byte swizzle; the swizzle only permutes the
// 16-byte chunks inside a row, so a row's sum of squares needs no un-swizzling).  Thread r handles row r.
// Contains two group barriers; call after the tiles have landed and before the tables are used.
__device__ __forceinline__ void prep_l2norm_fold(PrepScratch& ps, const uint8_t* kq, float* vec_out,
                                                 PrepCtx ctx = PrepCtx::whole_cta()) {
    const int tid = ctx.tid;
    float ss = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            // rotate the chunk order by the row number: rows are 128 B apart, so this spreads a warp over the banks
            const uint4 v = *reinterpret_cast<const uint4*>(kq + half * 16384 + tid * 128 + ((ch + tid) & 7) * 16);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                ss = fmaf(lo, lo, ss);
                ss = fmaf(hi, hi, ss);
            }
        }
    ps.rn[tid] = rsqrtf(ss + 1e-6f);
    ctx.sync();
    if (tid < kChunk) {
        ps.eg[tid] *= ps.rn[tid];
        if (vec_out) {
            vec_out[tid] *= ps.rn[tid];
            vec_out[kChunk + tid] *= ps.rn[kChunk + tid];
        }
    }
    if (tid < 96) {
        const int I = tid < 16 ? 1 : (tid < 48 ? 2 : 3);
        const int j = tid - (I == 1 ? 0 : (I == 2 ? 16 : 48));
        ps.ctab[I - 1][j] *= ps.rn[j];
    }
    ctx.sync();
}

// Per-thread setup for prep_row_factors: ri and the 16 diagonal-block factors of row i.
__device__ __forceinline__ void prep_row_setup(const PrepScratch& ps, int i, float& ri, float (&diag)[16]) {
    const int I = i >> 4, ii = i & 15;
    const float gi = ps.gam[i];
    ri = exp2f(gi - ps.gam[16 * I]);
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) diag[jj] = (jj <= ii) ? exp2f(gi - ps.gam[16 * I + jj]) : 0.f;
}

// Same with the column norms 1/|k_j| folded into the diagonal-block factors (L2 normalisation on).
__device__ __forceinline__ void prep_row_setup_l2(const PrepScratch& ps, int i, float& ri, float (&diag)[16]) {
    prep_row_setup(ps, i, ri, diag);
    const int I = i >> 4;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) diag[jj] *= ps.rn[16 * I + jj];
}

__device__ __forceinline__ uint32_t f32_to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// Warp-level 16x8x8 TF32 product with fp32 accumulation (legacy tensor path; used only for the
// small merge products of the triangular inverse, about 1% of the chunk's arithmetic).
__device__ __forceinline__ void mma_tf32_16x8x8(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// A fragment (16 rows x 8 k) of a row-major fp32 matrix with row stride `ld`.
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const float* m, int ld, int lane) {
    const int g = lane >> 2, t = lane & 3;
    a[0] = f32_to_tf32(m[g * ld + t]);
    a[1] = f32_to_tf32(m[(g + 8) * ld + t]);
    a[2] = f32_to_tf32(m[g * ld + t + 4]);
    a[3] = f32_to_tf32(m[(g + 8) * ld + t + 4]);
}
// B fragment (8 k x 8 n) of a row-major fp32 matrix B[k][n] with row stride `ld`.
__device__ __forceinline__ void load_b_frag(uint32_t (&b)[2], const float* m, int ld, int lane) {
    const int g = lane >> 2, t = lane & 3;
    b[0] = f32_to_tf32(m[t * ld + g]);
    b[1] = f32_to_tf32(m[(t + 4) * ld + g]);
}
// Store an accumulator fragment (16 x 8), optionally negated.
__device__ __forceinline__ void store_c_frag(float* m, int ld, int lane, const float (&c)[4], float sign) {
    const int g = lane >> 2, t = lane & 3;
    *reinterpret_cast<float2*>(m + g * ld + 2 * t) = make_float2(sign * c[0], sign * c[1]);
    *reinterpret_cast<float2*>(m + (g + 8) * ld + 2 * t) = make_float2(sign * c[2], sign * c[3]);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Mask epilogue, one exponential per element.  The pairwise decay exp(gamma_i - gamma_j) for j <= i is
// 2^(g_i - g_j) with the cumsum kept in log2 units; the argument is <= 0 wherever the value is used, and what lies
// above the diagonal is selected away, never multiplied.  With L2 normalisation the column table ps.ctab[0] carries
// g_j - log2(1/|k_j|) (the caller fills it), so the same exponential also applies 1/|k_j|.
// Thread = row i = one TMEM lane; `trow` = tensor-memory address of column 0 of the warp's lanes; low_rows (warp-uniform):
// the warp's rows are 0-31, whose columns 32-63 lie above the diagonal.

// Raw K K^T row -> row i of A = tril(beta_i * decay * K K^T, -1), fp32, into `As` (columns 32-63 of rows 0-31 are
// not written: the inverse never reads them).  Returns |k_i|^2 (the diagonal entry) when want_ksq.
__device__ __forceinline__ float prep_mask_row_A(const PrepScratch& ps, bool l2norm, uint32_t trow, int i, bool low_rows,
                                                 float* As, bool want_ksq) {
    const float* gcol = l2norm ? ps.ctab[0] : ps.gam;
    const float gi = ps.gam[i];
    const float bi = l2norm ? ps.bet[i] * ps.rn[i] : ps.bet[i];
    float ksq = 0.f;
    uint32_t r[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        if (half == 1 && low_rows) break;
        tmem_ld_x32(trow + half * 32, r);
        tmem_ld_wait();
        if (want_ksq && (i >> 5) == half) {
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c == (i & 31)) ksq = __uint_as_float(r[c]);
        }
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float4 gj = *reinterpret_cast<const float4*>(gcol + half * 32 + c);
            float4 o;
            o.x = (half * 32 + c + 0 < i) ? bi * fast_exp2(gi - gj.x) * __uint_as_float(r[c + 0]) : 0.f;
            o.y = (half * 32 + c + 1 < i) ? bi * fast_exp2(gi - gj.y) * __uint_as_float(r[c + 1]) : 0.f;
            o.z = (half * 32 + c + 2 < i) ? bi * fast_exp2(gi - gj.z) * __uint_as_float(r[c + 2]) : 0.f;
            o.w = (half * 32 + c + 3 < i) ? bi * fast_exp2(gi - gj.w) * __uint_as_float(r[c + 3]) : 0.f;
            *reinterpret_cast<float4*>(As + i * kSolveStride + half * 32 + c) = o;
        }
    }
    return ksq;
}

// max over the warp's rows of beta_i |k_i|^2 (the premise of the decay bound for split sequences), +inf when a gate
// of the row is outside beta >= 0, g <= 0.  ksq: the raw diagonal entry of K K^T.
__device__ __forceinline__ float prep_bound_of_rows(const PrepScratch& ps, bool l2norm, int i, float ksq) {
    const float rk = l2norm ? ps.rn[i] : 1.f;
    const bool in_range = ps.bet[i] >= 0.f && ps.gam[i] <= (i > 0 ? ps.gam[i - 1] : 0.f);
    float bound = in_range ? ps.bet[i] * ksq * rk * rk : INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, o));
    return bound;
}

// Raw Q K^T row -> row i of P = tril(scale * decay * Q K^T) as 64 bf16 values in registers (eight 16-byte chunks).
// The row factor (positive) travels in the exponent.
__device__ __forceinline__ void prep_mask_row_P_packed(const PrepScratch& ps, bool l2norm, float scale0, uint32_t trow,
                                                       int i, bool low_rows, uint4 (&pk)[8]) {
    const float* gcol = l2norm ? ps.ctab[0] : ps.gam;
    const float gis = ps.gam[i] + __log2f(l2norm ? scale0 * ps.rn[kChunk + i] : scale0);
    uint32_t r[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        if (half == 1 && low_rows) {               // above the diagonal: zeros
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) pk[4 + ch] = make_uint4(0, 0, 0, 0);
            break;
        }
        tmem_ld_x32(trow + half * 32, r);
        tmem_ld_wait();
        float x[32];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float4 gj = *reinterpret_cast<const float4*>(gcol + half * 32 + c);
            x[c + 0] = (half * 32 + c + 0 <= i) ? fast_exp2(gis - gj.x) * __uint_as_float(r[c + 0]) : 0.f;
            x[c + 1] = (half * 32 + c + 1 <= i) ? fast_exp2(gis - gj.y) * __uint_as_float(r[c + 1]) : 0.f;
            x[c + 2] = (half * 32 + c + 2 <= i) ? fast_exp2(gis - gj.z) * __uint_as_float(r[c + 2]) : 0.f;
            x[c + 3] = (half * 32 + c + 3 <= i) ? fast_exp2(gis - gj.w) * __uint_as_float(r[c + 3]) : 0.f;
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            pk[4 * half + ch].x = pack_bf16x2(x[8 * ch + 0], x[8 * ch + 1]);
            pk[4 * half + ch].y = pack_bf16x2(x[8 * ch + 2], x[8 * ch + 3]);
            pk[4 * half + ch].z = pack_bf16x2(x[8 * ch + 4], x[8 * ch + 5]);
            pk[4 * half + ch].w = pack_bf16x2(x[8 * ch + 6], x[8 * ch + 7]);
        }
    }
}

// The same row, straight to the workspace (`prow`: 64 values).
__device__ __forceinline__ void prep_mask_row_P(const PrepScratch& ps, bool l2norm, float scale0, uint32_t trow, int i,
                                                bool low_rows, __nv_bfloat16* prow) {
    uint4 pk[8];
    prep_mask_row_P_packed(ps, l2norm, scale0, trow, i, low_rows, pk);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(prow + 8 * ch) = pk[ch];
}

// Blocked inversion of T = (I + A)^-1 for the strictly lower-triangular 64x64 A in `As` (fp32, row stride
// kSolveStride), result in `Tm` (same layout):
//   8x8 diagonal blocks by forward substitution in fp32 registers, then
//   [[L11,0],[L21,L22]]^-1 = [[X11,0],[-X22 L21 X11, X22]] at block size 8 in fp32 and at block sizes 16 and 32 with
//   TF32 warp MMAs.
// Everything up to the two 32x32 diagonal blocks involves only 32 consecutive rows, so ONE WARP does it for the rows
// it owns with no CTA-level barrier (prep_invert_diag32); only the last level crosses (prep_invert_level2).

// One warp: the 32x32 diagonal block p (rows and columns 32p .. 32p+31) of T, zeros above its diagonal included.
// Needs rows 32p .. 32p+31 of `As` visible to the warp (after the warp's own writes a __syncwarp is enough).
// `y`: kDiagScratch floats of scratch of its own.
__device__ __forceinline__ void prep_invert_diag32(const float* As, float* Tm, float* y, int p, int lane) {
    {   // four 8x8 diagonal blocks: lane = (block, column), forward substitution in registers
        const int blk = 4 * p + (lane >> 3), c = lane & 7;
        const float* a = As + (8 * blk) * kSolveStride + 8 * blk;
        float4 rowv[7][2];
#pragma unroll
        for (int i = 1; i < 8; ++i)
#pragma unroll
            for (int q = 0; q < 2; ++q)
                if (4 * q < i) rowv[i - 1][q] = *reinterpret_cast<const float4*>(a + i * kSolveStride + 4 * q);
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (i == c) ? 1.f : 0.f;
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            float acc0 = x[i], acc1 = 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) {
                const float4 v4 = rowv[i - 1][j >> 2];
                const float aij = (j & 3) == 0 ? v4.x : ((j & 3) == 1 ? v4.y : ((j & 3) == 2 ? v4.z : v4.w));
                if (j & 1) acc1 = fmaf(-aij, x[j], acc1);
                else acc0 = fmaf(-aij, x[j], acc0);
            }
            x[i] = acc0 + acc1;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) Tm[(8 * blk + i) * kSolveStride + 8 * blk + c] = x[i];
        // zeros in the upper-right 8x8 of the two 16x16 diagonal blocks (one float4 per lane) ...
        const int b16 = 2 * p + (lane >> 4), r = (lane >> 1) & 7, q = lane & 1;
        *reinterpret_cast<float4*>(Tm + (16 * b16 + r) * kSolveStride + 16 * b16 + 8 + 4 * q) = make_float4(0.f, 0.f, 0.f, 0.f);
        // ... and in the upper-right 16x16 of the 32x32 block (two per lane; rows r0 and r0 + 4 share a quarter-warp, which
        // keeps the 16-byte stores off each other's banks)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int q4 = lane & 3, rr = ((lane >> 2) & 1) * 4 + (lane >> 3) + 8 * e;
            *reinterpret_cast<float4*>(Tm + (32 * p + rr) * kSolveStride + 32 * p + 16 + 4 * q4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncwarp();
    {   // 8 -> 16 in fp32: X21 = -X22 (A21 X11).  lane = (16-block, row r, four columns c0 ..) of the 8x8 result; the
        // block index is the lowest lane bit and the blocks' temporaries lie 72 floats apart, which keeps the lanes of a
        // quarter-warp on different banks in the row reads, the temporaries' reads and the result's stores
        const int b16 = 2 * p + (lane & 1), r = (lane >> 1) & 7, c0 = 4 * (lane >> 4);
        const float* a21 = As + (16 * b16 + 8 + r) * kSolveStride + 16 * b16;
        const float* x11 = Tm + (16 * b16) * kSolveStride + 16 * b16 + c0;
        const float* x22 = Tm + (16 * b16 + 8 + r) * kSolveStride + 16 * b16 + 8;
        float* yb = y + 72 * (lane & 1);
        {
            const float4 a0 = *reinterpret_cast<const float4*>(a21), a1 = *reinterpret_cast<const float4*>(a21 + 4);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float4 xv = *reinterpret_cast<const float4*>(x11 + k * kSolveStride);
                acc.x = fmaf(av[k], xv.x, acc.x);
                acc.y = fmaf(av[k], xv.y, acc.y);
                acc.z = fmaf(av[k], xv.z, acc.z);
                acc.w = fmaf(av[k], xv.w, acc.w);
            }
            *reinterpret_cast<float4*>(yb + 8 * r + c0) = acc;
        }
        __syncwarp();
        {
            const float4 b0 = *reinterpret_cast<const float4*>(x22), b1 = *reinterpret_cast<const float4*>(x22 + 4);
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float4 yv = *reinterpret_cast<const float4*>(yb + 8 * k + c0);
                acc.x = fmaf(-bv[k], yv.x, acc.x);
                acc.y = fmaf(-bv[k], yv.y, acc.y);
                acc.z = fmaf(-bv[k], yv.z, acc.z);
                acc.w = fmaf(-bv[k], yv.w, acc.w);
            }
            *reinterpret_cast<float4*>(Tm + (16 * b16 + 8 + r) * kSolveStride + 16 * b16 + c0) = acc;
        }
    }
    __syncwarp();
    {   // 16 -> 32 with TF32 warp MMAs: Y = A21 X11, X21 = -X22 Y (16 x 16 each)
        float* y1 = y;   // the 8 -> 16 temporaries are dead
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t a[4];
            load_a_frag(a, As + (32 * p + 16) * kSolveStride + 32 * p + 8 * ks, kSolveStride, lane);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                uint32_t b[2];
                load_b_frag(b, Tm + (32 * p + 8 * ks) * kSolveStride + 32 * p + 8 * nt, kSolveStride, lane);
                mma_tf32_16x8x8(acc[nt], a, b);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) store_c_frag(y1 + 8 * nt, kY1Stride, lane, acc[nt], 1.f);
        __syncwarp();
        float acc2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t a[4];
            load_a_frag(a, Tm + (32 * p + 16) * kSolveStride + 32 * p + 16 + 8 * ks, kSolveStride, lane);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                uint32_t b[2];
                load_b_frag(b, y1 + (8 * ks) * kY1Stride + 8 * nt, kY1Stride, lane);
                mma_tf32_16x8x8(acc2[nt], a, b);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
            store_c_frag(Tm + (32 * p + 16) * kSolveStride + 32 * p + 8 * nt, kSolveStride, lane, acc2[nt], -1.f);
    }
}

// All 128 threads: the 32x32 lower-left block of T, X21 = -X22 (A21 X11), from the two diagonal blocks (which must be
// complete: one barrier before).  `Yt`: 32*kY2Stride floats.  Ends with a barrier.  warp -> (16-row block rb, 16-column block cb)
__device__ __forceinline__ void prep_invert_level2(const float* As, float* Tm, float* Yt, PrepCtx ctx = PrepCtx::whole_cta()) {
    const int tid = ctx.tid, warp = tid >> 5, lane = tid & 31;
    const int rb = warp >> 1, cb = warp & 1;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        load_a_frag(a, As + (32 + 16 * rb) * kSolveStride + 8 * ks, kSolveStride, lane);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint32_t b[2];
            load_b_frag(b, Tm + (8 * ks) * kSolveStride + 16 * cb + 8 * nt, kSolveStride, lane);
            mma_tf32_16x8x8(acc[nt], a, b);
        }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
        store_c_frag(Yt + (16 * rb) * kY2Stride + 16 * cb + 8 * nt, kY2Stride, lane, acc[nt], 1.f);
    ctx.sync();
    float acc2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        load_a_frag(a, Tm + (32 + 16 * rb) * kSolveStride + 32 + 8 * ks, kSolveStride, lane);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint32_t b[2];
            load_b_frag(b, Yt + (8 * ks) * kY2Stride + 16 * cb + 8 * nt, kY2Stride, lane);
            mma_tf32_16x8x8(acc2[nt], a, b);
        }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
        store_c_frag(Tm + (32 + 16 * rb) * kSolveStride + 16 * cb + 8 * nt, kSolveStride, lane, acc2[nt], -1.f);
    ctx.sync();
}

// The whole inversion by 128 threads.  `Tm` must be zero above the 16x16 diagonal blocks on entry (the caller zeroes
// it), `As` complete (one barrier before).  `Yt`: scratch of at least 32*kY2Stride floats.
__device__ __forceinline__ void prep_invert_unit_lower(const float* As, float* Tm, float* Yt,
                                                       PrepCtx ctx = PrepCtx::whole_cta()) {
    const int warp = ctx.tid >> 5, lane = ctx.tid & 31;
    if (warp < 2) prep_invert_diag32(As, Tm, Yt + kDiagScratch * warp, warp, lane);
    ctx.sync();
    prep_invert_level2(As, Tm, Yt, ctx);
}

// Zeroes the six 16x16 blocks of `Tm` above the block diagonal (all 128 threads; what prep_invert_unit_lower
// expects on entry).
__device__ __forceinline__ void prep_zero_upper_blocks(float* Tm, PrepCtx ctx = PrepCtx::whole_cta()) {
    const int tid = ctx.tid;
#pragma unroll
    for (int e = 0; e < 3; ++e) {
        const int idx = tid + 128 * e;              // 384 float4 = 6 blocks x 16 rows x 4 float4
        const int blk = idx >> 6, r = (idx >> 2) & 15, q = idx & 3;
        const int I = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
        const int J = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);
        *reinterpret_cast<float4*>(Tm + (16 * I + r) * kSolveStride + 16 * J + 4 * q) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// Row `i` of  T diag(f)  as bf16 into row `dst_row` of a 128-byte-swizzled K-major tile
// (f = beta e^gamma gives the operand that produces W, f = beta the one that produces U).
__device__ __forceinline__ void prep_store_scaled_T_row(const float* Tm, const float* f, int i, uint8_t* tile,
                                                        uint32_t dst_row) {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const float4 t0 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8);
        const float4 t1 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8 + 4);
        const float4 f0 = *reinterpret_cast<const float4*>(f + ch * 8);
        const float4 f1 = *reinterpret_cast<const float4*>(f + ch * 8 + 4);
        uint4 pk;
        pk.x = pack_bf16x2(t0.x * f0.x, t0.y * f0.y);
        pk.y = pack_bf16x2(t0.z * f0.z, t0.w * f0.w);
        pk.z = pack_bf16x2(t1.x * f1.x, t1.y * f1.y);
        pk.w = pack_bf16x2(t1.z * f1.z, t1.w * f1.w);
        *reinterpret_cast<uint4*>(tile + swz_chunk_offset<128>(dst_row, ch)) = pk;
    }
}

// Columns [32 hh, 32 hh + 32) of row i of T, read once, as bf16 into BOTH consumers: T diag(fa) into row `dst_row` of
// a 128-byte-swizzled K-major tile and T diag(fb) into a plain row of 64 values in global memory.  The block of T
// above its two 32x32 diagonal blocks (rows 0-31, columns 32-63) is zero by definition and is not read, so that
// part of `Tm` need not be defined.  hh and i < 32 must be uniform over a warp.
__device__ __forceinline__ void prep_store_T_half_row_both(const float* Tm, const float* fa, const float* fb, int i, int hh,
                                                           uint8_t* tile, uint32_t dst_row, __nv_bfloat16* grow) {
    if (hh == 1 && i < 32) {
#pragma unroll
        for (int ch = 4; ch < 8; ++ch) {
            *reinterpret_cast<uint4*>(tile + swz_chunk_offset<128>(dst_row, ch)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(grow + ch * 8) = make_uint4(0, 0, 0, 0);
        }
        return;
    }
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
        const int ch = 4 * hh + c4;
        const float4 t0 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8);
        const float4 t1 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8 + 4);
        const float4 a0 = *reinterpret_cast<const float4*>(fa + ch * 8), a1 = *reinterpret_cast<const float4*>(fa + ch * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(fb + ch * 8), b1 = *reinterpret_cast<const float4*>(fb + ch * 8 + 4);
        uint4 pa, pb;
        pa.x = pack_bf16x2(t0.x * a0.x, t0.y * a0.y);
        pa.y = pack_bf16x2(t0.z * a0.z, t0.w * a0.w);
        pa.z = pack_bf16x2(t1.x * a1.x, t1.y * a1.y);
        pa.w = pack_bf16x2(t1.z * a1.z, t1.w * a1.w);
        pb.x = pack_bf16x2(t0.x * b0.x, t0.y * b0.y);
        pb.y = pack_bf16x2(t0.z * b0.z, t0.w * b0.w);
        pb.z = pack_bf16x2(t1.x * b1.x, t1.y * b1.y);
        pb.w = pack_bf16x2(t1.z * b1.z, t1.w * b1.w);
        *reinterpret_cast<uint4*>(tile + swz_chunk_offset<128>(dst_row, ch)) = pa;
        *reinterpret_cast<uint4*>(grow + ch * 8) = pb;
    }
}

// The same with T diag(fb) into row `row_b` of a second 128-byte-swizzled tile in shared memory (a staging tile that a
// TMA store takes to global memory: a row per thread written straight to global memory costs a wavefront per lane).
__device__ __forceinline__ void prep_store_T_half_row_tiles(const float* Tm, const float* fa, const float* fb, int i, int hh,
                                                            uint8_t* tile_a, uint32_t row_a, uint8_t* tile_b, uint32_t row_b) {
    if (hh == 1 && i < 32) {
#pragma unroll
        for (int ch = 4; ch < 8; ++ch) {
            *reinterpret_cast<uint4*>(tile_a + swz_chunk_offset<128>(row_a, ch)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(tile_b + swz_chunk_offset<128>(row_b, ch)) = make_uint4(0, 0, 0, 0);
        }
        return;
    }
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
        const int ch = 4 * hh + c4;
        const float4 t0 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8);
        const float4 t1 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8 + 4);
        const float4 a0 = *reinterpret_cast<const float4*>(fa + ch * 8), a1 = *reinterpret_cast<const float4*>(fa + ch * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(fb + ch * 8), b1 = *reinterpret_cast<const float4*>(fb + ch * 8 + 4);
        uint4 pa, pb;
        pa.x = pack_bf16x2(t0.x * a0.x, t0.y * a0.y);
        pa.y = pack_bf16x2(t0.z * a0.z, t0.w * a0.w);
        pa.z = pack_bf16x2(t1.x * a1.x, t1.y * a1.y);
        pa.w = pack_bf16x2(t1.z * a1.z, t1.w * a1.w);
        pb.x = pack_bf16x2(t0.x * b0.x, t0.y * b0.y);
        pb.y = pack_bf16x2(t0.z * b0.z, t0.w * b0.w);
        pb.z = pack_bf16x2(t1.x * b1.x, t1.y * b1.y);
        pb.w = pack_bf16x2(t1.z * b1.z, t1.w * b1.w);
        *reinterpret_cast<uint4*>(tile_a + swz_chunk_offset<128>(row_a, ch)) = pa;
        *reinterpret_cast<uint4*>(tile_b + swz_chunk_offset<128>(row_b, ch)) = pb;
    }
}

// Row `i` of  T diag(f)  as bf16 into a plain row-major row of 64 values in global memory (16-byte stores).
__device__ __forceinline__ void prep_store_scaled_T_row_plain(const float* Tm, const float* f, int i, __nv_bfloat16* dst) {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const float4 t0 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8);
        const float4 t1 = *reinterpret_cast<const float4*>(Tm + i * kSolveStride + ch * 8 + 4);
        const float4 f0 = *reinterpret_cast<const float4*>(f + ch * 8);
        const float4 f1 = *reinterpret_cast<const float4*>(f + ch * 8 + 4);
        uint4 pk;
        pk.x = pack_bf16x2(t0.x * f0.x, t0.y * f0.y);
        pk.y = pack_bf16x2(t0.z * f0.z, t0.w * f0.w);
        pk.z = pack_bf16x2(t1.x * f1.x, t1.y * f1.y);
        pk.w = pack_bf16x2(t1.z * f1.z, t1.w * f1.w);
        *reinterpret_cast<uint4*>(dst + ch * 8) = pk;
    }
}

}  // namespace gdn
