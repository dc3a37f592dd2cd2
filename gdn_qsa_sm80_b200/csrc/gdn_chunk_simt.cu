// Token-by-token gated delta rule in fp32 on CUDA cores.
//
// This is the exact (unchunked) form of the operator, the one the reference's torch function
// torch_recurrent_gated_delta_rule defines (gdn_qsa_sm80/reference/gdn_chunk_ref.py:133-141):
//     S <- exp(g_t) S ;  delta = beta_t (v_t - S^T k_t) ;  S <- S + k_t delta^T ;  o_t = S^T (q_t / sqrt(D))
// Thread c of a 128-thread CTA owns column c of the 128x128 state in registers, so every step of
// the recurrence is thread-local and the only shared data are the token's k and q vectors.
// It needs no scratch and no tensor cores; it exists as an independent on-device check of the
// fused tcgen05 path and as a path that works for any shape.
#include "gdn_common.cuh"

namespace gdn {

template <bool GATE_F32>
__device__ __forceinline__ float load_gate(const void* p, size_t idx) {
    if (GATE_F32) return static_cast<const float*>(p)[idx];
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

template <bool GATE_F32>
__global__ void __launch_bounds__(128) gdn_recurrent_simt_kernel(Problem p) {
    const int c = threadIdx.x;
    const int b = blockIdx.x / p.Hv, h = blockIdx.x % p.Hv;
    const int hq = h / (p.Hv / p.Hq);
    const float scale = rsqrtf(static_cast<float>(kD));
    __shared__ float ks[2][kD];
    __shared__ float qs[2][kD];

    float st[kD];
    const size_t st_base = (static_cast<size_t>(b) * p.Hv + h) * kD * kD;
#pragma unroll
    for (int r = 0; r < kD; ++r) st[r] = p.h0 ? p.h0[st_base + static_cast<size_t>(r) * kD + c] : 0.f;

    // software pipeline: the next token's operands are in flight while this token is processed
    float k_n = 0.f, q_n = 0.f, v_n = 0.f, g_n = 0.f, b_n = 0.f;
    auto fetch = [&](int i) {
        const size_t tok = static_cast<size_t>(b) * p.S + i;
        k_n = __bfloat162float(p.k[(tok * p.Hq + hq) * kD + c]);
        q_n = __bfloat162float(p.q[(tok * p.Hq + hq) * kD + c]);
        v_n = __bfloat162float(p.v[(tok * p.Hv + h) * kD + c]);
        g_n = load_gate<GATE_F32>(p.g, tok * p.Hv + h);
        b_n = load_gate<GATE_F32>(p.beta, tok * p.Hv + h);
    };
    if (p.S > 0) fetch(0);
    for (int i = 0; i < p.S; ++i) {
        const int buf = i & 1;
        ks[buf][c] = k_n;
        qs[buf][c] = q_n * scale;
        float gt = g_n, bt = b_n;
        if (p.gate_act) {   // raw gates: g = -softplus(.), beta = sigmoid(.)
            gt = gt > 20.f ? -gt : -log1pf(__expf(gt));
            bt = 1.f / (1.f + __expf(-bt));
        }
        const float vi = v_n, dec = __expf(gt);
        if (i + 1 < p.S) fetch(i + 1);
        __syncthreads();
        float kv = 0.f, rk = 1.f, rq = 1.f;
        if (p.l2norm) {   // every thread sums the squares itself: the vectors are in shared memory anyway
            float kk = 0.f, qq = 0.f;
#pragma unroll
            for (int r = 0; r < kD; ++r) {
                kk = fmaf(ks[buf][r], ks[buf][r], kk);
                qq = fmaf(qs[buf][r], qs[buf][r], qq);
            }
            rk = rsqrtf(kk + 1e-6f);
            rq = rsqrtf(qq / (scale * scale) + 1e-6f);   // qs holds q * scale
        }
#pragma unroll
        for (int r = 0; r < kD; ++r) {
            st[r] *= dec;
            kv = fmaf(st[r], ks[buf][r], kv);
        }
        const float dl = (vi - kv * rk) * bt * rk;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < kD; ++r) {
            st[r] = fmaf(ks[buf][r], dl, st[r]);
            o = fmaf(st[r], qs[buf][r], o);
        }
        o *= rq;
        p.out[((static_cast<size_t>(b) * p.S + i) * p.Hv + h) * kD + c] = __float2bfloat16(o);
    }
    if (p.hT) {
#pragma unroll
        for (int r = 0; r < kD; ++r) p.hT[st_base + static_cast<size_t>(r) * kD + c] = st[r];
    }
}

cudaError_t launch_simt(const Problem& p, cudaStream_t stream) {
    const dim3 grid(p.B * p.Hv), block(128);
    if (p.gate_f32) gdn_recurrent_simt_kernel<true><<<grid, block, 0, stream>>>(p);
    else gdn_recurrent_simt_kernel<false><<<grid, block, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace gdn
