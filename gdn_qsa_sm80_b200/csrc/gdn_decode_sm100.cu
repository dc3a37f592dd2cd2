// Token-by-token gated delta rule for very short sequences (decode: one or a few new tokens per sequence on top
// of a stored state).  Same recurrence as the reference's recurrent torch definition
// (gdn_qsa_sm80/reference/gdn_chunk_ref.py:133-141), fp32 throughout:
//     S <- exp(g) S ;  delta = beta (v - S^T k) ;  S <- S + k delta^T ;  o = S^T q / sqrt(D)
// With one token the operator is nothing but a read and a write of the 64 KB state per (batch, value head), so
// the kernel is laid out for HBM: a CTA of 256 threads owns one state; warp w holds rows w, w+8, ... (16 rows),
// lane l the four columns 4l..4l+3 of each, so every load and store is a whole 512-byte row per warp and a thread
// keeps 16 independent 16-byte loads in flight; two CTAs per SM.  The two column sums a token needs (S^T k and
// S^T q) are partial per warp and meet in shared memory.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int kDecThreads = 256, kDecWarps = 8, kRowsPerWarp = kD / kDecWarps;

template <bool GATE_F32>
__device__ __forceinline__ float dec_gate(const void* p, size_t idx) {
    if (GATE_F32) return static_cast<const float*>(p)[idx];
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

template <bool GATE_F32>
__global__ void __launch_bounds__(kDecThreads, 2) gdn_decode_kernel(Problem p) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x / p.Hv, h = blockIdx.x % p.Hv;
    const int hq = h / (p.Hv / p.Hq);
    const float scale = rsqrtf(static_cast<float>(kD));
    __shared__ float ks[kD], qs[kD];
    __shared__ __align__(16) float part[2][kDecWarps][kD];

    const size_t st_base = (static_cast<size_t>(b) * p.Hv + h) * kD * kD;
    float4 st[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
        const int r = warp + kDecWarps * i;
        st[i] = p.h0 ? *reinterpret_cast<const float4*>(p.h0 + st_base + static_cast<size_t>(r) * kD + 4 * lane)
                     : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s = 0; s < p.S; ++s) {
        const size_t tok = static_cast<size_t>(b) * p.S + s;
        if (tid < kD) ks[tid] = __bfloat162float(p.k[(tok * p.Hq + hq) * kD + tid]);
        else qs[tid - kD] = __bfloat162float(p.q[(tok * p.Hq + hq) * kD + tid - kD]) * scale;
        float gt = dec_gate<GATE_F32>(p.g, tok * p.Hv + h), bt = dec_gate<GATE_F32>(p.beta, tok * p.Hv + h);
        if (p.gate_act) {   // raw gates: g = -softplus(.), beta = sigmoid(.)
            gt = gt > 20.f ? -gt : -log1pf(__expf(gt));
            bt = 1.f / (1.f + __expf(-bt));
        }
        const float dec = __expf(gt);
        const uint2 vraw = *reinterpret_cast<const uint2*>(p.v + (tok * p.Hv + h) * kD + 4 * lane);
        __syncthreads();
        float rk = 1.f, rq = 1.f;
        if (p.l2norm) {   // every warp sums the squares itself: the vectors are in shared memory anyway
            const float4 k4 = *reinterpret_cast<const float4*>(ks + 4 * lane), q4 = *reinterpret_cast<const float4*>(qs + 4 * lane);
            float kk = k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w;
            float qq = q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                kk += __shfl_xor_sync(0xffffffffu, kk, o);
                qq += __shfl_xor_sync(0xffffffffu, qq, o);
            }
            rk = rsqrtf(kk + 1e-6f);
            rq = rsqrtf(qq / (scale * scale) + 1e-6f);   // qs holds q * scale
        }
        // S^T k, this warp's rows
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
            const float kr = ks[warp + kDecWarps * i];
            acc.x = fmaf(st[i].x, kr, acc.x); acc.y = fmaf(st[i].y, kr, acc.y);
            acc.z = fmaf(st[i].z, kr, acc.z); acc.w = fmaf(st[i].w, kr, acc.w);
        }
        *reinterpret_cast<float4*>(&part[0][warp][4 * lane]) = acc;
        __syncthreads();
        float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float4 x = *reinterpret_cast<const float4*>(&part[0][w][4 * lane]);
            kv.x += x.x; kv.y += x.y; kv.z += x.z; kv.w += x.w;
        }
        const float f = dec * rk, bk = bt * rk;
        float4 dl;   // delta = beta (v - (decayed S)^T k), with the key's norm folded in
        dl.x = (__uint_as_float(vraw.x << 16) - kv.x * f) * bk;
        dl.y = (__uint_as_float(vraw.x & 0xffff0000u) - kv.y * f) * bk;
        dl.z = (__uint_as_float(vraw.y << 16) - kv.z * f) * bk;
        dl.w = (__uint_as_float(vraw.y & 0xffff0000u) - kv.w * f) * bk;
        float4 oa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
            const float kr = ks[warp + kDecWarps * i], qr = qs[warp + kDecWarps * i];
            st[i].x = fmaf(kr, dl.x, dec * st[i].x); st[i].y = fmaf(kr, dl.y, dec * st[i].y);
            st[i].z = fmaf(kr, dl.z, dec * st[i].z); st[i].w = fmaf(kr, dl.w, dec * st[i].w);
            oa.x = fmaf(st[i].x, qr, oa.x); oa.y = fmaf(st[i].y, qr, oa.y);
            oa.z = fmaf(st[i].z, qr, oa.z); oa.w = fmaf(st[i].w, qr, oa.w);
        }
        *reinterpret_cast<float4*>(&part[1][warp][4 * lane]) = oa;
        __syncthreads();
        if (warp == 0) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) {
                const float4 x = *reinterpret_cast<const float4*>(&part[1][w][4 * lane]);
                o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
            }
            const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * rq, o.y * rq), hi = __floats2bfloat162_rn(o.z * rq, o.w * rq);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(p.out + (tok * p.Hv + h) * kD + 4 * lane) = pk;
        }
    }
    if (p.hT) {
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
            const int r = warp + kDecWarps * i;
            *reinterpret_cast<float4*>(p.hT + st_base + static_cast<size_t>(r) * kD + 4 * lane) = st[i];
        }
    }
}

}  // namespace

cudaError_t launch_decode(const Problem& p, cudaStream_t stream) {
    const dim3 grid(p.B * p.Hv), block(kDecThreads);
    if (p.gate_f32) gdn_decode_kernel<true><<<grid, block, 0, stream>>>(p);
    else gdn_decode_kernel<false><<<grid, block, 0, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

}  // namespace gdn
