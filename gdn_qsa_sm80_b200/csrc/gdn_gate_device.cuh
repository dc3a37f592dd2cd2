// Device pieces of the gated RMS normalisation, kept apart from the kernel so that a fused epilogue can reuse
// them and produce the same bits.
//   out[r, :] = y[r, :] * rsqrt(mean(y[r, :]^2) + eps) * weight[:] * silu(z[r, :]),   rows of 128 bf16 values
// (the reference's rmsnorm_gated, csrc/output_gate/output_gate.cu:47-98).
// Sixteen lanes own one row, eight consecutive columns each; a warp therefore works on two rows at a time and
// all 32 lanes must call gate_row_slice together (it shuffles inside each half-warp).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace gdn {

__device__ __forceinline__ void gate_unpack8(const uint4& v, float (&x)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        x[2 * e] = __uint_as_float(w[e] << 16);
        x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint32_t gate_pack2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// yv, zv: this lane's eight values of its row of y and z; w: its eight weights.  Rows that do not exist are
// passed as zeros (their result is not stored).
__device__ __forceinline__ uint4 gate_row_slice(const uint4& yv, const uint4& zv, const float (&w)[8], float eps) {
    float a[8], g[8];
    gate_unpack8(yv, a);
    gate_unpack8(zv, g);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(a[e], a[e], ss);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // stays inside the 16 lanes of the row
    const float rstd = rsqrtf(ss * (1.f / 128.f) + eps);
    float o8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        // fast division (reciprocal + multiply, 2 ulp): the exact one costs several times the instructions and made
        // the kernel issue-bound (70 % of issue slots) instead of memory-bound; the result is rounded to bf16 anyway
        const float silu = __fdividef(g[e], 1.f + __expf(-g[e]));
        o8[e] = a[e] * (rstd * w[e]) * silu;
    }
    uint4 pk;
    pk.x = gate_pack2(o8[0], o8[1]);
    pk.y = gate_pack2(o8[2], o8[3]);
    pk.z = gate_pack2(o8[4], o8[5]);
    pk.w = gate_pack2(o8[6], o8[7]);
    return pk;
}

}  // namespace gdn
