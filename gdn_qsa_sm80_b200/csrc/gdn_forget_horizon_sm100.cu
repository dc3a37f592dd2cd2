// After how many leading chunks has EVERY (batch, value head) of a stretch of tokens forgotten the state it started
// from?  By the decay bound of the split sequences (||A||_2 <= exp(sum of g) when 0 <= beta |k|^2 <= 2 and g <= 0)
// that is the first chunk c with  sum_{t < 64 (c + 1)} g[b][t][h] < -115  for all b, h.  The sequence-parallel driver
// asks this once per call and reads the answer on the host while its first pass is running, so the question has to
// cost microseconds: one streaming pass over g and beta (a warp per chunk, a lane per head, whole rows of heads per
// load) that leaves the per-chunk sums and checks the gates' ranges, then one tiny kernel that walks each head's sums
// until they cross the threshold.  The premise on the keys comes from gdn_key_norm_sq_max_sm100.
// The reference decides its "reset" path from a measured max |A| instead (csrc/gdn_chunk/gdn_scan_stage3_reset.cu:22-54).
#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int kHzThreads = 256;

template <bool GATE_F32>
__device__ __forceinline__ float hz_load(const void* p, size_t idx) {
    if (GATE_F32) return static_cast<const float*>(p)[idx];
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

// flags[0]: bits of max beta (non-negative floats order like their bit patterns); flags[1]: 1 if a gate is out of range
// (g > 0, beta < 0, or not a number).
template <bool GATE_F32>
__global__ void __launch_bounds__(kHzThreads) gdn_chunk_gate_sums_kernel(const void* __restrict__ g,
                                                                        const void* __restrict__ beta, int B, int S, int Hv,
                                                                        int NT, float* __restrict__ sums, int* flags) {
    const int lane = threadIdx.x & 31, warps = kHzThreads / 32;
    const long long units = static_cast<long long>(B) * NT;
    float bmax = 0.f;
    bool bad = false;
    for (long long u = static_cast<long long>(blockIdx.x) * warps + (threadIdx.x >> 5); u < units;
         u += static_cast<long long>(gridDim.x) * warps) {
        const int b = static_cast<int>(u / NT), c = static_cast<int>(u % NT);
        const int t0 = c * kChunk, t1 = min(S, t0 + kChunk);
        for (int h = lane; h < Hv; h += 32) {
            float s0 = 0.f, s1 = 0.f;
            const size_t base = (static_cast<size_t>(b) * S + t0) * Hv + h;
            int t = 0;
            for (; t + 1 < t1 - t0; t += 2) {
                const float g0 = hz_load<GATE_F32>(g, base + static_cast<size_t>(t) * Hv);
                const float g1 = hz_load<GATE_F32>(g, base + static_cast<size_t>(t + 1) * Hv);
                const float b0 = hz_load<GATE_F32>(beta, base + static_cast<size_t>(t) * Hv);
                const float b1 = hz_load<GATE_F32>(beta, base + static_cast<size_t>(t + 1) * Hv);
                s0 += g0;
                s1 += g1;
                bad = bad || !(g0 <= 0.f) || !(g1 <= 0.f) || !(b0 >= 0.f) || !(b1 >= 0.f);
                bmax = fmaxf(bmax, fmaxf(b0, b1));
            }
            if (t < t1 - t0) {
                const float g0 = hz_load<GATE_F32>(g, base + static_cast<size_t>(t) * Hv);
                const float b0 = hz_load<GATE_F32>(beta, base + static_cast<size_t>(t) * Hv);
                s0 += g0;
                bad = bad || !(g0 <= 0.f) || !(b0 >= 0.f);
                bmax = fmaxf(bmax, b0);
            }
            sums[u * Hv + h] = s0 + s1;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, o));
    const bool any_bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) {
        if (bmax > 0.f) atomicMax(&flags[0], __float_as_int(bmax));
        if (any_bad) atomicOr(&flags[1], 1);
    }
}

// One thread per (batch, head): the first chunk after which its sum of g is below the threshold; the answer is the
// latest of them.  result[0] = that chunk (NT when some head never gets there), result[1] = 1 when the premise holds.
__global__ void __launch_bounds__(kHzThreads) gdn_forget_chunk_kernel(const float* __restrict__ sums, const int* flags,
                                                                     const float* kk_max, int B, int Hv, int NT,
                                                                     int* result) {
    const long long idx = static_cast<long long>(blockIdx.x) * kHzThreads + threadIdx.x;
    if (idx < static_cast<long long>(B) * Hv) {
        const int b = static_cast<int>(idx / Hv), h = static_cast<int>(idx % Hv);
        const float* s = sums + static_cast<size_t>(b) * NT * Hv + h;
        float acc = 0.f;
        int first = NT;
        for (int c = 0; c < NT; ++c) {
            acc += s[static_cast<size_t>(c) * Hv];
            if (acc < kForgetLn) {
                first = c;
                break;
            }
        }
        atomicMax(&result[0], first);
    }
    if (idx == 0) {
        const float kk = kk_max ? *kk_max : 1.f;
        const float bmax = __int_as_float(flags[0]);
        result[1] = (flags[1] == 0 && kk * bmax <= 2.f) ? 1 : 0;   // false for a NaN key norm as well
    }
}

}  // namespace
}  // namespace gdn

extern "C" int gdn_forgetting_horizon_sm100(const void* g, const void* beta, int gate_dtype, int B, int S, int Hv,
                                            const float* kk_max, float* scratch, int* result, void* stream_) {
    using namespace gdn;
    if (B <= 0 || S <= 0 || Hv <= 0 || !g || !beta || !scratch || !result) return GDN_ERR_BAD_ARGUMENT;
    if (gate_dtype != GDN_GATE_BF16 && gate_dtype != GDN_GATE_F32) return GDN_ERR_BAD_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int NT = (S + kChunk - 1) / kChunk;
    float* sums = scratch;
    int* flags = reinterpret_cast<int*>(scratch + static_cast<size_t>(B) * NT * Hv);
    if (cudaMemsetAsync(flags, 0, 2 * sizeof(int), stream) != cudaSuccess) return GDN_ERR_CUDA;
    if (cudaMemsetAsync(result, 0, 2 * sizeof(int), stream) != cudaSuccess) return GDN_ERR_CUDA;
    const long long units = static_cast<long long>(B) * NT, warps = kHzThreads / 32;
    long long blocks = (units + warps - 1) / warps;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (gate_dtype == GDN_GATE_F32)
        gdn_chunk_gate_sums_kernel<true><<<static_cast<unsigned>(blocks), kHzThreads, 0, stream>>>(g, beta, B, S, Hv, NT, sums, flags);
    else
        gdn_chunk_gate_sums_kernel<false><<<static_cast<unsigned>(blocks), kHzThreads, 0, stream>>>(g, beta, B, S, Hv, NT, sums, flags);
    count_launch();
    const long long heads = static_cast<long long>(B) * Hv;
    gdn_forget_chunk_kernel<<<static_cast<unsigned>((heads + kHzThreads - 1) / kHzThreads), kHzThreads, 0, stream>>>(
        sums, flags, kk_max, B, Hv, NT, result);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
}
