// max over rows of |k_row|^2 for rows of 128 bf16 values: the premise check of the decay bound used by the
// two-level and sequence-parallel drivers (||I - beta k k^T|| <= 1 needs beta |k|^2 <= 2).  One streaming pass
// over k: 16 lanes per row, one 16-byte load per lane, four rows in flight per thread; a warp folds its maxima by
// shuffles and issues one atomicMax (non-negative floats order like their bit patterns).
#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "gdn_gate_device.cuh"

namespace gdn {
namespace {

constexpr int kThreads = 512, kRows = 4, kBlocksPerSm = 2;

__global__ void __launch_bounds__(kThreads, kBlocksPerSm) gdn_key_norm_max_kernel(const uint4* __restrict__ k,
                                                                                long long n_rows, float* out_max) {
    const int sub = threadIdx.x & 15;
    const long long rows_per_block = kThreads / 16, r_in_block = threadIdx.x >> 4;
    const long long step = static_cast<long long>(gridDim.x) * rows_per_block;
    float best = 0.f;
    for (long long r0 = static_cast<long long>(blockIdx.x) * rows_per_block + r_in_block; r0 - (r_in_block & 1) < n_rows;
         r0 += step * kRows) {
        uint4 kv[kRows];
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            const long long r = r0 + u * step;
            kv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (r < n_rows) kv[u] = __ldcs(k + r * 16 + sub);
        }
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            float a[8];
            gate_unpack8(kv[u], a);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(a[e], a[e], ss);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            best = fmaxf(best, ss);
        }
    }
    best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 16));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out_max), __float_as_int(best));
}

}  // namespace
}  // namespace gdn

extern "C" int gdn_key_norm_sq_max_sm100(const void* k, long long n_rows, float* out_max, void* stream_) {
    if (n_rows < 0 || !out_max || (n_rows > 0 && !k) || (reinterpret_cast<uintptr_t>(k) & 15u)) return GDN_ERR_BAD_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaMemsetAsync(out_max, 0, sizeof(float), stream) != cudaSuccess) return GDN_ERR_CUDA;
    if (n_rows == 0) return GDN_OK;
    const long long rows_per_pass = (gdn::kThreads / 16) * gdn::kRows;
    long long blocks = (n_rows + rows_per_pass - 1) / rows_per_pass;
    const long long cap = static_cast<long long>(gdn::sm_count()) * gdn::kBlocksPerSm;
    if (blocks > cap) blocks = cap;
    gdn::gdn_key_norm_max_kernel<<<static_cast<unsigned>(blocks), gdn::kThreads, 0, stream>>>(
        static_cast<const uint4*>(k), n_rows, out_max);
    gdn::count_launch();
    return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
}
