// Second level of the two-level chunk scan: combine per-group affine state transfers.
//
// A long sequence is cut into G groups of chunks.  Group g maps its incoming state to its outgoing
// state by  S_out = A_g S_in + B_g  (A_g, B_g: 128x128 fp32 per value head; B_g is the group's final
// state from a zero start, A_g its final state from an identity start with zero values).  This
// kernel walks the groups of one sequence in order and writes the state every group starts from,
// plus the final state.  It is the exact counterpart of the reference's affine prefix scan over
// (A_g, B_g) (csrc/gdn_chunk/gdn_scan_stage2.cu:4-10, :73-220), which runs in bf16 with mma.sync;
// here it is a short fp32 CUDA-core loop (G is small, the work is 2*G*128^3 flops per head and
// HBM-bound on the 64 KB transfer tiles), so the chained state stays fp32 end to end.
//
// One CTA per (sequence, 32-column slice): thread (r, c) owns rows r, r+4, ... of column c.
#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int kScanCols = 32;

__global__ void __launch_bounds__(128) gdn_scan_transfers_kernel(const float* __restrict__ A, const float* __restrict__ Bm,
                                                                 const float* __restrict__ h0, float* __restrict__ s_in,
                                                                 float* __restrict__ s_final, int G) {
    __shared__ float S[kD][kScanCols + 1];
    const int seq = blockIdx.y, c0 = blockIdx.x * kScanCols;
    const int c = threadIdx.x & 31, r0 = threadIdx.x >> 5;   // 4 row groups
    const size_t mat = static_cast<size_t>(kD) * kD;
    for (int r = r0; r < kD; r += 4) S[r][c] = h0 ? h0[seq * mat + static_cast<size_t>(r) * kD + c0 + c] : 0.f;
    __syncthreads();
    for (int g = 0; g < G; ++g) {
        const size_t base = (static_cast<size_t>(seq) * G + g) * mat;
        float acc[kD / 4];
#pragma unroll
        for (int j = 0; j < kD / 4; ++j) {
            const int r = r0 + 4 * j;
            s_in[base + static_cast<size_t>(r) * kD + c0 + c] = S[r][c];          // the state group g starts from
            acc[j] = Bm[base + static_cast<size_t>(r) * kD + c0 + c];
        }
        for (int k = 0; k < kD; ++k) {
            const float sk = S[k][c];
#pragma unroll
            for (int j = 0; j < kD / 4; ++j) acc[j] = fmaf(A[base + static_cast<size_t>(r0 + 4 * j) * kD + k], sk, acc[j]);
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kD / 4; ++j) S[r0 + 4 * j][c] = acc[j];
        __syncthreads();
    }
    if (s_final)
        for (int r = r0; r < kD; r += 4) s_final[seq * mat + static_cast<size_t>(r) * kD + c0 + c] = S[r][c];
}

}  // namespace
}  // namespace gdn

extern "C" int gdn_chunk_scan_transfers(const float* A, const float* Bm, const float* h0, float* s_in, float* s_final,
                                        int n_seq, int G, void* stream) {
    if (!A || !Bm || !s_in || n_seq <= 0 || G <= 0 || n_seq > 65535) return GDN_ERR_BAD_ARGUMENT;
    const dim3 grid(gdn::kD / gdn::kScanCols, n_seq), block(128);
    gdn::gdn_scan_transfers_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(A, Bm, h0, s_in, s_final, G);
    gdn::count_launch();
    return cudaGetLastError() == cudaSuccess ? GDN_OK : GDN_ERR_CUDA;
}
