// Diagnostic kernel: one UMMA product D = A * B^T with operands staged exactly as the fused
// gdn_chunk kernel stages them (same swizzle helper, same descriptor builder, same TMA box
// shapes), then a dump of all 128 TMEM lanes.  Used by the GPU tests to pin every
// (layout, majorness, swizzle span) combination the fused kernel relies on against a plain matmul.
#include <cuda.h>
#include <string.h>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"
#include "ptx_sm100.cuh"

namespace gdn {
namespace {

struct ProbeArgs {
    const __nv_bfloat16* a;   // thread staging: [M][K]; TMA + MN-major: [K][M]
    const __nv_bfloat16* b;   // thread staging: [N][K]; TMA + MN-major: [K][N]
    float* d;                 // [128][N]
    int* status;
    int M, N, K, a_major, b_major, b_span, use_tma;
};

constexpr uint32_t kOpBytes = 32768;   // per operand: two 16 KB groups of 128 rows x 128 B

// Byte offset of element (mn, k) of an operand tile inside its 32 KB staging area.
__device__ __forceinline__ uint32_t operand_offset(int major, int span, int mn, int k) {
    if (major == MAJOR_K)       // rows run along M/N, 64 k per 128-byte row, second k-half 16 KB further
        return (k >> 6) * 16384u + swz_chunk_offset<128>(mn, (k & 63) >> 3) + (k & 7) * 2u;
    if (span == 128)            // rows run along K, 64 mn per row, next 64 mn 16 KB further
        return (mn >> 6) * 16384u + swz_chunk_offset<128>(k, (mn & 63) >> 3) + (mn & 7) * 2u;
    return (mn >> 5) * 8192u + swz_chunk_offset<64>(k, (mn & 31) >> 3) + (mn & 7) * 2u;
}

__global__ void __launch_bounds__(128, 1)
umma_probe_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, ProbeArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sa = sm;
    uint8_t* sb = sm + kOpBytes;
    __shared__ __align__(8) uint64_t bar_tma;
    __shared__ __align__(8) uint64_t bar_mma;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 256);
        tmem_relinquish();
    }
    // zero both staging areas so rows the product does not define read as zeros
    for (uint32_t e = tid * 16; e < 2 * kOpBytes; e += 128 * 16) *reinterpret_cast<uint4*>(sm + e) = make_uint4(0, 0, 0, 0);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    bool ok = true;

    if (p.use_tma) {
        fence_proxy_async_smem();   // the zero fill above precedes the TMA writes
        __syncthreads();
        if (tid == 0) {
            const uint32_t bytes = static_cast<uint32_t>(p.M) * p.K * 2 + static_cast<uint32_t>(p.N) * p.K * 2;
            mbar_arrive_expect_tx(&bar_tma, bytes);
            if (p.a_major == MAJOR_K) {
                for (int kh = 0; kh < (p.K + 63) / 64; ++kh) tma_load_2d(sa + kh * 16384, &tm_a, &bar_tma, kh * 64, 0);
            } else {
                for (int gr = 0; gr < p.M / 64; ++gr) tma_load_2d(sa + gr * 16384, &tm_a, &bar_tma, gr * 64, 0);
            }
            if (p.b_major == MAJOR_K) {
                for (int kh = 0; kh < (p.K + 63) / 64; ++kh) tma_load_2d(sb + kh * 16384, &tm_b, &bar_tma, kh * 64, 0);
            } else if (p.b_span == 128) {
                for (int gr = 0; gr < p.N / 64; ++gr) tma_load_2d(sb + gr * 16384, &tm_b, &bar_tma, gr * 64, 0);
            } else {
                for (int gr = 0; gr < p.N / 32; ++gr) tma_load_2d(sb + gr * 8192, &tm_b, &bar_tma, gr * 32, 0);
            }
        }
        ok = mbar_wait(&bar_tma, 0, p.status, kDevTimeoutTma);
    } else {
        if (p.a_major >= 2) {
            // A goes to tensor memory: row m on lane m, k pairs packed into 32-bit columns 128 + k/2
            for (int k0 = 0; k0 < p.K; k0 += 32) {
                uint32_t r[16];
                for (int c = 0; c < 16; ++c) {
                    const __nv_bfloat16 lo = p.a[tid * p.K + k0 + 2 * c], hi = p.a[tid * p.K + k0 + 2 * c + 1];
                    r[c] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&lo)) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
                }
                tmem_st_x16(tmem_addr(tmem, warp * 32, 128 + k0 / 2), r);
            }
            tmem_st_wait();
            tc_fence_before_sync();
        } else {
            for (int e = tid; e < p.M * p.K; e += 128) {
                const int m = e / p.K, k = e % p.K;
                *reinterpret_cast<__nv_bfloat16*>(sa + operand_offset(p.a_major, 128, m, k)) = p.a[e];
            }
        }
        for (int e = tid; e < p.N * p.K; e += 128) {
            const int n = e / p.K, k = e % p.K;
            *reinterpret_cast<__nv_bfloat16*>(sb + operand_offset(p.b_major, p.b_span, n, k)) = p.b[e];
        }
        fence_proxy_async_smem();
    }
    ok = __syncthreads_and(ok);

    if (ok) {
        if (tid == 0) {
            tc_fence_after_sync();
            const uint32_t idesc = p.a_major >= 2 ? umma_idesc_bf16(p.M, p.N, MAJOR_K, p.b_major, p.a_major == 3)
                                                  : umma_idesc_bf16(p.M, p.N, p.a_major, p.b_major);
            const uint32_t a0 = smem_u32(sa), b0 = smem_u32(sb);
            for (int ks = 0; ks < p.K / 16; ++ks) {
                uint64_t ad = 0, bd;
                if (p.a_major >= 2) {}
                else if (p.a_major == MAJOR_K) ad = umma_smem_desc(a0 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                else ad = umma_smem_desc(a0 + ks * 2048, 16384, 1024, SWZ_128B);
                if (p.b_major == MAJOR_K) bd = umma_smem_desc(b0 + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, SWZ_128B);
                else if (p.b_span == 128) bd = umma_smem_desc(b0 + ks * 2048, 16384, 1024, SWZ_128B);
                else bd = umma_smem_desc(b0 + ks * 1024, 8192, 512, SWZ_64B);
                if (p.a_major >= 2) umma_bf16_ts(tmem, tmem + 128 + ks * 8, bd, idesc, ks > 0);
                else umma_bf16_ss(tmem, ad, bd, idesc, ks > 0);
            }
            umma_commit(&bar_mma);
        }
        ok = mbar_wait(&bar_mma, 0, p.status, kDevTimeoutMma);
        ok = __syncthreads_and(ok);
    }
    if (ok) {
        tc_fence_after_sync();
        uint32_t r[32];
        for (int col = 0; col < p.N; col += 32) {
            tmem_ld_x32(tmem_addr(tmem, warp * 32, col), r);
            tmem_ld_wait();
            for (int c = 0; c < 32; ++c) p.d[static_cast<size_t>(warp * 32 + lane) * p.N + col + c] = __uint_as_float(r[c]);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace
}  // namespace gdn

using namespace gdn;

extern "C" int gdn_umma_probe(const void* a, const void* b, float* d_out, int* status_word, int M, int N, int K,
                              int a_major, int b_major, int b_span, int use_tma, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if ((M != 64 && M != 128) || N < 32 || N > 128 || N % 32 || K < 16 || K > 128 || K % 16) return GDN_ERR_BAD_ARGUMENT;
    if (a_major < 0 || a_major > 3 || b_major < 0 || b_major > 1 || (b_span != 128 && b_span != 64)) return GDN_ERR_BAD_ARGUMENT;
    if (a_major == MAJOR_MN && M != 128 && M != 64) return GDN_ERR_BAD_ARGUMENT;
    if (a_major >= 2 && (M != 128 || use_tma || K % 32)) return GDN_ERR_BAD_ARGUMENT;   // A in tensor memory: thread staging only
    if (b_major == MAJOR_MN && b_span == 128 && N % 64) return GDN_ERR_BAD_ARGUMENT;
    if (!a || !b || !d_out || !status_word) return GDN_ERR_BAD_ARGUMENT;
    if (cudaMemsetAsync(status_word, 0, sizeof(int), stream) != cudaSuccess) return GDN_ERR_CUDA;
    if (cudaMemsetAsync(d_out, 0, sizeof(float) * 128 * N, stream) != cudaSuccess) return GDN_ERR_CUDA;

    alignas(64) CUtensorMap ta, tb;
    memset(&ta, 0, sizeof(ta));
    memset(&tb, 0, sizeof(tb));
    if (use_tma) {
        // K-major operand: global [rows][K], box 64 k x rows.  MN-major: global [K][mn], box span x K rows.
        auto enc = [&](CUtensorMap* tm, const void* base, int major, int mn, int span) -> int {
            if (major == MAJOR_K) {
                const unsigned long long dims[2] = {static_cast<unsigned long long>(K), static_cast<unsigned long long>(mn)};
                const unsigned long long str[1] = {static_cast<unsigned long long>(K) * 2};
                const unsigned box[2] = {static_cast<unsigned>(K < 64 ? K : 64), static_cast<unsigned>(mn)};
                return encode_tma_bf16(tm, base, 2, dims, str, box, 128);
            }
            const unsigned long long dims[2] = {static_cast<unsigned long long>(mn), static_cast<unsigned long long>(K)};
            const unsigned long long str[1] = {static_cast<unsigned long long>(mn) * 2};
            const unsigned box[2] = {static_cast<unsigned>(span / 2), static_cast<unsigned>(K)};
            return encode_tma_bf16(tm, base, 2, dims, str, box, span);
        };
        if (K % 64 && (a_major == MAJOR_K || b_major == MAJOR_K)) return GDN_ERR_BAD_ARGUMENT;
        if (enc(&ta, a, a_major, M, 128)) return GDN_ERR_DRIVER;
        if (enc(&tb, b, b_major, N, b_span)) return GDN_ERR_DRIVER;
    }
    ProbeArgs p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d_out, status_word,
                M, N, K, a_major, b_major, b_span, use_tma};
    const int smem = 2 * kOpBytes + 1024;
    if (cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return GDN_ERR_CUDA;
    umma_probe_kernel<<<1, 128, smem, stream>>>(ta, tb, p);
    count_launch();
    if (cudaGetLastError() != cudaSuccess) return GDN_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return GDN_ERR_CUDA;
    int st = 0;
    if (cudaMemcpy(&st, status_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return GDN_ERR_CUDA;
    return st == 0 ? GDN_OK : GDN_ERR_DEVICE;
}
