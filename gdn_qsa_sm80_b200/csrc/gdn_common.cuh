// Declarations shared by the gdn_chunk translation units (internal; the public surface is
// include/gdn_chunk_sm100.h).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace gdn {

constexpr int kD = 128;      // head dimension (keys and values)
constexpr int kChunk = 64;   // tokens per chunk
constexpr float kLog2e = 1.4426950408889634f;

struct Problem {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    const void* g;
    const void* beta;
    const float* h0;       // may be null
    __nv_bfloat16* out;
    float* hT;             // may be null
    int* status;           // device status word (never null)
    long long* prof;       // optional: 16 per-phase cycle counters written by CTA (0,0,0); null = off
    int B, S, Hq, Hv;
    int gate_f32;          // 0: g/beta are bf16, 1: fp32
};

// Device status codes written by kernels (0 = fine).  The low byte says which wait gave up.
constexpr int kDevTimeoutTma = 0x101;
constexpr int kDevTimeoutMma = 0x102;

void count_launch();

// Token-by-token fp32 kernel on CUDA cores (one CTA per (batch, value head)).
cudaError_t launch_simt(const Problem& p, cudaStream_t stream);

// Fused tcgen05 kernel; nv = value columns per CTA (32 or 64).  Returns a GDN_* status.
int launch_fused(const Problem& p, int nv, cudaStream_t stream);

// Host helper: encode a tiled TMA descriptor for a row-major bf16 tensor of `rank` dims
// (dims/strides innermost first; strides in bytes for dims 1..rank-1).  swizzle_bytes: 128 or 64.
// Returns 0 on success.
int encode_tma_bf16(void* tmap_out, const void* base, int rank, const unsigned long long* dims,
                    const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes);

}  // namespace gdn
