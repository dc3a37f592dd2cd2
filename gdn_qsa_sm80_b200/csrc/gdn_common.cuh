// Declarations shared by the gdn_chunk translation units (internal; the public surface is
// include/gdn_chunk_sm100.h).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

// The kernels' cycle accounting is compiled in only with -DGDN_DIAGNOSTICS; otherwise every "is accounting on"
// test is the constant false and the accounting code disappears from the kernels.
#ifdef GDN_DIAGNOSTICS
#define GDN_DIAG(x) (x)
#else
#define GDN_DIAG(x) false
#endif

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
    int gate_act;          // 1: g and beta hold raw values; the kernels apply g = -softplus(.), beta = sigmoid(.)
    int l2norm;            // 1: q and k are L2-normalised per head vector inside the kernels
    int dbg;               // experiment switch (environment variable GDN_CHUNK_DBG); 0 in production
};

// Workspace of the two-kernel path (device pointers into the caller's scratch buffer).
// One tile per (batch, value head, chunk): tile = (b * Hv + hv) * NT + t.
struct Workspace {
    __nv_bfloat16* W;   // [tiles][64][128]  W = T (beta e^gamma K)
    __nv_bfloat16* P;   // [tiles][64][64]   masked, scaled Q K^T
    __nv_bfloat16* U;   // [tiles][64][128]  U = T (beta V); the transposed chain's T'' = T diag(beta), [tiles][64][64], instead
    float* vec;         // [tiles][256]      exp(gamma_C-gamma_i) | scale exp(gamma_i) | exp(gamma_C) | pad
    float* meta;        // [tiles][2]        sum of g over the chunk | max_j beta_j |k_j|^2 (+inf if a gate is out of range);
                        //                   null when sequences are not split
    int n_seg;          // segments a sequence is split into by the transposed chain (1 = not split)
};

// Byte offsets of the workspace arrays inside the scratch buffer (the status word sits at offset 0).
struct WorkspaceLayout {
    size_t W, P, U, vec, flags, flag_bytes, meta, total;
};
// with_meta: room for the two scalars per tile that the on-device decision to split sequences reads
inline WorkspaceLayout workspace_layout(size_t tiles, bool with_meta = false) {
    WorkspaceLayout l;
    l.W = 1024;
    l.P = l.W + tiles * 16384;
    l.U = l.P + tiles * 8192;
    l.vec = l.U + tiles * 16384;
    l.flags = l.vec + tiles * 1024;                      // one int per tile: "prepared" flags of the single-launch path
    l.flag_bytes = (tiles * 4 + 1023) / 1024 * 1024;
    l.meta = l.flags + l.flag_bytes;
    l.total = l.meta + (with_meta ? (tiles * 8 + 1023) / 1024 * 1024 : 0);
    return l;
}
// Into how many contiguous segments the transposed chain splits every sequence (1 = not at all): only when there are
// too few sequences to fill the GPU, segments of at least 16 chunks, at most 8 of them.  A function of the shape and
// of the SM count alone.
inline int chain_segments(int B, int Hv, int S, int sms) {
    const long long seqs = static_cast<long long>(B) * Hv;
    const int NT = (S + kChunk - 1) / kChunk;
    if (seqs * 2 > sms) return 1;
    int g = static_cast<int>(sms / seqs);
    if (g > 8) g = 8;
    if (g > NT / 16) g = NT / 16;
    return g < 2 ? 1 : g;
}
constexpr float kForgetLn = -115.f;   // exp(-115) < 2^-149: a transfer matrix bounded by it is zero in fp32

// Device status codes written by kernels (0 = fine).  The low byte says which wait gave up.
constexpr int kDevTimeoutTma = 0x101;
constexpr int kDevTimeoutMma = 0x102;

void count_launch();

// Token-by-token fp32 kernel on CUDA cores (one CTA per (batch, value head)).
cudaError_t launch_simt(const Problem& p, cudaStream_t stream);

// "prepare" (state-independent per-chunk quantities into the workspace) and "chain" (the serial
// state recurrence plus outputs, reading the workspace).  Both return a GDN_* status.
// with_u = false (for the transposed chain): no U tile; T'' = T diag(beta), bf16 [tiles][64][64], is written at the
// start of the U array instead.
int launch_prepare(const Problem& p, const Workspace& ws, cudaStream_t stream, bool with_u = true);
// The same as launch_prepare(with_u = false), two value heads of a qk head per CTA (shared K / Q load and raw
// products, one product for both W); needs an even number of value heads per qk head.
int launch_prepare_pair(const Problem& p, const Workspace& ws, cudaStream_t stream);
int launch_chain(const Problem& p, const Workspace& ws, int nv, cudaStream_t stream);
// The chain in transposed form: one CTA per (batch, value head), all 128 value columns (gdn_chain_t_device.cuh).
// With ws.n_seg > 1 every sequence is cut into ws.n_seg segments that run as independent chains of one launch, each
// warmed up from a zero state over the chunks before it that make the state forget its past - for the heads whose
// gates allow that (decided on the device from ws.meta); the other heads run as one serial chain.  Exact in both cases.
int launch_chain_t(const Problem& p, const Workspace& ws, cudaStream_t stream);
// Single-launch variant (prepare shared among the four column CTAs of a head, chain in the same kernel);
// only when all CTAs fit on the GPU at once.
bool coop_supported(const Problem& p);
// skip_prepare (measurement aid): run only the chain roles on a workspace an earlier call left behind.
int launch_coop(const Problem& p, const Workspace& ws, int* flags, size_t flag_bytes, cudaStream_t stream,
                bool skip_prepare = false);

// Host helper: encode a tiled TMA descriptor for a row-major tensor of `rank` dims
// (dims/strides innermost first; strides in bytes for dims 1..rank-1).  swizzle_bytes: 128 or 64.
// elem_bytes: 2 = bf16, 4 = fp32.  Returns 0 on success.
int encode_tma(void* tmap_out, const void* base, int elem_bytes, int rank, const unsigned long long* dims,
               const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes);
inline int encode_tma_bf16(void* tmap_out, const void* base, int rank, const unsigned long long* dims,
                           const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes) {
    return encode_tma(tmap_out, base, 2, rank, dims, strides_bytes, box, swizzle_bytes);
}
// TMA descriptors of the workspace arrays: W, P and U as 64x64 bf16 boxes (128-byte swizzle; what the prepare side
// stores and the chain side loads for W and P), and U as nv x 64 boxes (swizzle span 2*nv bytes) for the chain's
// column slice.  tu_load may be null.
int encode_workspace_maps(const Problem& p, const Workspace& ws, void* tw, void* tp, void* tu_store, void* tu_load, int nv);
// Number of SMs of the current device (cached per device).
cudaError_t launch_decode(const Problem& p, cudaStream_t stream);
int sm_count();
cudaError_t launch_rmsnorm_gated(const void* y, const void* z, const void* weight, void* out, long long n_rows,
                                 float eps, cudaStream_t stream);
// The forward pass on device buffers (what gdn_chunk_fwd_sm100_ex does).  clear_status = false leaves the status
// word at the start of `scratch` as it is, so that several launches can share one sticky word.
// gate != nullptr: the output rows are replaced by rmsnorm_gated(row, z, weight), by the normalisation kernel
// launched right behind the forward pass.
struct OutputGate {
    const void* z;
    const void* weight;
    float eps;
};
int forward_device(const void* q, const void* k, const void* v, const void* g, const void* beta, const float* h0,
                   void* out, float* hT, void* scratch, size_t scratch_bytes, int B, int S, int Hq, int Hv,
                   int gate_dtype, int path, unsigned flags, cudaStream_t stream, bool clear_status,
                   const OutputGate* gate = nullptr);
// TMA descriptors of q, k ([B,S,Hq,128], 64x64 boxes) and v ([B,S,Hv,128], v_box_cols x 64 boxes).
int encode_qkv_maps(const Problem& p, void* tq, void* tk, void* tv, int v_box_cols);

}  // namespace gdn
