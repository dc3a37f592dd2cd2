// C ABI of the library (see include/gdn_chunk_sm100.h): argument checks, TMA descriptor
// encoding through the driver entry point, path selection, status word handling.
#include <cuda.h>

#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"

namespace gdn {

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

int encode_tma(void* tmap_out, const void* base, int elem_bytes, int rank, const unsigned long long* dims,
               const unsigned long long* strides_bytes, const unsigned* box, int swizzle_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return 1;
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                        : CU_TENSOR_MAP_SWIZZLE_NONE;
    const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult r = fn(static_cast<CUtensorMap*>(tmap_out), dt, rank,
                          const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1;
}

int encode_qkv_maps(const Problem& p, void* tq, void* tk, void* tv, int v_box_cols) {
    const unsigned long long dq[4] = {static_cast<unsigned long long>(kD), static_cast<unsigned long long>(p.Hq),
                                      static_cast<unsigned long long>(p.S), static_cast<unsigned long long>(p.B)};
    const unsigned long long sq[3] = {kD * 2ull, static_cast<unsigned long long>(p.Hq) * kD * 2ull,
                                      static_cast<unsigned long long>(p.S) * p.Hq * kD * 2ull};
    const unsigned long long dv[4] = {static_cast<unsigned long long>(kD), static_cast<unsigned long long>(p.Hv),
                                      static_cast<unsigned long long>(p.S), static_cast<unsigned long long>(p.B)};
    const unsigned long long sv[3] = {kD * 2ull, static_cast<unsigned long long>(p.Hv) * kD * 2ull,
                                      static_cast<unsigned long long>(p.S) * p.Hv * kD * 2ull};
    const unsigned box_qk[4] = {64, 1, 64, 1};
    const unsigned box_v[4] = {static_cast<unsigned>(v_box_cols), 1, 64, 1};
    if (encode_tma(tq, p.q, 2, 4, dq, sq, box_qk, 128)) return 1;
    if (encode_tma(tk, p.k, 2, 4, dq, sq, box_qk, 128)) return 1;
    if (encode_tma(tv, p.v, 2, 4, dv, sv, box_v, v_box_cols * 2)) return 1;
    return 0;
}

int encode_workspace_maps(const Problem& p, const Workspace& ws, void* tw, void* tp, void* tu_store, void* tu_load, int nv) {
    const int NT = (p.S + kChunk - 1) / kChunk;
    const unsigned long long rows = static_cast<unsigned long long>(p.B) * p.Hv * NT * kChunk;
    {
        const unsigned long long d[2] = {128, rows}, s[1] = {256};
        const unsigned box[2] = {64, 64};
        if (encode_tma(tw, ws.W, 2, 2, d, s, box, 128)) return 1;
    }
    {
        const unsigned long long d[2] = {64, rows}, s[1] = {128};
        const unsigned box[2] = {64, 64};
        if (encode_tma(tp, ws.P, 2, 2, d, s, box, 128)) return 1;
    }
    {
        const unsigned long long d[2] = {128, rows}, s[1] = {256};
        const unsigned box[2] = {64, 64};
        if (tu_store && encode_tma(tu_store, ws.U, 2, 2, d, s, box, 128)) return 1;
        const unsigned boxl[2] = {static_cast<unsigned>(nv), 64};
        if (tu_load && encode_tma(tu_load, ws.U, 2, 2, d, s, boxl, nv * 2)) return 1;
    }
    return 0;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static long long* g_phase_profile = nullptr;
constexpr int kDecodeMaxTokens = 8;   // sequences this short take the decode kernel under GDN_PATH_AUTO

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace gdn

using namespace gdn;

extern "C" {

static size_t tiles_of(int B, int S, int Hv) {
    return static_cast<size_t>(B) * Hv * ((S + kChunk - 1) / kChunk);
}

static bool path_uses_workspace(int path) {
    return path == GDN_PATH_AUTO || path == GDN_PATH_TWOPASS_NV64 || path == GDN_PATH_TWOPASS_NV32 ||
           path == GDN_PATH_PREPARE_ONLY || path == GDN_PATH_CHAIN_ONLY || path == GDN_PATH_COOP ||
           path == GDN_PATH_COOP_CHAIN_ONLY || path == GDN_PATH_TWOPASS_T ||
           path == GDN_PATH_PREPARE_ONLY_T || path == GDN_PATH_CHAIN_ONLY_T;
}

// segments the path cuts every sequence into (only the transposed chain splits sequences; 1 = not split)
static int segments_of(int B, int S, int Hv, int path) {
    if (path != GDN_PATH_TWOPASS_T && path != GDN_PATH_AUTO && path != GDN_PATH_PREPARE_ONLY_T && path != GDN_PATH_CHAIN_ONLY_T)
        return 1;
    return chain_segments(B, Hv, S, sm_count());
}

size_t gdn_chunk_scratch_bytes(int B, int S, int Hq, int Hv, int path) {
    (void)Hq;
    if (B <= 0 || S < 0 || Hv <= 0) return 0;
    if (!path_uses_workspace(path)) return 256;   // only the device status word, padded
    return workspace_layout(tiles_of(B, S, Hv), segments_of(B, S, Hv, path) > 1).total;
}

int gdn_chunk_workspace_offsets(int B, int S, int Hq, int Hv, size_t* offsets) {
    (void)Hq;
    if (B <= 0 || S < 0 || Hv <= 0 || !offsets) return GDN_ERR_BAD_ARGUMENT;
    const WorkspaceLayout l = workspace_layout(tiles_of(B, S, Hv));
    offsets[0] = l.W; offsets[1] = l.P; offsets[2] = l.U; offsets[3] = l.vec; offsets[4] = l.total;
    return GDN_OK;
}

int gdn_chunk_fwd_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                        const float* h0, void* out, float* hT, void* scratch, size_t scratch_bytes,
                        int B, int S, int Hq, int Hv, int gate_dtype, int path, void* stream_) {
    return gdn_chunk_fwd_sm100_ex(q, k, v, g, beta, h0, out, hT, scratch, scratch_bytes, B, S, Hq, Hv, gate_dtype,
                                  path, 0u, stream_);
}

int gdn_chunk_fwd_sm100_ex(const void* q, const void* k, const void* v, const void* g, const void* beta,
                           const float* h0, void* out, float* hT, void* scratch, size_t scratch_bytes,
                           int B, int S, int Hq, int Hv, int gate_dtype, int path, unsigned flags, void* stream_) {
    return forward_device(q, k, v, g, beta, h0, out, hT, scratch, scratch_bytes, B, S, Hq, Hv, gate_dtype, path,
                          flags, static_cast<cudaStream_t>(stream_), true);
}

int gdn_chunk_fwd_gated_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                              const float* h0, const void* z, const void* weight, float eps, void* out, float* hT,
                              void* scratch, size_t scratch_bytes, int B, int S, int Hq, int Hv, int gate_dtype,
                              int path, unsigned flags, void* stream_) {
    if (!z || !weight || !aligned16(z) || !aligned16(weight)) return GDN_ERR_BAD_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const OutputGate gate{z, weight, eps};
    return forward_device(q, k, v, g, beta, h0, out, hT, scratch, scratch_bytes, B, S, Hq, Hv, gate_dtype, path, flags,
                          stream, true, &gate);
}

}  // extern "C"

namespace gdn {
int forward_device(const void* q, const void* k, const void* v, const void* g, const void* beta, const float* h0,
                   void* out, float* hT, void* scratch, size_t scratch_bytes, int B, int S, int Hq, int Hv,
                   int gate_dtype, int path, unsigned flags, cudaStream_t stream, bool clear_status,
                   const OutputGate* gate) {
    if (flags & ~static_cast<unsigned>(GDN_FLAG_QK_L2NORM | GDN_FLAG_GATE_ACTIVATIONS)) return GDN_ERR_BAD_ARGUMENT;
    if (B <= 0 || S < 0 || Hq <= 0 || Hv <= 0 || Hv % Hq != 0) return GDN_ERR_BAD_ARGUMENT;
    if (gate_dtype != GDN_GATE_BF16 && gate_dtype != GDN_GATE_F32) return GDN_ERR_BAD_ARGUMENT;
    if (path < GDN_PATH_AUTO || path > GDN_PATH_CHAIN_ONLY_T || path == 2 || path == 3 || path == 10) return GDN_ERR_BAD_ARGUMENT;
    // the least a path needs; gdn_chunk_scratch_bytes may ask for more (room to split long sequences), which is used
    // when it is there
    const size_t need = path_uses_workspace(path) ? workspace_layout(tiles_of(B, S, Hv)).total : 256;
    if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 255u) || scratch_bytes < need) return GDN_ERR_SCRATCH;
    if (clear_status && cudaMemsetAsync(scratch, 0, 256, stream) != cudaSuccess) return GDN_ERR_CUDA;
    if (S == 0) {   // nothing to scan: the final state is the initial state
        if (hT) {
            const size_t bytes = static_cast<size_t>(B) * Hv * kD * kD * sizeof(float);
            const cudaError_t e = h0 ? cudaMemcpyAsync(hT, h0, bytes, cudaMemcpyDeviceToDevice, stream)
                                     : cudaMemsetAsync(hT, 0, bytes, stream);
            if (e != cudaSuccess) return GDN_ERR_CUDA;
        }
        return GDN_OK;
    }
    if (!q || !k || !v || !g || !beta || !out) return GDN_ERR_BAD_ARGUMENT;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(h0) || !aligned16(hT))
        return GDN_ERR_BAD_ARGUMENT;

    Problem p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.k = static_cast<const __nv_bfloat16*>(k);
    p.v = static_cast<const __nv_bfloat16*>(v);
    p.g = g;
    p.beta = beta;
    p.h0 = h0;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.hT = hT;
    p.status = static_cast<int*>(scratch);
    p.prof = g_phase_profile;
    p.B = B; p.S = S; p.Hq = Hq; p.Hv = Hv;
    p.gate_f32 = gate_dtype == GDN_GATE_F32;
    p.l2norm = (flags & GDN_FLAG_QK_L2NORM) ? 1 : 0;
    p.gate_act = (flags & GDN_FLAG_GATE_ACTIVATIONS) ? 1 : 0;
    {
        const char* e = getenv("GDN_CHUNK_DBG");
        p.dbg = e ? atoi(e) : 0;
    }
    // the normalisation kernel behind whatever produced `out`
    auto then_gate = [&](int st) -> int {
        if (st != GDN_OK || !gate) return st;
        const long long rows = static_cast<long long>(B) * S * Hv;
        return launch_rmsnorm_gated(out, gate->z, gate->weight, out, rows, gate->eps, stream) == cudaSuccess ? GDN_OK
                                                                                                          : GDN_ERR_CUDA;
    };

    // a few new tokens: the state read and write is all there is, and the decode kernel streams it (measured on
    // 2048 states: 55 us at one token = 4.8 TB/s, against 238 us through the chunk kernels; the two meet near 16 tokens)
    if (path == GDN_PATH_DECODE || (path == GDN_PATH_AUTO && S <= kDecodeMaxTokens))
        return then_gate(launch_decode(p, stream) == cudaSuccess ? GDN_OK : GDN_ERR_CUDA);
    if (path == GDN_PATH_SIMT) return then_gate(launch_simt(p, stream) == cudaSuccess ? GDN_OK : GDN_ERR_CUDA);
    // Automatic choice, by shape alone.  Few short sequences (up to 1024 tokens): the single-launch kernel whose four
    // 32-column CTAs per head share the prepare work.  Everything else: the prepare kernel and the transposed chain
    // (one CTA per head, state-dependent operands in tensor memory), which splits long sequences into segments when
    // there are too few of them to fill the GPU.  Measured on one B200, 32 sequences, single launch against the two
    // kernels: 512 tokens 0.036 / 0.037 ms, 1024 tokens 0.050 / 0.057, 2048 tokens 0.084 / 0.074.
    const bool automatic = path == GDN_PATH_AUTO;
    if (automatic) path = (S <= 1024 && coop_supported(p)) ? GDN_PATH_COOP : GDN_PATH_TWOPASS_T;
    int nv;
    if (path == GDN_PATH_TWOPASS_NV32) nv = 32;
    else nv = 64;
    // the transposed chain splits sequences when the scratch buffer has room for the per-tile scalars its decision
    // reads (a caller that sized it for an unsplit run, like the fixed-array entry point, gets the unsplit run)
    const bool transposed = path == GDN_PATH_TWOPASS_T || path == GDN_PATH_PREPARE_ONLY_T || path == GDN_PATH_CHAIN_ONLY_T;
    int n_seg = transposed ? segments_of(B, S, Hv, path) : 1;
    if (n_seg > 1 && scratch_bytes < workspace_layout(tiles_of(B, S, Hv), true).total) n_seg = 1;
    const WorkspaceLayout l = workspace_layout(tiles_of(B, S, Hv), n_seg > 1);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    Workspace ws;
    ws.W = reinterpret_cast<__nv_bfloat16*>(base + l.W);
    ws.P = reinterpret_cast<__nv_bfloat16*>(base + l.P);
    ws.U = reinterpret_cast<__nv_bfloat16*>(base + l.U);
    ws.vec = reinterpret_cast<float*>(base + l.vec);
    ws.meta = n_seg > 1 ? reinterpret_cast<float*>(base + l.meta) : nullptr;
    ws.n_seg = n_seg;
    if (path == GDN_PATH_COOP_CHAIN_ONLY)
        return then_gate(launch_coop(p, ws, reinterpret_cast<int*>(base + l.flags), l.flag_bytes, stream, true));
    if (path == GDN_PATH_COOP) {
        const int st = launch_coop(p, ws, reinterpret_cast<int*>(base + l.flags), l.flag_bytes, stream);
        // the single-launch kernel is a cooperative launch: when its grid cannot be resident all at once on this
        // context (fewer SMs than the device reports, a limited partition) the launch is refused and nothing has
        // run; the automatic path then takes the two-kernel route, which waits for nothing inside a launch
        if (!(automatic && st == GDN_ERR_CUDA)) return then_gate(st);
        (void)cudaGetLastError();
        path = GDN_PATH_TWOPASS_T;
    }
    if (path == GDN_PATH_CHAIN_ONLY) return then_gate(launch_chain(p, ws, nv, stream));   // workspace left by an earlier call
    if (path == GDN_PATH_CHAIN_ONLY_T) return then_gate(launch_chain_t(p, ws, stream));
    const bool pairs = transposed && (Hv / Hq) % 2 == 0 && p.dbg != 3;
    const int st = pairs ? launch_prepare_pair(p, ws, stream) : launch_prepare(p, ws, stream, !transposed);
    if (st != GDN_OK || path == GDN_PATH_PREPARE_ONLY || path == GDN_PATH_PREPARE_ONLY_T) return st;
    if (path == GDN_PATH_TWOPASS_T) return then_gate(launch_chain_t(p, ws, stream));
    return then_gate(launch_chain(p, ws, nv, stream));
}
}  // namespace gdn

extern "C" {

int gdn_chunk_read_status(const void* scratch, void* stream_, int* device_status) {
    if (!scratch || !device_status) return GDN_ERR_BAD_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int v = 0;
    if (cudaMemcpyAsync(&v, scratch, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return GDN_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return GDN_ERR_CUDA;
    *device_status = v;
    return v == 0 ? GDN_OK : GDN_ERR_DEVICE;
}

const char* gdn_chunk_error_string(int status) {
    switch (status) {
        case GDN_OK: return "ok";
        case GDN_ERR_BAD_ARGUMENT: return "bad argument (shape, alignment, dtype or path)";
        case GDN_ERR_SCRATCH: return "scratch buffer missing, misaligned or too small";
        case GDN_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case GDN_ERR_DRIVER: return "driver rejected a TMA tensor-map description";
        case GDN_ERR_DEVICE: return "a kernel gave up on a bounded wait (device status word is non-zero)";
        default: return "unknown status";
    }
}

// ---------------------------------------------------------------------------------------------
// Forward pass for callers that cannot provide scratch memory.
//
// Some hosts of this library may not allocate device memory at all when they call it: a serving
// runtime that reserved its whole memory budget at start-up and hands out fixed buffers for inputs
// and outputs only, or a latency-critical loop in which cudaMalloc (which synchronises the whole
// device) must never run.  For them the workspace of the automatic path (whichever kernels it picks) lives in the array
// below, which every GPU that loads this library holds until the process exits.
//
// `g_noalloc_scratch` is a HOST-side handle in host code, not a device address; its device address
// is looked up once per device with cudaGetSymbolAddress (with that device current) and kept in
// g_noalloc_addr.  All calls on a device share the one array: the status word at its start is cleared
// by every call, everything else is fully rewritten before it is read, and two calls that overlap on
// the GPU (different streams) would race on it.
// ---------------------------------------------------------------------------------------------
constexpr size_t kNoAllocBytes = 16u << 20;   // 16 MiB: up to 399 (batch x value head x 64-token chunk) tiles
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
static void* g_noalloc_addr[64] = {nullptr};
static std::mutex g_noalloc_mutex;

int gdn_chunk_fwd_sm100_noalloc(const void* q, const void* k, const void* v, const void* g, const void* beta,
                                const float* h0, void* out, float* hT, int B, int S, int Hq, int Hv,
                                int gate_dtype, void* stream) {
    if (B <= 0 || S < 0 || Hq <= 0 || Hv <= 0 || Hv % Hq != 0) return GDN_ERR_BAD_ARGUMENT;
    // reject problems whose workspace does not fit the fixed array (the caller gets a clear status, nothing runs)
    if (workspace_layout(tiles_of(B, S, Hv)).total > kNoAllocBytes) return GDN_ERR_SCRATCH;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GDN_ERR_CUDA;
    void* addr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_addr[dev]) {   // first call on this device: one-time set-up
            void* ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) return GDN_ERR_CUDA;
            g_noalloc_addr[dev] = ptr;
        }
        addr = g_noalloc_addr[dev];
    }
    return gdn_chunk_fwd_sm100(q, k, v, g, beta, h0, out, hT, addr, kNoAllocBytes, B, S, Hq, Hv, gate_dtype,
                               GDN_PATH_AUTO, stream);
}

void gdn_chunk_set_phase_profile(void* device_buffer) { g_phase_profile = static_cast<long long*>(device_buffer); }

unsigned long long gdn_chunk_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
