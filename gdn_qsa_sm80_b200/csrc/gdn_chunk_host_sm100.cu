// Forward pass on HOST buffers: the sequence is cut into segments and host->device copies, kernels and
// device->host copies of different segments overlap (see gdn_chunk_fwd_host_sm100 in the public header).
//
// Why this exists: with inputs and outputs in host memory the operator is bound by the host link, not by
// the kernels (the kernels of a step take a tenth of the time of its copies).  Copying everything in, running,
// and copying everything out uses the link in one direction at a time; cutting the sequence into segments
// lets the inputs of segment i+1, the kernels of segment i and the outputs of segment i-1 move at once, so a
// call costs about max(inputs, outputs) / link bandwidth instead of their sum.  Splitting the sequence is
// exact: segment i starts from the fp32 state segment i-1 ended with.
//
// Three streams per device: the caller's stream runs the kernels, two internal streams carry the copies.
// All ordering is by events; the call returns without waiting, and work the caller enqueues on its stream
// afterwards runs after the last output byte has landed in host memory.
#include <mutex>

#include "../../include/gdn_chunk_sm100.h"
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int kMaxSegments = 256;
constexpr int kInSlots = 3;    // input staging buffers in flight: one being filled, one queued, one being read
constexpr int kOutSlots = 2;   // output staging buffers: one being written, one being copied out

struct HostPipe {
    bool ready = false;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    cudaEvent_t start = nullptr, done = nullptr;
    cudaEvent_t in_ready[kMaxSegments], computed[kMaxSegments], out_copied[kMaxSegments];
    std::mutex enqueue;   // one call at a time enqueues on a device: the events are shared
};
HostPipe g_pipes[64];
std::mutex g_pipe_mutex;

// Streams and events of the current device, created on first use (no device memory involved).
HostPipe* pipe_for_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_pipe_mutex);
    HostPipe& hp = g_pipes[dev];
    if (hp.ready) return &hp;
    if (cudaStreamCreateWithFlags(&hp.h2d, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&hp.d2h, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    auto mk = [](cudaEvent_t* e) { return cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess; };
    if (!mk(&hp.start) || !mk(&hp.done)) return nullptr;
    for (int i = 0; i < kMaxSegments; ++i)
        if (!mk(&hp.in_ready[i]) || !mk(&hp.computed[i]) || !mk(&hp.out_copied[i])) return nullptr;
    hp.ready = true;
    return &hp;
}

inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct Arena {
    size_t q[kInSlots], k[kInSlots], v[kInSlots], g[kInSlots], beta[kInSlots];
    size_t out[kOutSlots], state[2], scratch, scratch_bytes, total;
};

Arena arena_layout(int B, int seg, int Hq, int Hv, int gate_bytes) {
    Arena a;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += align256(bytes);
        return at;
    };
    const size_t qk = static_cast<size_t>(B) * seg * Hq * kD * 2, vv = static_cast<size_t>(B) * seg * Hv * kD * 2;
    const size_t gb = static_cast<size_t>(B) * seg * Hv * gate_bytes;
    a.scratch_bytes = gdn_chunk_scratch_bytes(B, seg, Hq, Hv, GDN_PATH_AUTO);
    a.scratch = take(a.scratch_bytes);
    for (int s = 0; s < kInSlots; ++s) {
        a.q[s] = take(qk);
        a.k[s] = take(qk);
        a.v[s] = take(vv);
        a.g[s] = take(gb);
        a.beta[s] = take(gb);
    }
    for (int s = 0; s < kOutSlots; ++s) a.out[s] = take(vv);
    for (int s = 0; s < 2; ++s) a.state[s] = take(static_cast<size_t>(B) * Hv * kD * kD * sizeof(float));
    a.total = off;
    return a;
}

// Tokens per segment when the caller leaves the choice to the library: four segments, at least 256 tokens
// each.  The first segment's inputs and the last one's outputs cannot overlap with anything, which asks for
// many segments; every copy costs a few microseconds of idle link and every launch its ramp-up, which asks
// for few.  Measured on the default workload (8192 tokens, 138 MB in, 69 MB out): 3.79 / 3.66 / 3.41 / 3.37 /
// 3.50 / 4.05 ms per call with 32 / 16 / 8 / 4 / 2 / 1 segments.
int pick_segment(int S, int seg_tokens) {
    int seg = seg_tokens;
    if (seg <= 0) {
        seg = (S + 3) / 4;
        if (seg < 256) seg = 256;
    }
    seg = (seg + kChunk - 1) / kChunk * kChunk;
    while (seg > 0 && (S + seg - 1) / seg > kMaxSegments) seg *= 2;
    if (seg > S) seg = (S + kChunk - 1) / kChunk * kChunk;
    return seg > 0 ? seg : kChunk;
}

// rows [s0, s0+n) of every batch element of a host tensor [B][S][row_bytes] <-> a dense device tensor [B][n][row_bytes]
cudaError_t copy_rows(void* dev, const void* host, bool to_device, int B, int S, int s0, int n, size_t row_bytes,
                      cudaStream_t stream) {
    const size_t host_pitch = static_cast<size_t>(S) * row_bytes, width = static_cast<size_t>(n) * row_bytes;
    const char* h = static_cast<const char*>(host) + static_cast<size_t>(s0) * row_bytes;
    if (to_device) {
        if (B == 1 || n == S) return cudaMemcpyAsync(dev, h, width * (n == S ? B : 1), cudaMemcpyHostToDevice, stream);
        if (host_pitch < (1ull << 31))
            return cudaMemcpy2DAsync(dev, width, h, host_pitch, width, B, cudaMemcpyHostToDevice, stream);
        for (int b = 0; b < B; ++b) {
            const cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dev) + b * width, h + b * host_pitch, width,
                                                  cudaMemcpyHostToDevice, stream);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    char* hw = const_cast<char*>(h);
    if (B == 1 || n == S) return cudaMemcpyAsync(hw, dev, width * (n == S ? B : 1), cudaMemcpyDeviceToHost, stream);
    if (host_pitch < (1ull << 31))
        return cudaMemcpy2DAsync(hw, host_pitch, dev, width, width, B, cudaMemcpyDeviceToHost, stream);
    for (int b = 0; b < B; ++b) {
        const cudaError_t e = cudaMemcpyAsync(hw + b * host_pitch, static_cast<const char*>(dev) + b * width, width,
                                              cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace
}  // namespace gdn

using namespace gdn;

extern "C" {

size_t gdn_chunk_host_arena_bytes(int B, int S, int Hq, int Hv, int gate_dtype, int seg_tokens) {
    if (B <= 0 || S < 0 || Hq <= 0 || Hv <= 0) return 0;
    const int seg = pick_segment(S > 0 ? S : kChunk, seg_tokens);
    return arena_layout(B, seg, Hq, Hv, gate_dtype == GDN_GATE_F32 ? 4 : 2).total;
}

int gdn_chunk_fwd_host_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                             const float* h0, void* out, float* hT, void* arena, size_t arena_bytes, int B, int S,
                             int Hq, int Hv, int gate_dtype, int seg_tokens, unsigned flags, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (B <= 0 || S < 0 || Hq <= 0 || Hv <= 0 || Hv % Hq != 0) return GDN_ERR_BAD_ARGUMENT;
    if (gate_dtype != GDN_GATE_BF16 && gate_dtype != GDN_GATE_F32) return GDN_ERR_BAD_ARGUMENT;
    if (flags & ~static_cast<unsigned>(GDN_FLAG_QK_L2NORM | GDN_FLAG_GATE_ACTIVATIONS)) return GDN_ERR_BAD_ARGUMENT;
    if (S > 0 && (!q || !k || !v || !g || !beta || !out)) return GDN_ERR_BAD_ARGUMENT;
    if (!arena || (reinterpret_cast<uintptr_t>(arena) & 255u) ||
        arena_bytes < gdn_chunk_host_arena_bytes(B, S, Hq, Hv, gate_dtype, seg_tokens))
        return GDN_ERR_SCRATCH;
    HostPipe* hp = pipe_for_current_device();
    if (!hp) return GDN_ERR_CUDA;
    std::lock_guard<std::mutex> enqueue_lock(hp->enqueue);

    const int gate_bytes = gate_dtype == GDN_GATE_F32 ? 4 : 2;
    const int seg = pick_segment(S > 0 ? S : kChunk, seg_tokens);
    const Arena a = arena_layout(B, seg, Hq, Hv, gate_bytes);
    char* base = static_cast<char*>(arena);
    const size_t state_bytes = static_cast<size_t>(B) * Hv * kD * kD * sizeof(float);
    const int n_seg = S > 0 ? (S + seg - 1) / seg : 0;
#define GDN_TRY(call) \
    if ((call) != cudaSuccess) return GDN_ERR_CUDA

    // The copies and kernels of the call; a failure part-way leaves work on the copy streams, so the join below
    // runs whatever this returns.
    auto enqueue_all = [&]() -> int {
    // everything below is ordered after what the caller's stream holds so far (an earlier call's use of the arena included)
    GDN_TRY(cudaEventRecord(hp->start, stream));
    GDN_TRY(cudaStreamWaitEvent(hp->h2d, hp->start, 0));
    GDN_TRY(cudaStreamWaitEvent(hp->d2h, hp->start, 0));
    GDN_TRY(cudaMemsetAsync(base + a.scratch, 0, 256, stream));   // one sticky status word for all segments
    float* state[2] = {reinterpret_cast<float*>(base + a.state[0]), reinterpret_cast<float*>(base + a.state[1])};
    if (h0) GDN_TRY(cudaMemcpyAsync(state[0], h0, state_bytes, cudaMemcpyHostToDevice, hp->h2d));

    const size_t row_qk = static_cast<size_t>(Hq) * kD * 2, row_v = static_cast<size_t>(Hv) * kD * 2;
    const size_t row_g = static_cast<size_t>(Hv) * gate_bytes;
    for (int i = 0; i < n_seg; ++i) {
        const int s0 = i * seg, n = (S - s0 < seg) ? S - s0 : seg;
        const int si = i % kInSlots, so = i % kOutSlots;
        // inputs of segment i: wait until the kernels that read this slot last (segment i - kInSlots) are done
        if (i >= kInSlots) GDN_TRY(cudaStreamWaitEvent(hp->h2d, hp->computed[i - kInSlots], 0));
        GDN_TRY(copy_rows(base + a.q[si], q, true, B, S, s0, n, row_qk, hp->h2d));
        GDN_TRY(copy_rows(base + a.k[si], k, true, B, S, s0, n, row_qk, hp->h2d));
        GDN_TRY(copy_rows(base + a.v[si], v, true, B, S, s0, n, row_v, hp->h2d));
        GDN_TRY(copy_rows(base + a.g[si], g, true, B, S, s0, n, row_g, hp->h2d));
        GDN_TRY(copy_rows(base + a.beta[si], beta, true, B, S, s0, n, row_g, hp->h2d));
        GDN_TRY(cudaEventRecord(hp->in_ready[i], hp->h2d));
        // kernels of segment i on the caller's stream, from the state segment i-1 left
        GDN_TRY(cudaStreamWaitEvent(stream, hp->in_ready[i], 0));
        if (i >= kOutSlots) GDN_TRY(cudaStreamWaitEvent(stream, hp->out_copied[i - kOutSlots], 0));
        const float* s_in = (i == 0 && !h0) ? nullptr : state[i & 1];
        float* s_out = (hT || i + 1 < n_seg) ? state[(i + 1) & 1] : nullptr;
        const int st = forward_device(base + a.q[si], base + a.k[si], base + a.v[si], base + a.g[si], base + a.beta[si],
                                      s_in, base + a.out[so], s_out, base + a.scratch, a.scratch_bytes, B, n, Hq, Hv,
                                      gate_dtype, GDN_PATH_AUTO, flags, stream, false);
        if (st != GDN_OK) return st;
        GDN_TRY(cudaEventRecord(hp->computed[i], stream));
        // outputs of segment i
        GDN_TRY(cudaStreamWaitEvent(hp->d2h, hp->computed[i], 0));
        GDN_TRY(copy_rows(base + a.out[so], out, false, B, S, s0, n, row_v, hp->d2h));
        GDN_TRY(cudaEventRecord(hp->out_copied[i], hp->d2h));
    }
    if (hT) {
        if (n_seg == 0) {   // empty sequence: the final state is the initial state
            if (h0) {
                GDN_TRY(cudaEventRecord(hp->in_ready[0], hp->h2d));
                GDN_TRY(cudaStreamWaitEvent(hp->d2h, hp->in_ready[0], 0));
            } else {
                GDN_TRY(cudaMemsetAsync(state[0], 0, state_bytes, hp->d2h));
            }
        }
        GDN_TRY(cudaMemcpyAsync(hT, state[n_seg & 1], state_bytes, cudaMemcpyDeviceToHost, hp->d2h));
    }
    return GDN_OK;
    };
    const int st = enqueue_all();
    // The caller's stream continues only when every copy this call enqueued is complete - also after an error, so
    // that the caller may free or reuse the arena and the host buffers once its stream has drained.
    auto join = [&](cudaStream_t copies) -> int {
        GDN_TRY(cudaEventRecord(hp->done, copies));
        GDN_TRY(cudaStreamWaitEvent(stream, hp->done, 0));
        return GDN_OK;
    };
    const int j0 = join(hp->d2h), j1 = join(hp->h2d);
#undef GDN_TRY
    return st != GDN_OK ? st : (j0 != GDN_OK ? j0 : j1);
}

}  // extern "C"
