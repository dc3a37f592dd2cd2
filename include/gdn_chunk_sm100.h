/*
 * C ABI of the sm_100a gdn_chunk forward library (libgdn_chunk_sm100.so).
 *
 * This is the boundary a host binding talks to: plain pointers and sizes, no torch types.
 * Every pointer is a DEVICE pointer in the current CUDA context unless stated otherwise.
 * The library allocates no device memory, never synchronises the stream (except the two
 * diagnostic calls marked "synchronises") and never throws: every call returns a status.
 *
 * Each entry point names the interface of the reference project it stands in for
 * (paths are relative to the reference project's root).
 */
#ifndef GDN_CHUNK_SM100_H
#define GDN_CHUNK_SM100_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes returned by every call. */
#define GDN_OK 0
#define GDN_ERR_BAD_ARGUMENT 1   /* shape, alignment, dtype or path value not accepted            */
#define GDN_ERR_SCRATCH 2        /* scratch pointer missing, misaligned or smaller than required  */
#define GDN_ERR_CUDA 3           /* a CUDA runtime call or a kernel launch failed                  */
#define GDN_ERR_DRIVER 4         /* the driver rejected a TMA tensor-map description               */
#define GDN_ERR_DEVICE 5         /* a kernel reported a bounded wait that ran out (see read_status) */

/* dtype of g and beta */
#define GDN_GATE_BF16 0
#define GDN_GATE_F32 1

/* execution path */
#define GDN_PATH_AUTO 0          /* DECODE when S <= 8; COOP when S <= 1024 and 4*B*Hv <= #SMs; else TWOPASS_T     */
#define GDN_PATH_SIMT 1          /* token-by-token fp32 kernel on CUDA cores (exact; slow; for checks) */
                                 /* (values 2, 3 and 10 belonged to kernels that have been removed)    */
#define GDN_PATH_TWOPASS_NV64 4  /* prepare kernel + chain kernel, 64 value columns per chain CTA    */
#define GDN_PATH_TWOPASS_NV32 5  /* prepare kernel + chain kernel, 32 value columns per chain CTA    */
#define GDN_PATH_PREPARE_ONLY 6  /* measurement aid: only the prepare kernel (fills the workspace)    */
#define GDN_PATH_CHAIN_ONLY 7    /* measurement aid: only the chain kernel, on the workspace an earlier
                                    call with the same arguments and scratch left behind              */
#define GDN_PATH_COOP 8          /* one launch: the four 32-column CTAs of a head share the prepare work
                                    through the workspace while their chains run; needs 4*B*Hv <= #SMs    */
#define GDN_PATH_COOP_CHAIN_ONLY 9 /* measurement aid: COOP with its prepare roles switched off, on the
                                    workspace an earlier call with the same arguments and scratch left  */

/* option bits of gdn_chunk_fwd_sm100_ex */
#define GDN_FLAG_QK_L2NORM 1u    /* normalise every q and k head vector: x * rsqrt(sum x^2 + 1e-6)    */
#define GDN_FLAG_GATE_ACTIVATIONS 2u /* g and beta hold raw values: g = -softplus(g), beta = sigmoid(beta) inside */

#define GDN_PATH_DECODE 11       /* token-by-token fp32 kernel laid out for HBM: one or a few new tokens on top
                                    of a stored state (exact; time grows with S)                         */

#define GDN_PATH_TWOPASS_T 12    /* prepare kernel + transposed chain kernel: one CTA per (batch, value head)
                                    carries all 128 value columns, state-dependent operands in tensor memory */

#define GDN_PATH_PREPARE_ONLY_T 13 /* measurement aid: only the prepare kernel as TWOPASS_T runs it          */
#define GDN_PATH_CHAIN_ONLY_T 14   /* measurement aid: only the transposed chain, on the workspace an earlier
                                      TWOPASS_T / PREPARE_ONLY_T call with the same arguments and scratch left */

#define GDN_D 128                /* head dimension of keys and values (compile-time in the kernels) */
#define GDN_CHUNK 64             /* tokens per chunk                                                */

/*
 * Bytes of scratch gdn_chunk_fwd_sm100 needs for a problem.  256-byte aligned device memory,
 * owned by the caller, reusable across calls on the same stream.
 * Stands in for the workspace tensors the reference allocates inside its host wrapper
 * (csrc/gdn_chunk/gdn_ops.cu:324-336, :812-813).
 */
size_t gdn_chunk_scratch_bytes(int B, int S, int Hq, int Hv, int path);

/*
 * Byte offsets, inside the scratch buffer, of the per-chunk arrays the prepare kernel writes and the
 * chain kernel reads (paths AUTO and TWOPASS_*): offsets[0] W bf16 [tiles][64][128], [1] P bf16
 * [tiles][64][64], [2] U bf16 [tiles][64][128], [3] per-token factors fp32 [tiles][256], [4] total
 * bytes; tile = (b*Hv + hv)*ceil(S/64) + chunk.  For stage-level tests of "prepare", which the
 * reference exposes as prepare_workspace (csrc/gdn_chunk/gdn_ops.cu:1026-1030).
 */
int gdn_chunk_workspace_offsets(int B, int S, int Hq, int Hv, size_t* offsets);

/*
 * Forward pass of the chunked gated delta rule.
 *
 *   q, k   [B,S,Hq,128] bf16        v   [B,S,Hv,128] bf16        g, beta [B,S,Hv] bf16 or fp32
 *   h0     [B,Hv,128,128] fp32 (Dk rows, Dv columns) or NULL for a zero initial state
 *   out    [B,S,Hv,128] bf16        hT  [B,Hv,128,128] fp32 or NULL when the final state is not wanted
 *
 * g is the log decay (<= 0), beta the update gate; q is scaled by 128^-0.5 inside; v-head h reads
 * qk-head h / (Hv/Hq).  S need not be a multiple of 64.  All tensors contiguous, 16-byte aligned.
 * Launches on `stream` (a cudaStream_t) of the current device and returns without waiting.
 *
 * Replaces the production entry of the reference's extension, forward_gdn_chunk_auto
 * (csrc/gdn_chunk/gdn_ops.cu:969-1017), and the launchers beneath it: gdn_chunk_forward
 * (csrc/gdn_chunk/gdn_kernel.cu:2855), gdn_chunk_replay_fused (gdn_kernel.cu:2929-2961) and the
 * scan stages (csrc/gdn_chunk/gdn_scan_stage1.cu:562, gdn_scan_stage2.cu:228).  Extends them with
 * an initial state and an fp32 final state, as the reference's torch definition has
 * (gdn_qsa_sm80/reference/gdn_chunk_ref.py:20-31).
 */
int gdn_chunk_fwd_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                        const float* h0, void* out, float* hT, void* scratch, size_t scratch_bytes,
                        int B, int S, int Hq, int Hv, int gate_dtype, int path, void* stream);

/*
 * gdn_chunk_fwd_sm100 with option bits.  GDN_FLAG_QK_L2NORM: q and k are L2-normalised per token and
 * head inside the kernels (fp32, x * rsqrt(sum x^2 + 1e-6)), as use_qk_l2norm_in_kernel does in the
 * reference's torch definition (gdn_qsa_sm80/reference/gdn_chunk_ref.py:15-17, :43-45, :116-118); the
 * reference's CUDA kernels expect normalised inputs and have no such switch, so callers there normalise
 * in a separate pass over q and k.  GDN_FLAG_GATE_ACTIVATIONS: g and beta are the layer's raw gate
 * projections and the kernels apply g = -softplus(g), beta = sigmoid(beta) in fp32 where they load them (no
 * counterpart in the reference, whose callers run these element-wise passes beforehand).
 * Unknown bits are rejected.  flags = 0 is gdn_chunk_fwd_sm100.
 */
int gdn_chunk_fwd_sm100_ex(const void* q, const void* k, const void* v, const void* g, const void* beta,
                           const float* h0, void* out, float* hT, void* scratch, size_t scratch_bytes,
                           int B, int S, int Hq, int Hv, int gate_dtype, int path, unsigned flags, void* stream);

/*
 * The forward pass on HOST buffers, pipelined.  q, k, v, g, beta, h0, out, hT are HOST pointers with the
 * shapes and dtypes of gdn_chunk_fwd_sm100 (page-locked memory is needed for the copies to overlap; pageable
 * memory works but serialises); `arena` is DEVICE memory of gdn_chunk_host_arena_bytes(...) bytes, 256-byte
 * aligned, owned by the caller.  The sequence is cut into segments of seg_tokens tokens (a multiple of 64;
 * 0 = the library picks four segments); the inputs of segment i+1, the kernels of segment i and the
 * outputs of segment i-1 travel at the same time, each segment starting from the fp32 state the one before
 * ended with (exact).  Kernels run on `stream`, the copies on two internal streams of the device; the call
 * returns without waiting and everything enqueued on `stream` afterwards runs after the last output byte has
 * reached host memory - synchronise `stream` before reading out / hT on the host.  One status word at the
 * start of the arena collects the bounded-wait reports of all segments (gdn_chunk_read_status(arena, ...)).
 * Calls that share an arena must be issued on the same stream.  Calls with different arenas on different
 * streams may be in flight together: their kernels overlap the other call's copies, while the copies
 * themselves share one queue per direction and device (one internal stream each way); with two calls in flight one
 * segment per call (seg_tokens = S) uses the link best, with one call at a time the default of four does.  After an error return
 * the caller's stream is still ordered behind every copy the call had enqueued.
 * flags as in gdn_chunk_fwd_sm100_ex.
 * Replaces what a caller of the reference writes around it by hand: `.cuda()` on every input, the operator,
 * `.cpu()` on the results (the reference's benchmarks create their tensors on the device,
 * benchmarks/bench_gdn_chunk.py:23-27, and leave the host link out of the picture).
 */
size_t gdn_chunk_host_arena_bytes(int B, int S, int Hq, int Hv, int gate_dtype, int seg_tokens);
int gdn_chunk_fwd_host_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                             const float* h0, void* out, float* hT, void* arena, size_t arena_bytes, int B, int S,
                             int Hq, int Hv, int gate_dtype, int seg_tokens, unsigned flags, void* stream);

/*
 * Gated RMS normalisation of rows of 128 bf16 values, the step after gdn_chunk in the layer:
 *   out[r,:] = y[r,:] * rsqrt(mean(y[r,:]^2) + eps) * weight[:] * silu(z[r,:]),   fp32 arithmetic.
 * y, z, out [n_rows][128] bf16 (out may be y), weight [128] bf16, all 16-byte aligned.
 * Replaces the reference's rmsnorm_gated (csrc/output_gate/output_gate.cu:47-98, Python wrapper
 * gdn_qsa_sm80/output_gate_interface.py:15-27; its eps is the constant 1e-6).
 */
int gdn_rmsnorm_gated_sm100(const void* y, const void* z, const void* weight, void* out, long long n_rows,
                            float eps, void* stream);

/*
 * gdn_chunk_fwd_sm100_ex followed by the gated normalisation of its output, as one call: `out` receives
 * rmsnorm_gated(O, z, weight) with O the operator's output (z [B,S,Hv,128] bf16, weight [128] bf16).  The
 * normalisation runs right behind the forward pass on the same stream and in place, while O is still in L2.
 * Stands in for the reference's sequence gdn_chunk -> rmsnorm_gated (README.md:127-139 and :184-190).
 */
int gdn_chunk_fwd_gated_sm100(const void* q, const void* k, const void* v, const void* g, const void* beta,
                              const float* h0, const void* z, const void* weight, float eps, void* out, float* hT,
                              void* scratch, size_t scratch_bytes, int B, int S, int Hq, int Hv, int gate_dtype,
                              int path, unsigned flags, void* stream);

/*
 * *out_max (device) = max over the n_rows rows of k [n_rows][128] bf16 of the row's sum of squares, fp32.
 * Premise check of the exact decay bound that lets the two-level and sequence-parallel drivers skip work
 * (||I - beta k k^T|| <= 1 needs beta |k|^2 <= 2).  Launches on `stream`, does not wait.  The reference has
 * no counterpart: its reset test measures max|A| after computing A (csrc/gdn_chunk/gdn_scan_stage3_reset.cu:22-54).
 */
int gdn_key_norm_sq_max_sm100(const void* k, long long n_rows, float* out_max, void* stream);

/*
 * After how many leading 64-token chunks has every (batch, value head) of the stretch g, beta [B][S][Hv] (gate_dtype
 * as in gdn_chunk_fwd_sm100) forgotten the state it started from: result[0] (device) = the first chunk c with
 * sum_{t < 64 (c + 1)} g < -115 for all b, h, or ceil(S/64) if there is none; result[1] = 1 when the premise of the
 * bound holds (g <= 0, beta >= 0, max beta * *kk_max <= 2; kk_max = NULL stands for keys of unit norm, e.g. from
 * gdn_key_norm_sq_max_sm100 otherwise).  scratch: B * ceil(S/64) * Hv + 2 floats of device memory.  Two small
 * launches on `stream`, no wait.  Used by the sequence-parallel driver to let a rank leave the serial ripple; the
 * reference's counterpart is its measured reset test (csrc/gdn_chunk/gdn_scan_stage3_reset.cu:22-54).
 */
int gdn_forgetting_horizon_sm100(const void* g, const void* beta, int gate_dtype, int B, int S, int Hv,
                                 const float* kk_max, float* scratch, int* result, void* stream);

/*
 * Second level of the two-level chunk scan.  A [n_seq][G][128][128] and Bm (same shape), fp32: group g
 * of sequence s maps its incoming state to its outgoing state by S_out = A S_in + Bm.  Writes the
 * state every group starts from into s_in [n_seq][G][128][128] and the state after the last group
 * into s_final [n_seq][128][128] (may be NULL); h0 [n_seq][128][128] is the state before group 0
 * (NULL = zeros).  n_seq = batch * value heads (<= 65535).  Launches on `stream`, does not wait.
 * Replaces the reference's affine prefix scans over (A_g, B_g): gdn_scan_stage2
 * (csrc/gdn_chunk/gdn_scan_stage2.cu:228) and gdn_scan_stage2_blelloch
 * (csrc/gdn_chunk/gdn_scan_stage2_blelloch.cu:487-522).
 */
int gdn_chunk_scan_transfers(const float* A, const float* Bm, const float* h0, float* s_in, float* s_final,
                             int n_seq, int G, void* stream);

/*
 * The same forward pass for callers that cannot hand over scratch memory and must not trigger an
 * allocation: for instance a serving runtime that carved up all device memory at start-up and only
 * passes fixed input/output buffers to its plugins, or a latency-critical loop where cudaMalloc (a
 * device-wide synchronisation) is not acceptable.  The workspace is a fixed 16 MiB array inside the
 * library's device image (held by every GPU that loads the library, for the life of the process), so
 * the problem must satisfy  B * Hv * ceil(S/64) <= 399  (e.g. 4 value heads x 6144 tokens); larger
 * problems return GDN_ERR_SCRATCH and launch nothing.  Arguments and results are those of
 * gdn_chunk_fwd_sm100 with path = GDN_PATH_AUTO.  The call itself allocates nothing.
 * The first call on each device looks up the array's device address (a one-time set-up step); make
 * that first call outside any stream capture.  All calls on a device share the array: do not let two
 * of them overlap on the GPU (e.g. on different streams).
 * This entry point has no counterpart in the reference, which allocates its workspaces with torch
 * inside every call.
 */
int gdn_chunk_fwd_sm100_noalloc(const void* q, const void* k, const void* v, const void* g, const void* beta,
                                const float* h0, void* out, float* hT, int B, int S, int Hq, int Hv,
                                int gate_dtype, void* stream);

/*
 * Synchronises `stream`, then copies the device status word kept at the start of `scratch` into
 * *device_status (0 = no kernel reported a problem).  Returns GDN_ERR_DEVICE when it is non-zero.
 * Counterpart of C10_CUDA_KERNEL_LAUNCH_CHECK after the reference's launches
 * (csrc/gdn_chunk/gdn_ops.cu:382, :862).
 */
int gdn_chunk_read_status(const void* scratch, void* stream, int* device_status);

/* Static description of a status code (host pointer, never NULL). */
const char* gdn_chunk_error_string(int status);

/* Number of kernels this library has launched in this process so far (all devices). */
unsigned long long gdn_chunk_kernel_launches(void);

/*
 * Diagnostic, effective only in a library built with -DGDN_DIAGNOSTICS (python -m gdn_qsa_sm80_b200.build
 * --diagnostics; a production build compiles none of the accounting in): when `device_buffer` (128 x int64,
 * device memory) is not NULL, one CTA of every later launch writes the SM clock cycles some of its threads
 * spent in each phase of the chunk loop, summed over chunks.  NULL switches it off.  Process-wide, not thread-safe.
 * Plays the role of the temporary clock64() instrumentation the reference's authors describe
 * (docs/VALIDATION_LOG.md:108-109).
 */
void gdn_chunk_set_phase_profile(void* device_buffer);

/*
 * Diagnostic: one UMMA (tcgen05.mma) product with operands laid out by the library's own
 * shared-memory layout helpers, for checking descriptors in isolation.  Synchronises.
 *
 *   a_rowmajor [M][K] bf16, b_rowmajor [N][K] bf16 (device) ; d_out [128][N] fp32 (device):
 *   TMEM lanes 0..127 as read back, so an M = 64 product shows where its rows live.
 *   a_major / b_major: 0 = K-major (128-byte swizzled rows), 1 = MN-major; a_major 2 = A held in tensor memory
 *   (K-major, M = 128, thread staging only), 3 = the same with the instruction's negate-A bit set;
 *   b_span: bytes per row of the MN-major B tile (128 or 64); use_tma != 0 stages the tiles
 *   with TMA instead of thread stores.
 * No counterpart in the reference (it unit-tests layouts by hand, csrc/gdn_chunk/gdn_scan_stage1.cu:238-245).
 */
int gdn_umma_probe(const void* a_rowmajor, const void* b_rowmajor, float* d_out, int* status_word,
                   int M, int N, int K, int a_major, int b_major, int b_span, int use_tma, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GDN_CHUNK_SM100_H */
