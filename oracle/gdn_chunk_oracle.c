/*
 * CPU oracle for the gdn_chunk forward pass, plain C (fp32 data, fp32 math).
 *
 * TEST INFRASTRUCTURE ONLY: linked by nothing that ships.  The tests, the smoke
 * check and the CPU-baseline leg of the benchmark load it through ctypes.
 *
 * Two restatements of the reference's pure-torch definition of the operator:
 *   gdn_oracle_recurrent_f32  follows gdn_qsa_sm80/reference/gdn_chunk_ref.py:103-147
 *                             (torch_recurrent_gated_delta_rule), one token at a time;
 *   gdn_oracle_chunk_f32      follows gdn_qsa_sm80/reference/gdn_chunk_ref.py:20-100
 *                             (torch_chunk_gated_delta_rule), chunked WY form.
 * Both are pinned against outputs of the real reference stored in tests/golden/.
 *
 * Layouts (row-major, as the reference's tensors):
 *   q, k [B,S,Hk,D]   v, out [B,S,Hv,D]   g, beta [B,S,Hv]   h0, hT [B,Hv,D,D] (Dk rows, Dv columns)
 * v-head h reads qk-head h / (Hv/Hk) (csrc/gdn_chunk/gdn_kernel.cu:385-387).
 * Independent (b, h) sequences are spread over OpenMP threads.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GDN_D 128

int gdn_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* gdn_chunk_ref.py:133-141.  Returns 0, or -1 on bad arguments. */
int gdn_oracle_recurrent_f32(const float* q, const float* k, const float* v, const float* g,
                             const float* beta, const float* h0, float* out, float* hT,
                             int B, int S, int Hk, int Hv, int nthreads) {
    if (B <= 0 || S < 0 || Hk <= 0 || Hv <= 0 || Hv % Hk) return -1;
    const int D = GDN_D, rep = Hv / Hk;
    const float scale = 1.0f / sqrtf((float)D);
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
    (void)nthreads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * Hv; ++bh) {
        const int b = bh / Hv, h = bh % Hv, hk = h / rep;
        float* st = (float*)malloc(sizeof(float) * D * D);
        float kv[GDN_D], dl[GDN_D], o[GDN_D];
        if (h0) memcpy(st, h0 + (size_t)bh * D * D, sizeof(float) * D * D);
        else memset(st, 0, sizeof(float) * D * D);
        for (int i = 0; i < S; ++i) {
            const float* qi = q + (((size_t)b * S + i) * Hk + hk) * D;
            const float* ki = k + (((size_t)b * S + i) * Hk + hk) * D;
            const float* vi = v + (((size_t)b * S + i) * Hv + h) * D;
            const float dec = expf(g[((size_t)b * S + i) * Hv + h]);
            const float bt = beta[((size_t)b * S + i) * Hv + h];
            for (int c = 0; c < D; ++c) kv[c] = 0.f;
            for (int r = 0; r < D; ++r) {
                float* row = st + (size_t)r * D;
                const float kr = ki[r];
                for (int c = 0; c < D; ++c) { row[c] *= dec; kv[c] += row[c] * kr; }
            }
            for (int c = 0; c < D; ++c) { dl[c] = (vi[c] - kv[c]) * bt; o[c] = 0.f; }
            for (int r = 0; r < D; ++r) {
                float* row = st + (size_t)r * D;
                const float kr = ki[r], qr = qi[r] * scale;
                for (int c = 0; c < D; ++c) { row[c] += kr * dl[c]; o[c] += row[c] * qr; }
            }
            memcpy(out + (((size_t)b * S + i) * Hv + h) * D, o, sizeof(float) * D);
        }
        if (hT) memcpy(hT + (size_t)bh * D * D, st, sizeof(float) * D * D);
        free(st);
    }
    return 0;
}

/* gdn_chunk_ref.py:49-94 for one (b, h) sequence at a time; chunk size C (<= 64). */
int gdn_oracle_chunk_f32(const float* q, const float* k, const float* v, const float* g,
                         const float* beta, const float* h0, float* out, float* hT,
                         int B, int S, int Hk, int Hv, int C, int nthreads) {
    if (B <= 0 || S < 0 || Hk <= 0 || Hv <= 0 || Hv % Hk || C <= 0 || C > 64) return -1;
    const int D = GDN_D, rep = Hv / Hk;
    const float scale = 1.0f / sqrtf((float)D);
    const int NT = (S + C - 1) / C;
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
    (void)nthreads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < B * Hv; ++bh) {
        const int b = bh / Hv, h = bh % Hv, hk = h / rep;
        /* per-sequence work buffers */
        float* st = (float*)malloc(sizeof(float) * D * D);
        float* kc = (float*)malloc(sizeof(float) * 64 * D);   /* k chunk (zero padded) */
        float* qc = (float*)malloc(sizeof(float) * 64 * D);   /* scaled q chunk */
        float* W = (float*)malloc(sizeof(float) * 64 * D);    /* k_cumdecay */
        float* U = (float*)malloc(sizeof(float) * 64 * D);    /* new_values, then v_new */
        float* A = (float*)malloc(sizeof(float) * 64 * 64);   /* ut_system (strict lower) */
        float* P = (float*)malloc(sizeof(float) * 64 * 64);   /* intra_chunk_attn */
        float* acc = (float*)malloc(sizeof(float) * D * D);
        float gam[64], bet[64];
        if (h0) memcpy(st, h0 + (size_t)bh * D * D, sizeof(float) * D * D);
        else memset(st, 0, sizeof(float) * D * D);
        for (int t = 0; t < NT; ++t) {
            float run = 0.f;
            for (int i = 0; i < C; ++i) {
                const int s = t * C + i;
                if (s < S) {
                    const size_t tok = (size_t)b * S + s;
                    memcpy(kc + (size_t)i * D, k + (tok * Hk + hk) * D, sizeof(float) * D);
                    for (int d = 0; d < D; ++d) qc[(size_t)i * D + d] = q[(tok * Hk + hk) * D + d] * scale;
                    bet[i] = beta[tok * Hv + h];
                    run += g[tok * Hv + h];
                    for (int d = 0; d < D; ++d) {               /* :56-57, :75 right-hand sides */
                        U[(size_t)i * D + d] = v[(tok * Hv + h) * D + d] * bet[i];
                    }
                } else {                                        /* :49-51 zero padding */
                    memset(kc + (size_t)i * D, 0, sizeof(float) * D);
                    memset(qc + (size_t)i * D, 0, sizeof(float) * D);
                    memset(U + (size_t)i * D, 0, sizeof(float) * D);
                    bet[i] = 0.f;
                }
                gam[i] = run;                                   /* :67 */
                const float e = expf(run) * bet[i];
                for (int d = 0; d < D; ++d) W[(size_t)i * D + d] = kc[(size_t)i * D + d] * e;
            }
            for (int i = 0; i < C; ++i)                         /* :69-74 */
                for (int j = 0; j <= i; ++j) {
                    float kk = 0.f, qk = 0.f;
                    for (int d = 0; d < D; ++d) {
                        kk += kc[(size_t)i * D + d] * kc[(size_t)j * D + d];
                        qk += qc[(size_t)i * D + d] * kc[(size_t)j * D + d];
                    }
                    const float m = expf(gam[i] - gam[j]);
                    A[i * 64 + j] = (j < i) ? kk * bet[i] * m : 0.f;
                    P[i * 64 + j] = qk * m;
                }
            for (int i = 1; i < C; ++i)                         /* :77-78 forward substitution */
                for (int j = 0; j < i; ++j) {
                    const float a = A[i * 64 + j];
                    for (int d = 0; d < D; ++d) {
                        W[(size_t)i * D + d] -= a * W[(size_t)j * D + d];
                        U[(size_t)i * D + d] -= a * U[(size_t)j * D + d];
                    }
                }
            for (int i = 0; i < C; ++i)                         /* :91 v_new = U - W S */
                for (int r = 0; r < D; ++r) {
                    const float w = W[(size_t)i * D + r];
                    const float* row = st + (size_t)r * D;
                    for (int c = 0; c < D; ++c) U[(size_t)i * D + c] -= w * row[c];
                }
            for (int i = 0; i < C; ++i) {                       /* :92-93 output rows */
                const int s = t * C + i;
                if (s >= S) break;
                float o[GDN_D];
                const float eg = expf(gam[i]);
                for (int c = 0; c < D; ++c) o[c] = 0.f;
                for (int r = 0; r < D; ++r) {
                    const float qr = qc[(size_t)i * D + r] * eg;
                    const float* row = st + (size_t)r * D;
                    for (int c = 0; c < D; ++c) o[c] += qr * row[c];
                }
                for (int j = 0; j <= i; ++j) {
                    const float p = P[i * 64 + j];
                    for (int c = 0; c < D; ++c) o[c] += p * U[(size_t)j * D + c];
                }
                memcpy(out + (((size_t)b * S + s) * Hv + h) * D, o, sizeof(float) * D);
            }
            const float cd = expf(gam[C - 1]);                  /* :94 state update */
            for (size_t e = 0; e < (size_t)D * D; ++e) acc[e] = st[e] * cd;
            for (int i = 0; i < C; ++i) {
                const float kd = expf(gam[C - 1] - gam[i]);
                for (int r = 0; r < D; ++r) {
                    const float kr = kc[(size_t)i * D + r] * kd;
                    float* row = acc + (size_t)r * D;
                    for (int c = 0; c < D; ++c) row[c] += kr * U[(size_t)i * D + c];
                }
            }
            memcpy(st, acc, sizeof(float) * D * D);
        }
        if (hT) memcpy(hT + (size_t)bh * D * D, st, sizeof(float) * D * D);
        free(st); free(kc); free(qc); free(W); free(U); free(A); free(P); free(acc);
    }
    return 0;
}
