/*
 * CPU oracle for the gated-linear-attention forward path.  TEST INFRASTRUCTURE ONLY: the
 * product library never links or calls this file.  It restates, in plain C, the token
 * recurrence the reference uses as its own ground truth
 * (engine/gtr/backbone/csrc/test_gla.py:124-132, `_recurrence_fp64`):
 *
 *     S_t = exp(g_t)[:,None] * S_{t-1} + k_t v_t^T        (state [K,V] per batch and head)
 *     o_t = scale * q_t^T S_t
 *
 * extended with an optional initial state / final state (the arguments of the FLA call in
 * engine/gtr/backbone/vit_adapter.py:566-568) and an optional scan-order permutation
 * `perm[p]` = token read at sequence step p (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:88-94).
 *
 * Layouts: q,k,g [B,T,H,K], v,o [B,T,H,V], states [B,H,K,V]; all contiguous.
 * `acc64` selects double accumulation (the reference's fp64 check) or float (the fp32
 * recurrent reference the tolerances are stated against).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define GLA_ORACLE_MAX_D 256

int gla_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static void seq_f32(const float* q, const float* k, const float* v, const float* g, float* o,
                    const float* s0, float* sT, int T, int H, int K, int V, float scale,
                    const int32_t* perm) {
    float* S = (float*)malloc(sizeof(float) * (size_t)K * V);
    float dec[GLA_ORACLE_MAX_D];
    if (s0) memcpy(S, s0, sizeof(float) * (size_t)K * V);
    else memset(S, 0, sizeof(float) * (size_t)K * V);
    for (int p = 0; p < T; ++p) {
        const size_t t = perm ? (size_t)perm[p] : (size_t)p;
        const float* qt = q + t * H * K;
        const float* kt = k + t * H * K;
        const float* gt = g + t * H * K;
        const float* vt = v + t * H * V;
        float* ot = o + t * H * V;
        for (int c = 0; c < K; ++c) dec[c] = expf(gt[c]);
        for (int x = 0; x < V; ++x) ot[x] = 0.f;
        for (int c = 0; c < K; ++c) {
            float* Sc = S + (size_t)c * V;
            const float d = dec[c], kc = kt[c], qc = qt[c];
            for (int x = 0; x < V; ++x) {
                Sc[x] = d * Sc[x] + kc * vt[x];
                ot[x] += qc * Sc[x];
            }
        }
        for (int x = 0; x < V; ++x) ot[x] *= scale;
    }
    if (sT) memcpy(sT, S, sizeof(float) * (size_t)K * V);
    free(S);
}

static void seq_f64(const float* q, const float* k, const float* v, const float* g, float* o,
                    const float* s0, float* sT, int T, int H, int K, int V, float scale,
                    const int32_t* perm) {
    double* S = (double*)malloc(sizeof(double) * (size_t)K * V);
    double dec[GLA_ORACLE_MAX_D], acc[GLA_ORACLE_MAX_D];
    for (size_t i = 0; i < (size_t)K * V; ++i) S[i] = s0 ? (double)s0[i] : 0.0;
    for (int p = 0; p < T; ++p) {
        const size_t t = perm ? (size_t)perm[p] : (size_t)p;
        const float* qt = q + t * H * K;
        const float* kt = k + t * H * K;
        const float* gt = g + t * H * K;
        const float* vt = v + t * H * V;
        float* ot = o + t * H * V;
        for (int c = 0; c < K; ++c) dec[c] = exp((double)gt[c]);
        for (int x = 0; x < V; ++x) acc[x] = 0.0;
        for (int c = 0; c < K; ++c) {
            double* Sc = S + (size_t)c * V;
            const double d = dec[c], kc = kt[c], qc = qt[c];
            for (int x = 0; x < V; ++x) {
                Sc[x] = d * Sc[x] + kc * (double)vt[x];
                acc[x] += qc * Sc[x];
            }
        }
        for (int x = 0; x < V; ++x) ot[x] = (float)((double)scale * acc[x]);
    }
    if (sT) for (size_t i = 0; i < (size_t)K * V; ++i) sT[i] = (float)S[i];
    free(S);
}

/* Returns 0, or -1 on bad arguments.  s0 / sT / perm may be NULL. */
int gla_oracle_forward(const float* q, const float* k, const float* v, const float* g, float* o,
                       const float* s0, float* sT, int B, int T, int H, int K, int V,
                       float scale, const int32_t* perm, int acc64) {
    if (B < 0 || T < 0 || H <= 0 || K <= 0 || V <= 0 || K > GLA_ORACLE_MAX_D || V > GLA_ORACLE_MAX_D)
        return -1;
    if ((long)B * T == 0) return 0;
    if (!q || !k || !v || !g || !o) return -1;
    const long n = (long)B * H;
#pragma omp parallel for schedule(dynamic, 1)
    for (long bh = 0; bh < n; ++bh) {
        const int b = (int)(bh / H), h = (int)(bh % H);
        const size_t offk = (size_t)b * T * H * K + (size_t)h * K;
        const size_t offv = (size_t)b * T * H * V + (size_t)h * V;
        const size_t offs = ((size_t)b * H + h) * K * V;
        if (acc64)
            seq_f64(q + offk, k + offk, v + offv, g + offk, o + offv, s0 ? s0 + offs : 0,
                    sT ? sT + offs : 0, T, H, K, V, scale, perm);
        else
            seq_f32(q + offk, k + offk, v + offv, g + offk, o + offv, s0 ? s0 + offs : 0,
                    sT ? sT + offs : 0, T, H, K, V, scale, perm);
    }
    return 0;
}
