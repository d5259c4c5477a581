/* CPU oracle, C part.  TEST INFRASTRUCTURE ONLY: nothing shipped links this file.
 *
 * Plain-C restatement of the reference project's host-side single-head mLSTM forward
 * (mlstmCpu, cuda-src/cpu_utils.cuh:126-170) with its helpers matmulTranspose (:82-92),
 * cumsum (:95-97), log_sigmoid_cpu (:100-102), compute_d_tilde (:105-113), compute_b (:116-123)
 * and matmul (:69-79).  The arithmetic is fp32 on values the caller has already widened from
 * fp16, like the reference which widens each half on use; the caller rounds H back to fp16.
 *
 * Parity pin: tests compare this function with the reference's own mlstmCpu compiled from the
 * reference checkout (oracle/_ref/libmlstm_ref.so) and with the committed golden vector that
 * binary produced for the reference demo's input recipe.
 *
 * eps_inside_max = 1 gives the host variant n = max(|b|, exp(-m) + 1e-6) (cpu_utils.cuh:157);
 * 0 gives the GPU kernels' n = max(|b|, exp(-m)) + 1e-6 (cuda-src/mlstm_forward.cu:178-179).
 */
#include <float.h>
#include <math.h>
#include <stdlib.h>

int mlstm_cpu_forward(const float *Q, const float *K, const float *V, const float *F,
                      const float *I, float *H, unsigned S, unsigned D, int eps_inside_max)
{
    float *C = (float *)malloc((size_t)S * S * sizeof(float));
    float *Fc = (float *)malloc((size_t)S * sizeof(float));
    float *m = (float *)malloc((size_t)S * sizeof(float));
    float *nrm = (float *)malloc((size_t)S * sizeof(float));
    if (!C || !Fc || !m || !nrm) { free(C); free(Fc); free(m); free(nrm); return -1; }
    const float scale = 1.0f / sqrtf((float)D);

    /* log-sigmoid then inclusive cumulative sum (:143-144) */
    for (unsigned t = 0; t < S; t++) Fc[t] = -logf(1.0f + expf(-F[t]));
    for (unsigned t = 1; t < S; t++) Fc[t] += Fc[t - 1];

#pragma omp parallel for schedule(dynamic, 8)
    for (unsigned r = 0; r < S; r++) {
        /* row maximum of d_tilde over the causal part (:105-113) */
        float mr = -FLT_MAX;
        for (unsigned c = 0; c <= r; c++) {
            float d = Fc[r] - Fc[c] + I[c];
            if (d > mr) mr = d;
        }
        m[r] = mr;
        /* scaled Q K^T (:147) times exp(d_tilde - m) (:152-156); zero above the diagonal */
        float b = 0.0f;
        for (unsigned c = 0; c < S; c++) {
            float x = 0.0f;
            if (c <= r) {
                float acc = 0.0f;
                for (unsigned d = 0; d < D; d++) acc += Q[(size_t)r * D + d] * K[(size_t)c * D + d];
                x = acc * scale * expf(Fc[r] - Fc[c] + I[c] - mr);
            }
            C[(size_t)r * S + c] = x;
            b += x;
        }
        /* normaliser (:157) */
        float e = expf(-mr);
        nrm[r] = eps_inside_max ? fmaxf(fabsf(b), e + 1e-6f) : fmaxf(fabsf(b), e) + 1e-6f;
        for (unsigned c = 0; c <= r; c++) C[(size_t)r * S + c] /= nrm[r];
    }
    /* H = C V (:163) */
#pragma omp parallel for schedule(dynamic, 8)
    for (unsigned r = 0; r < S; r++) {
        for (unsigned d = 0; d < D; d++) H[(size_t)r * D + d] = 0.0f;
        for (unsigned c = 0; c <= r; c++) {
            float w = C[(size_t)r * S + c];
            for (unsigned d = 0; d < D; d++) H[(size_t)r * D + d] += w * V[(size_t)c * D + d];
        }
    }
    free(C); free(Fc); free(m); free(nrm);
    return 0;
}
