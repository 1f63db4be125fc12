/*
 * csr_ref.c -- plain C (OpenMP) restatement of the aggregation math over a CSR.
 *
 * TEST INFRASTRUCTURE ONLY: linked by nothing under turbo_gnn_b200/.  It exists so
 * that graphs too large for the [E, F] message tensors of the torch scatter
 * restatement (oracle/scatter_oracle.py) can still be checked, and as an
 * independent second statement of the same formulas.  Every loop is the direct
 * per-destination-row form of:
 *   min/max/sum/mean  src/backends/torch_native_backend/conv.py:472-503
 *   edge softmax      src/backends/torch_native_backend/conv.py:32-68
 *   GATv2 aggregation src/backends/torch_native_backend/conv.py:506-529
 *   GT aggregation    src/backends/torch_native_backend/conv.py:532-552
 * (paths inside the reference project).  Accumulation is in double so the result
 * can serve as ground truth for fp32 kernels.  CSR rows are destinations, columns
 * sources; indices are int64.
 *
 * Build: gcc -O2 -fopenmp -fPIC -shared csr_ref.c -o _build/libcsr_ref.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* reduce: 0 min, 1 max, 2 sum, 3 mean.  x [n_src, f], out [n_rows, f]; arg [n_rows, f] or NULL. */
void ref_segment_reduce(const int64_t *indptr, const int64_t *indices, int64_t n_rows, const float *x, int64_t f,
                        int reduce, float *out, int64_t *arg) {
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t v = 0; v < n_rows; ++v) {
        const int64_t e0 = indptr[v], e1 = indptr[v + 1];
        for (int64_t j = 0; j < f; ++j) {
            if (reduce <= 1) {
                float best = reduce == 0 ? INFINITY : -INFINITY;
                int64_t who = -1;
                for (int64_t e = e0; e < e1; ++e) {
                    const int64_t u = indices[e];
                    const float val = x[u * f + j];
                    const int better = reduce == 0 ? (val < best) : (val > best);
                    if (better || (val == best && who >= 0 && u < who)) {
                        best = val;
                        who = u;
                    }
                }
                out[v * f + j] = who >= 0 ? best : 0.0f;
                if (arg) arg[v * f + j] = who;
            } else {
                double acc = 0.0;
                for (int64_t e = e0; e < e1; ++e) acc += x[indices[e] * f + j];
                if (reduce == 3) acc /= (double)(e1 - e0 > 1 ? e1 - e0 : 1);
                out[v * f + j] = (float)acc;
            }
        }
    }
}

/* GATv2 aggregation.  l [n_rows, h, d], r [n_src, h, d], a [h, d]; out [n_rows, h, d], lse [n_rows, h]. */
void ref_gatv2_forward(const int64_t *indptr, const int64_t *indices, int64_t n_rows, const float *l, const float *r,
                       const float *a, int64_t h, int64_t d, float slope, float *out, float *lse) {
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t v = 0; v < n_rows; ++v) {
        const int64_t e0 = indptr[v], e1 = indptr[v + 1];
        for (int64_t hh = 0; hh < h; ++hh) {
            float *o = out + (v * h + hh) * d;
            for (int64_t k = 0; k < d; ++k) o[k] = 0.0f;
            if (e0 == e1) {
                lse[v * h + hh] = -INFINITY;
                continue;
            }
            double top = -INFINITY;
            double *score = (double *)malloc(sizeof(double) * (size_t)(e1 - e0));
            for (int64_t e = e0; e < e1; ++e) {
                const float *lr = l + (v * h + hh) * d;
                const float *rr = r + (indices[e] * h + hh) * d;
                double s = 0.0;
                for (int64_t k = 0; k < d; ++k) {
                    const double z = (double)lr[k] + (double)rr[k];
                    s += (double)a[hh * d + k] * (z > 0 ? z : z * slope);
                }
                score[e - e0] = s;
                if (s > top) top = s;
            }
            double denom = 0.0;
            for (int64_t e = e0; e < e1; ++e) denom += exp(score[e - e0] - top);
            double *acc = (double *)calloc((size_t)d, sizeof(double));
            for (int64_t e = e0; e < e1; ++e) {
                const double alpha = exp(score[e - e0] - top) / denom;
                const float *rr = r + (indices[e] * h + hh) * d;
                for (int64_t k = 0; k < d; ++k) acc[k] += alpha * rr[k];
            }
            for (int64_t k = 0; k < d; ++k) o[k] = (float)acc[k];
            lse[v * h + hh] = (float)(top + log(denom));
            free(acc);
            free(score);
        }
    }
}

/* Graph-transformer aggregation: score = <q[src], k[dst]> * scale. */
void ref_gt_forward(const int64_t *indptr, const int64_t *indices, int64_t n_rows, const float *q, const float *k,
                    const float *vv, int64_t h, int64_t d, float scale, float *out, float *lse) {
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t v = 0; v < n_rows; ++v) {
        const int64_t e0 = indptr[v], e1 = indptr[v + 1];
        for (int64_t hh = 0; hh < h; ++hh) {
            float *o = out + (v * h + hh) * d;
            for (int64_t c = 0; c < d; ++c) o[c] = 0.0f;
            if (e0 == e1) {
                lse[v * h + hh] = -INFINITY;
                continue;
            }
            double top = -INFINITY;
            double *score = (double *)malloc(sizeof(double) * (size_t)(e1 - e0));
            const float *kr = k + (v * h + hh) * d;
            for (int64_t e = e0; e < e1; ++e) {
                const float *qr = q + (indices[e] * h + hh) * d;
                double s = 0.0;
                for (int64_t c = 0; c < d; ++c) s += (double)qr[c] * (double)kr[c];
                s *= scale;
                score[e - e0] = s;
                if (s > top) top = s;
            }
            double denom = 0.0;
            for (int64_t e = e0; e < e1; ++e) denom += exp(score[e - e0] - top);
            double *acc = (double *)calloc((size_t)d, sizeof(double));
            for (int64_t e = e0; e < e1; ++e) {
                const double alpha = exp(score[e - e0] - top) / denom;
                const float *vr = vv + (indices[e] * h + hh) * d;
                for (int64_t c = 0; c < d; ++c) acc[c] += alpha * vr[c];
            }
            for (int64_t c = 0; c < d; ++c) o[c] = (float)acc[c];
            lse[v * h + hh] = (float)(top + log(denom));
            free(acc);
            free(score);
        }
    }
}
