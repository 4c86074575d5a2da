/* CPU oracle for triangle attention in plain C (TEST INFRASTRUCTURE, not product code).
 *
 * Restates the reference's definition of the op, reference_tt_attn
 * (flash_tt_attn.py:845-864): logits = q.k^T * sm_scale + bias (853-857, bias shared by
 * all L1 rows), P = softmax over keys (860), O = P.V (863); and the gradients autograd
 * derives from it, which are what the reference's backward kernels compute
 * (flash_tt_attn.py:338-359, 414-430):
 *   dV = P^T dO, dP = dO V^T, delta = rowsum(dO*O), dS = P*(dP-delta),
 *   dQ = sm_scale dS K, dK = sm_scale dS^T Q, dBias[b,h,j,k] = sum_i dS[b,h,i,j,k].
 *
 * Inputs and outputs are float32, row-major contiguous, q/k/v/o/do of shape
 * (B,H,L1,L2,D) and bias of shape (B,H,L2,L2). The logits are rounded to float32 where the
 * reference's float32 tensors round them; all sums are carried in double, so the result is
 * the reference's answer for the float32 inputs to well below the tolerances the tests use. Rows (b,h,i) run in parallel under OpenMP; dBias is reduced
 * over threads in a fixed order.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC (oracle/c_oracle.py: build()). Loaded through ctypes by
 * tests/, by the smoke check and by the benchmark's cpu_baseline leg only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LOG2E 1.4426950408889634

int tt_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* One row problem: q,k,v (L2,D), bias (L2,L2). p is scratch (L2,L2) doubles. */
static void row_softmax(const float* q, const float* k, const float* bias, int L2, int D,
                        double scale, double* p, float* lse2) {
  for (int j = 0; j < L2; ++j) {
    double* pj = p + (size_t)j * L2;
    const float* qj = q + (size_t)j * D;
    double m = -INFINITY;
    for (int n = 0; n < L2; ++n) {
      const float* kn = k + (size_t)n * D;
      double s = 0.0;
      for (int d = 0; d < D; ++d) s += (double)qj[d] * (double)kn[d];
      /* The reference forms the logits in the tensors' dtype before its float32 softmax:
       * qk (853), qk * sm_scale (856), + bias (857), each a float32 tensor here. Those three
       * roundings only matter for keys masked with a huge negative bias (-1e9 absorbs the
       * q.k term entirely: a fully masked row gets the uniform distribution), and there they
       * ARE the reference's answer, so they are reproduced; everything after is in double. */
      const float qk = (float)s;
      const float qk_scaled = qk * (float)scale;
      const float logit = qk_scaled + bias[(size_t)j * L2 + n];
      s = (double)logit;
      pj[n] = s;
      if (s > m) m = s;
    }
    double l = 0.0;
    for (int n = 0; n < L2; ++n) {
      pj[n] = exp(pj[n] - m);
      l += pj[n];
    }
    double inv = 1.0 / l;
    for (int n = 0; n < L2; ++n) pj[n] *= inv;
    if (lse2) lse2[j] = (float)((m + log(l)) * LOG2E); /* base-2, flash_tt_attn.py:258 */
  }
}

int tt_oracle_forward(const float* q, const float* k, const float* v, const float* bias,
                      int B, int H, int L1, int L2, int D, float sm_scale, float* o,
                      float* lse2 /* may be NULL; (B,H,L1,L2) */) {
  if (B <= 0 || H <= 0 || L1 <= 0 || L2 <= 0 || D <= 0) return -1;
  const size_t row = (size_t)L2 * D;
  const long nrows = (long)B * H * L1;
  int err = 0;
#pragma omp parallel
  {
    double* p = (double*)malloc(sizeof(double) * (size_t)L2 * L2);
    double* acc = (double*)malloc(sizeof(double) * (size_t)D);
    if (!p || !acc) {
#pragma omp atomic write
      err = 1;
    } else {
#pragma omp for schedule(static)
      for (long r = 0; r < nrows; ++r) {
        const long bh = r / L1;
        const float* bb = bias + (size_t)bh * L2 * L2;
        row_softmax(q + r * row, k + r * row, bb, L2, D, (double)sm_scale, p,
                    lse2 ? lse2 + (size_t)r * L2 : NULL);
        for (int j = 0; j < L2; ++j) {
          for (int d = 0; d < D; ++d) acc[d] = 0.0;
          for (int n = 0; n < L2; ++n) {
            const double pv = p[(size_t)j * L2 + n];
            const float* vn = v + r * row + (size_t)n * D;
            for (int d = 0; d < D; ++d) acc[d] += pv * (double)vn[d];
          }
          for (int d = 0; d < D; ++d) o[r * row + (size_t)j * D + d] = (float)acc[d];
        }
      }
    }
    free(p);
    free(acc);
  }
  return err ? -2 : 0;
}

int tt_oracle_forward_backward(const float* q, const float* k, const float* v,
                               const float* bias, const float* dout, int B, int H, int L1,
                               int L2, int D, float sm_scale, float* o, float* dq, float* dk,
                               float* dv, float* dbias) {
  if (B <= 0 || H <= 0 || L1 <= 0 || L2 <= 0 || D <= 0) return -1;
  const size_t row = (size_t)L2 * D;
  const size_t plane = (size_t)L2 * L2;
  const double scale = (double)sm_scale;
  int nthreads = tt_oracle_num_threads();
  double* partial = (double*)calloc((size_t)nthreads * plane, sizeof(double));
  if (!partial) return -2;
  int err = 0;
  for (long bh = 0; bh < (long)B * H; ++bh) {
    memset(partial, 0, sizeof(double) * (size_t)nthreads * plane);
    const float* bb = bias + (size_t)bh * plane;
#pragma omp parallel
    {
#ifdef _OPENMP
      const int t = omp_get_thread_num();
#else
      const int t = 0;
#endif
      double* mydb = partial + (size_t)t * plane;
      double* p = (double*)malloc(sizeof(double) * plane);
      double* ds = (double*)malloc(sizeof(double) * plane);
      double* acc = (double*)malloc(sizeof(double) * (size_t)D);
      double* orow = (double*)malloc(sizeof(double) * (size_t)D);
      if (!p || !ds || !acc || !orow) {
#pragma omp atomic write
        err = 1;
      } else {
#pragma omp for schedule(static)
        for (int i = 0; i < L1; ++i) {
          const size_t r = (size_t)bh * L1 + i;
          const float *qr = q + r * row, *kr = k + r * row, *vr = v + r * row,
                      *dor = dout + r * row;
          row_softmax(qr, kr, bb, L2, D, scale, p, NULL);
          /* O, delta, dP, dS, dQ per query row */
          for (int j = 0; j < L2; ++j) {
            const double* pj = p + (size_t)j * L2;
            double* dsj = ds + (size_t)j * L2;
            for (int d = 0; d < D; ++d) orow[d] = 0.0;
            for (int n = 0; n < L2; ++n)
              for (int d = 0; d < D; ++d) orow[d] += pj[n] * (double)vr[(size_t)n * D + d];
            double delta = 0.0;
            for (int d = 0; d < D; ++d) {
              o[r * row + (size_t)j * D + d] = (float)orow[d];
              delta += orow[d] * (double)dor[(size_t)j * D + d];
            }
            for (int d = 0; d < D; ++d) acc[d] = 0.0;
            for (int n = 0; n < L2; ++n) {
              double dp = 0.0;
              for (int d = 0; d < D; ++d)
                dp += (double)dor[(size_t)j * D + d] * (double)vr[(size_t)n * D + d];
              const double s = pj[n] * (dp - delta);
              dsj[n] = s;
              mydb[(size_t)j * L2 + n] += s;
              for (int d = 0; d < D; ++d) acc[d] += s * (double)kr[(size_t)n * D + d];
            }
            for (int d = 0; d < D; ++d) dq[r * row + (size_t)j * D + d] = (float)(acc[d] * scale);
          }
          /* dK, dV per key row */
          for (int n = 0; n < L2; ++n) {
            for (int d = 0; d < D; ++d) { acc[d] = 0.0; orow[d] = 0.0; }
            for (int j = 0; j < L2; ++j) {
              const double s = ds[(size_t)j * L2 + n];
              const double pp = p[(size_t)j * L2 + n];
              for (int d = 0; d < D; ++d) {
                acc[d] += s * (double)qr[(size_t)j * D + d];
                orow[d] += pp * (double)dor[(size_t)j * D + d];
              }
            }
            for (int d = 0; d < D; ++d) {
              dk[r * row + (size_t)n * D + d] = (float)(acc[d] * scale);
              dv[r * row + (size_t)n * D + d] = (float)orow[d];
            }
          }
        }
      }
      free(p); free(ds); free(acc); free(orow);
    }
    /* fixed-order reduction over threads */
    for (size_t e = 0; e < plane; ++e) {
      double s = 0.0;
      for (int t = 0; t < nthreads; ++t) s += partial[(size_t)t * plane + e];
      dbias[(size_t)bh * plane + e] = (float)s;
    }
  }
  free(partial);
  return err ? -2 : 0;
}
