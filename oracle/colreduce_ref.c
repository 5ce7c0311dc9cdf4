/*
 * Plain-C restatement of the reference's definition of the operator, kept
 * independent of PyTorch so that the Python oracle has a second opinion.
 *
 * TEST INFRASTRUCTURE ONLY: built into oracle/_build/libcolreduce_ref.so by
 * oracle/build_oracle.py and loaded by tests; never linked into the product.
 *
 * Follows z-lab/flash-colreduce flash_colreduce/naive.py:8-40:
 *   :19     score(i,j) = sum_d q[i,d] * k[j,d] * scale
 *   :20-24  causal: key j is masked for query i when i + max(N-M,0) < j
 *   :25     softmax over j (here: max-subtracted, in double precision)
 *   :27-37  fold over i: sum / mean / max; mean divisor M for the first max(N-M,0)
 *           columns and for every column when not causal, else N-c, ..., 1
 *
 * Pinning: checked against tests/golden/naive_golden.npz (outputs of the
 * reference's naive_colreduce) by tests/test_oracle.py.
 *
 * reduction: 0 sum, 1 mean, 2 max.  q: (B*H, M, D), k: (B*H, N, D) row-major
 * floats; out: (B*H, N) doubles.  Returns 0, or 1 on bad arguments.
 */
#include <math.h>
#include <stdlib.h>

int colreduce_ref(const float* q, const float* k, double* out, int BH, int M, int N, int D,
                  int reduction, int is_causal, double scale) {
  if (!q || !k || !out || BH <= 0 || M <= 0 || N <= 0 || D <= 0 || reduction < 0 || reduction > 2)
    return 1;
  const int c = N > M ? N - M : 0;
  int status = 0;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < BH; ++bh) {
    double* row = (double*)malloc(sizeof(double) * (size_t)N);
    double* o = out + (size_t)bh * N;
    if (!row) {
      status = 1;
      continue;
    }
    for (int j = 0; j < N; ++j) o[j] = 0.0;
    for (int i = 0; i < M; ++i) {
      const float* qi = q + ((size_t)bh * M + i) * D;
      int nvis = N;
      if (is_causal) {
        long lim = (long)i + c + 1; /* keys 0 .. i + c */
        nvis = lim < N ? (int)lim : N;
      }
      double mx = -INFINITY;
      for (int j = 0; j < nvis; ++j) {
        const float* kj = k + ((size_t)bh * N + j) * D;
        double s = 0.0;
        for (int d = 0; d < D; ++d) s += (double)qi[d] * (double)kj[d];
        s *= scale;
        row[j] = s;
        if (s > mx) mx = s;
      }
      double den = 0.0;
      for (int j = 0; j < nvis; ++j) {
        row[j] = exp(row[j] - mx);
        den += row[j];
      }
      for (int j = 0; j < nvis; ++j) {
        const double p = row[j] / den;
        if (reduction == 2) {
          if (p > o[j]) o[j] = p;
        } else {
          o[j] += p;
        }
      }
    }
    if (reduction == 1) {
      for (int j = 0; j < N; ++j) {
        double div = (double)M;
        if (is_causal && j >= c) div = (double)(N - j);
        o[j] /= div;
      }
    }
    free(row);
  }
  return status;
}
