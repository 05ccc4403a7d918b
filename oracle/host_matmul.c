/* TEST INFRASTRUCTURE — not part of the product path.
 *
 * CPU restatement of the GEMM the reference generates, used only as the checker
 * in tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg.
 *
 * Follows, in plain C:
 *   - the naive GEMM definition the reference lowers from: loop order i, j, k,
 *     C initialised to 0, one multiply then one add per k
 *     (src/lib/Operators/Matmul.cc:41-66; A indexed [k][i] when transposed, :52-57);
 *   - hostMatmul, the reference's own CPU check: C[i*N+j] += A[k*M+i] * B[k*N+j]
 *     (matmul.cpp:2351-2360), which accumulates into whatever C holds.
 *
 * Pinning: oracle/build_oracle.py compiles the reference's hostMatmul from the
 * reference tree into oracle/_ref/ when that tree is present; the fixtures under
 * tests/golden/ are its outputs, and this file reproduces them bit for bit
 * (both built with -ffp-contract=off). The reference holds no golden vectors of
 * its own for this path.
 */
#include <stddef.h>
#include <string.h>

#define KCG_ORACLE_DEFINE(NAME, T)                                                            \
  void NAME(const T* A, const T* B, T* C, int M, int N, int K, int a_transposed,              \
            int accumulate) {                                                                 \
    if (!accumulate) memset(C, 0, (size_t)M * (size_t)N * sizeof(T));                         \
    for (int i = 0; i < M; i++) {                                                             \
      for (int j = 0; j < N; j++) {                                                           \
        T acc = C[(size_t)i * N + j];                                                         \
        for (int k = 0; k < K; k++) {                                                         \
          const T a = a_transposed ? A[(size_t)k * M + i] : A[(size_t)i * K + k];             \
          const T prod = a * B[(size_t)k * N + j];                                            \
          acc = acc + prod;                                                                   \
        }                                                                                     \
        C[(size_t)i * N + j] = acc;                                                           \
      }                                                                                       \
    }                                                                                         \
  }

KCG_ORACLE_DEFINE(kcg_oracle_matmul_f32, float)
KCG_ORACLE_DEFINE(kcg_oracle_matmul_f64, double)

/* fp32 inputs, fp64 accumulation: the "fp64 host GEMM" the fp32 results are judged against. */
void kcg_oracle_matmul_f32_acc64(const float* A, const float* B, double* C, int M, int N, int K,
                                 int a_transposed) {
  for (int i = 0; i < M; i++) {
    for (int j = 0; j < N; j++) {
      double acc = 0.0;
      for (int k = 0; k < K; k++) {
        const double a = a_transposed ? (double)A[(size_t)k * M + i] : (double)A[(size_t)i * K + k];
        acc = acc + a * (double)B[(size_t)k * N + j];
      }
      C[(size_t)i * N + j] = acc;
    }
  }
}

/* The reference's verify(): count of |host - device| >= tol (matmul.cpp:2363-2383, tol 0.01). */
long kcg_oracle_verify_f32(const float* host, const float* device, int M, int N, double tol) {
  long bad = 0;
  for (long idx = 0; idx < (long)M * N; idx++) {
    double d = (double)host[idx] - (double)device[idx];
    if (d < 0) d = -d;
    if (d >= tol) bad++;
  }
  return bad;
}
