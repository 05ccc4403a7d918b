// TEST INFRASTRUCTURE. C entry points around the reference's own hostMatmul template.
// build_oracle.py extracts that function from the reference tree (matmul.cpp, the
// `template <typename T> void hostMatmul(...)` definition) into
// oracle/_ref/hostMatmul_extract.inc at build time and compiles this file against it;
// nothing of the reference is stored in this repository.
#include <cstddef>
#include "_ref/hostMatmul_extract.inc"

extern "C" {
// A is K x M (transposed), B is K x N, C is M x N and is accumulated into (caller zeroes it).
void ref_host_matmul_f32(float* A, float* B, float* C, int M, int N, int K) { hostMatmul<float>(A, B, C, M, N, K); }
void ref_host_matmul_f64(double* A, double* B, double* C, int M, int N, int K) { hostMatmul<double>(A, B, C, M, N, K); }
}
