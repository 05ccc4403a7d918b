// Fused epilogue shared by every GEMM kernel: D = act(alpha * acc + beta * C + bias[col]).
// The reference plans matmul -> bias/ReLU -> matmul graphs but ships no fused epilogue; this
// is the step either side of the GEMM folded into its store. All arithmetic is fp32, in the
// fixed order scale, beta * C, bias, ReLU; callers test p.epi_flags != 0 first, so that the
// plain GEMM pays one uniform branch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_params.h"

namespace kcg {

__device__ __forceinline__ float epi_to_f32(float x) { return x; }
__device__ __forceinline__ float epi_to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float epi_to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

// N consecutive values of type T starting at src -> fp32. 16-byte loads when the span allows
// (callers keep src 16-byte aligned then), scalar loads otherwise.
template <typename T, int N>
__device__ __forceinline__ void epi_load_span(const T* src, float (&out)[N]) {
  constexpr int PER = 16 / static_cast<int>(sizeof(T));
  if constexpr (N % PER == 0) {
#pragma unroll
    for (int i = 0; i < N / PER; ++i) {
      const uint4 raw = reinterpret_cast<const uint4*>(src)[i];  // plain load: C is written later by this kernel
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < PER; ++j) out[i * PER + j] = epi_to_f32(e[j]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = epi_to_f32(src[i]);
  }
}

// v holds the accumulators of C[row, col .. col + N).
template <typename OutT, int N>
__device__ __forceinline__ void epi_span(const KcgGemmParams& p, float (&v)[N], int row, int col) {
  const unsigned int f = p.epi_flags;
  if (f & KCG_EPI_SCALE) {
    const float alpha = p.alpha, beta = p.beta;
    if (beta != 0.f) {
      float cv[N];
      epi_load_span<OutT, N>(reinterpret_cast<const OutT*>(p.C) + static_cast<size_t>(row) * p.ldc + col, cv);
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] = fmaf(beta, cv[i], alpha * v[i]);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] *= alpha;
    }
  }
  if (f & KCG_EPI_BIAS) {
    float bv[N];
    epi_load_span<OutT, N>(reinterpret_cast<const OutT*>(p.bias) + col, bv);
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] += bv[i];
  }
  if (f & KCG_EPI_RELU) {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = fmaxf(v[i], 0.f);
  }
}

}  // namespace kcg
