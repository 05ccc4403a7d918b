// Row softmax, in place: X[r, :] = softmax(scale * X[r, :]) for a row-major matrix of fp16, bf16
// or fp32 values, fp32 arithmetic. It is the middle step of the attention-shaped chain
// Q.K^T -> softmax -> P.V that the reference lists after batched GEMM among its next operators
// (doc/结果汇总.md); the two products on either side of it are batched launches of the GEMM kernels.
//
// HBM-bound elementwise work: one CTA per row at a time (grid-stride over the rows), 16-byte
// loads and stores, the row is read three times (max, sum, normalise) of which the second and
// third hit L1/L2; a 2048-column bf16 row is 4 KB.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/kcg_b200.h"

extern "C" int kcg_internal_fail(int code, const char* msg);
extern "C" void kcg_internal_count_launch(void);

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = kMax ? fmaxf(v, other) : v + other;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) r = kMax ? fmaxf(r, scratch[i]) : r + scratch[i];
  return r;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(T* x, long long rows, int cols, long long ld,
                                                                float scale) {
  constexpr int PER = 16 / static_cast<int>(sizeof(T));  // elements per 16-byte vector
  __shared__ float scratch[kThreads / 32];
  const int nvec = cols / PER;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    uint4* row = reinterpret_cast<uint4*>(x + r * ld);
    float m = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      const uint4 raw = row[v];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < PER; ++j) m = fmaxf(m, scale * to_f32(e[j]));
    }
    m = block_reduce<true>(m, scratch);
    float sum = 0.f;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      const uint4 raw = row[v];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < PER; ++j) sum += __expf(scale * to_f32(e[j]) - m);
    }
    sum = block_reduce<false>(sum, scratch);
    const float inv = 1.f / sum;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      uint4 raw = row[v];
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int j = 0; j < PER; ++j) e[j] = from_f32<T>(__expf(scale * to_f32(e[j]) - m) * inv);
      row[v] = raw;
    }
  }
}

int fail(int code, const std::string& msg) { return kcg_internal_fail(code, msg.c_str()); }

}  // namespace

extern "C" int kcg_softmax_rows(int device, uint64_t stream, uint64_t X, int64_t rows, int cols, int64_t ld,
                                float scale, int dtype) {
  if (!X || rows <= 0 || cols <= 0) return fail(KCG_E_BAD_ARG, "null matrix or empty shape");
  const int eb = dtype == KCG_DTYPE_FLOAT32 ? 4 : 2;
  if (dtype != KCG_DTYPE_FLOAT32 && dtype != KCG_DTYPE_FLOAT16 && dtype != KCG_DTYPE_BFLOAT16)
    return fail(KCG_E_BAD_ARG, "softmax takes float16, bfloat16 or float32 data");
  if (ld == 0) ld = cols;
  if (ld < cols) return fail(KCG_E_BAD_ARG, "leading dimension below the row length");
  if (X % 16 || (static_cast<int64_t>(cols) * eb) % 16 || (ld * eb) % 16)
    return fail(KCG_E_BAD_ARG, "softmax rows must start and end on 16-byte boundaries");
  int prev = -1;
  cudaError_t e = cudaGetDevice(&prev);
  if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  const int grid = static_cast<int>(rows < 148 * 16 ? rows : 148 * 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == KCG_DTYPE_FLOAT32) {
    softmax_rows_kernel<float><<<grid, kThreads, 0, st>>>(reinterpret_cast<float*>(X), rows, cols, ld, scale);
  } else if (dtype == KCG_DTYPE_FLOAT16) {
    softmax_rows_kernel<__half><<<grid, kThreads, 0, st>>>(reinterpret_cast<__half*>(X), rows, cols, ld, scale);
  } else {
    softmax_rows_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(X), rows, cols, ld,
                                                                 scale);
  }
  e = cudaGetLastError();
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("softmax launch: ") + cudaGetErrorString(e));
  kcg_internal_count_launch();
  return 0;
}
