// Row softmax: Y[r, :] = softmax(scale * X[r, :]) for row-major matrices of fp16, bf16 or fp32 values
// (in place, or from one matrix into another of another type - fp32 scores in, 16-bit probabilities out),
// fp32 arithmetic. It is the middle step of the attention-shaped chain
// Q.K^T -> softmax -> P.V that the reference lists after batched GEMM among its next operators
// (doc/结果汇总.md); the two products on either side of it are batched launches of the GEMM kernels.
//
// HBM-bound elementwise work: one CTA per row at a time (grid-stride over the rows), 16-byte
// loads and stores of eight values at a time, the row is read three times (max, sum, normalise) of which the second and
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

__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
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

// Eight consecutive values of a row: one 16-byte vector of a 16-bit type, two of fp32.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_f32(e[j]);
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(v[j]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
}

// Y[r, :] = softmax(scale * X[r, :]); Y may be X (same type) or another matrix of another type.
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(const Tin* x, long long ldx, Tout* y, long long ldy,
                                                                long long rows, int cols, float scale) {
  __shared__ float scratch[kThreads / 32];
  const int nvec = cols / 8;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const Tin* row = x + r * ldx;
    Tout* out = y + r * ldy;
    float m = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float e[8];
      load8(row + 8 * v, e);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, scale * e[j]);
    }
    m = block_reduce<true>(m, scratch);
    float sum = 0.f;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float e[8];
      load8(row + 8 * v, e);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += __expf(scale * e[j] - m);
    }
    sum = block_reduce<false>(sum, scratch);
    const float inv = 1.f / sum;
    for (int v = threadIdx.x; v < nvec; v += kThreads) {
      float e[8];
      load8(row + 8 * v, e);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __expf(scale * e[j] - m) * inv;
      store8(out + 8 * v, e);
    }
  }
}

int fail(int code, const std::string& msg) { return kcg_internal_fail(code, msg.c_str()); }

template <typename Tin>
void launch_for_output(int grid, cudaStream_t st, const Tin* x, int64_t ldx, uint64_t Y, int dtype_out, int64_t ldy,
                       int64_t rows, int cols, float scale) {
  if (dtype_out == KCG_DTYPE_FLOAT32) {
    softmax_rows_kernel<Tin, float><<<grid, kThreads, 0, st>>>(x, ldx, reinterpret_cast<float*>(Y), ldy, rows, cols, scale);
  } else if (dtype_out == KCG_DTYPE_FLOAT16) {
    softmax_rows_kernel<Tin, __half><<<grid, kThreads, 0, st>>>(x, ldx, reinterpret_cast<__half*>(Y), ldy, rows, cols,
                                                              scale);
  } else {
    softmax_rows_kernel<Tin, __nv_bfloat16><<<grid, kThreads, 0, st>>>(x, ldx, reinterpret_cast<__nv_bfloat16*>(Y), ldy,
                                                                     rows, cols, scale);
  }
}

bool known_dtype(int dt) { return dt == KCG_DTYPE_FLOAT32 || dt == KCG_DTYPE_FLOAT16 || dt == KCG_DTYPE_BFLOAT16; }

}  // namespace

extern "C" int kcg_softmax_rows_ex(int device, uint64_t stream, uint64_t X, int dtype_in, int64_t ldx, uint64_t Y,
                                   int dtype_out, int64_t ldy, int64_t rows, int cols, float scale) {
  if (!X || !Y || rows <= 0 || cols <= 0) return fail(KCG_E_BAD_ARG, "null matrix or empty shape");
  if (!known_dtype(dtype_in) || !known_dtype(dtype_out))
    return fail(KCG_E_BAD_ARG, "softmax takes float16, bfloat16 or float32 data");
  const int eb_in = dtype_in == KCG_DTYPE_FLOAT32 ? 4 : 2, eb_out = dtype_out == KCG_DTYPE_FLOAT32 ? 4 : 2;
  if (ldx == 0) ldx = cols;
  if (ldy == 0) ldy = cols;
  if (ldx < cols || ldy < cols) return fail(KCG_E_BAD_ARG, "leading dimension below the row length");
  if (cols % 8 || X % 16 || Y % 16 || (ldx * eb_in) % 16 || (ldy * eb_out) % 16)
    return fail(KCG_E_BAD_ARG, "softmax rows must hold a multiple of 8 values and start on 16-byte boundaries");
  if (X == Y && (dtype_in != dtype_out || ldx != ldy))
    return fail(KCG_E_BAD_ARG, "an in-place softmax keeps the type and the pitch of the matrix");
  int prev = -1;
  cudaError_t e = cudaGetDevice(&prev);
  if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  const int grid = static_cast<int>(rows < 148 * 16 ? rows : 148 * 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype_in == KCG_DTYPE_FLOAT32) {
    launch_for_output(grid, st, reinterpret_cast<const float*>(X), ldx, Y, dtype_out, ldy, rows, cols, scale);
  } else if (dtype_in == KCG_DTYPE_FLOAT16) {
    launch_for_output(grid, st, reinterpret_cast<const __half*>(X), ldx, Y, dtype_out, ldy, rows, cols, scale);
  } else {
    launch_for_output(grid, st, reinterpret_cast<const __nv_bfloat16*>(X), ldx, Y, dtype_out, ldy, rows, cols, scale);
  }
  e = cudaGetLastError();
  if (prev != device && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) return fail(static_cast<int>(e), std::string("softmax launch: ") + cudaGetErrorString(e));
  kcg_internal_count_launch();
  return 0;
}

extern "C" int kcg_softmax_rows(int device, uint64_t stream, uint64_t X, int64_t rows, int cols, int64_t ld,
                                float scale, int dtype) {
  return kcg_softmax_rows_ex(device, stream, X, dtype, ld, X, dtype, ld, rows, cols, scale);
}
