// kcg_gemm_bf16_splitk_noalloc: a split-K bf16 GEMM that allocates nothing.
//
// Some callers of this library are not allowed to allocate device memory when they
// reach the GEMM: code that runs inside a memory pool or arena it must not grow, a
// real-time or serving loop with a fixed memory budget, or a host that has handed all
// free HBM to another allocator, where a cudaMalloc / cuMemAlloc would fail or stall
// (device allocation also synchronises the device). The regular launch entry
// (kcg_launch_gemm) allocates its split-K workspace on first use and grows it on
// demand; this entry point never does. Its workspace - the fp32 partial tiles of every
// K split plus one arrival counter per output tile - is a fixed array in the library's
// device image, so it exists as soon as the library's module is loaded on a GPU and
// stays until the process exits, on every GPU that loads it.
//
// The kernel is the same template as the JIT-compiled one (gemm_tcgen05.cuh) at one
// fixed config: bf16, tile 128x256x64, 4 stages, K split 4 ways, raster group 8.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/kcg_b200.h"
#include "kernels/gemm_tcgen05.cuh"

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4, kSplitK = KCG_NOALLOC_SPLITK, kGroup = 8;
using Gemm = kcg::TcGemm<KCG_DT_BF16, kBM, kBN, kBK, kStages, /*ATrans*/ 0, kSplitK, kGroup>;

constexpr size_t kPartialBytes = static_cast<size_t>(KCG_NOALLOC_MAX_PARTIAL_FLOATS) * sizeof(float);
constexpr size_t kCounterBytes = static_cast<size_t>(KCG_NOALLOC_MAX_TILES) * sizeof(unsigned int);

// The whole scratch: [ partial tiles | tile counters | 4 status words ]. Static device memory
// starts out zeroed. Host code must not
// pass `g_scratch` itself to a kernel - in host code the name is only a handle for
// cudaGetSymbolAddress, which yields the address the device sees.
static __device__ __align__(256) unsigned char g_scratch[kPartialBytes + kCounterBytes + 256];

__global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
kcg_noalloc_gemm_kernel(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}

struct PerDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_scratch on this GPU
  int num_sms = 0;
};
PerDevice g_state[16];
std::mutex g_mutex;
extern "C" int kcg_internal_fail(int code, const char* msg);
extern "C" void kcg_internal_count_launch(void);

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

int fail(int code, const std::string& msg) { return kcg_internal_fail(code, msg.c_str()); }
int cuda_fail(cudaError_t e, const char* what) {
  return fail(static_cast<int>(e), std::string(what) + ": " + cudaGetErrorString(e));
}

// Makes `device` current for the length of a call and puts the caller's device back afterwards.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t enter(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev == device) return cudaSuccess;
    e = cudaSetDevice(device);
    switched = (e == cudaSuccess);
    return e;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// One-time set-up per device, with that device current (the caller holds a DeviceGuard): resolve
// the device address of the scratch array and opt the kernel in to its dynamic shared memory.
// No allocation call is made; with CUDA's lazy module loading this is, however, the moment the
// library's device image (the scratch array included) is materialised on the GPU.
int setup_device(int device, PerDevice** out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  PerDevice& d = g_state[device];
  if (!d.ready) {
    cudaError_t e;
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(scratch)");
    e = cudaFuncSetAttribute(kcg_noalloc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Gemm::SMEM_BYTES);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
    e = cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return fail(KCG_E_NO_DRIVER, "cuTensorMapEncodeTiled not available from the driver");
      g_encode = reinterpret_cast<EncodeFn>(fn);
    }
    d.scratch = static_cast<unsigned char*>(ptr);
    d.ready = true;
  }
  *out = &d;
  return 0;
}

int encode(CUtensorMap* tm, uint64_t ptr, uint64_t inner, uint64_t outer, int box_inner, int box_outer, int swizzle,
           bool fp32 = false) {
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {inner * (fp32 ? 4 : 2)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(tm, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              reinterpret_cast<void*>(ptr), gdim, gstride,
                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(swizzle),
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(static_cast<int>(r), "cuTensorMapEncodeTiled failed");
  return 0;
}

}  // namespace

extern "C" {

int kcg_gemm_bf16_splitk_noalloc(int device, uint64_t stream, uint64_t A, uint64_t B, uint64_t C, int M, int N,
                                 int K, int synchronize) {
  if (!A || !B || !C) return fail(KCG_E_BAD_ARG, "null device pointer");
  if (M <= 0 || N <= 0 || K <= 0 || M % kBM || N % kBN || K % kBK)
    return fail(KCG_E_BAD_CONFIG, "M, N, K must be positive multiples of 128, 256, 64");
  if (K / kBK < kSplitK) return fail(KCG_E_BAD_CONFIG, "K must hold at least one 64-wide block per K split");
  if ((A | B | C) % 16) return fail(KCG_E_BAD_ARG, "A, B and C must be 16-byte aligned");
  const size_t partial_floats = static_cast<size_t>(kSplitK) * M * N;
  const size_t tiles = static_cast<size_t>(M / kBM) * (N / kBN);
  if (partial_floats > KCG_NOALLOC_MAX_PARTIAL_FLOATS || tiles > KCG_NOALLOC_MAX_TILES) {
    char buf[256];
    snprintf(buf, sizeof(buf),
             "problem too large for the built-in workspace: %d*M*N = %zu floats (limit %d) over %zu tiles (limit %d)",
             kSplitK, partial_floats, KCG_NOALLOC_MAX_PARTIAL_FLOATS, tiles, KCG_NOALLOC_MAX_TILES);
    return fail(KCG_E_TOO_LARGE, buf);
  }
  if (device < 0 || device >= 16) return fail(KCG_E_BAD_ARG, "device out of range");
  DeviceGuard guard;  // the caller's current device is restored on every return path
  cudaError_t ce = guard.enter(device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  PerDevice* d = nullptr;
  if (int e = setup_device(device, &d)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  KcgGemmParams p;
  memset(&p, 0, sizeof(p));
  constexpr kcg::TcLayout L = kcg::make_tc_layout(KCG_DT_BF16, kBM, kBN, kBK, 0);
  if (int e = encode(&p.tmA, A, K, M, L.a_box_inner, L.a_box_outer, L.a_tma_swizzle)) return e;
  if (int e = encode(&p.tmB, B, N, K, L.b_box_inner, L.b_box_outer, L.b_tma_swizzle)) return e;
  // every tile is K-split here, so C is written by the reducing CTA with plain stores; the map is
  // still a valid one because the kernel prefetches its descriptor
  if (int e = encode(&p.tmC, C, N, M, 64, 32, 3 /*CU_TENSOR_MAP_SWIZZLE_128B*/)) return e;
  // partial tiles leave through TMA stores: the scratch array as one tall fp32 matrix of kBN
  // columns, 32 x 32 boxes with the 128B swizzle of the kernel's staging buffers
  if (int e = encode(&p.tmWs, reinterpret_cast<uint64_t>(d->scratch), kBN, kPartialBytes / (kBN * 4), 32, 32,
                     3 /*CU_TENSOR_MAP_SWIZZLE_128B*/, true))
    return e;
  p.A = reinterpret_cast<const void*>(A);
  p.B = reinterpret_cast<const void*>(B);
  p.C = reinterpret_cast<void*>(C);
  p.M = M;
  p.N = N;
  p.K = K;
  p.lda = K;
  p.ldb = N;
  p.ldc = N;
  p.split_first_tile = 0;  // every tile is split
  p.split_factor = kSplitK;
  p.splitk_ws = reinterpret_cast<float*>(d->scratch);
  p.tile_counters = reinterpret_cast<unsigned int*>(d->scratch + kPartialBytes);
  p.status = reinterpret_cast<unsigned int*>(d->scratch + kPartialBytes + kCounterBytes);
  // The array keeps whatever the previous call left: the counters must start at zero (partials
  // are fully rewritten before they are read). The status words are NOT cleared here: a kernel of
  // an earlier asynchronous call that gave up in a bounded wait stays on record until a
  // synchronising call reads (and clears) it below.
  ce = cudaMemsetAsync(d->scratch + kPartialBytes, 0, kCounterBytes, st);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemsetAsync(counters)");
  const int units = static_cast<int>(tiles) * kSplitK;
  const int grid = units < d->num_sms ? units : d->num_sms;
  kcg_noalloc_gemm_kernel<<<grid, Gemm::NUM_THREADS, Gemm::SMEM_BYTES, st>>>(p);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return cuda_fail(ce, "kernel launch");
  kcg_internal_count_launch();
  if (synchronize) {
    ce = cudaStreamSynchronize(st);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamSynchronize");
    unsigned int status[4] = {0, 0, 0, 0};
    ce = cudaMemcpy(status, p.status, sizeof(status), cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemcpy(status)");
    if (status[0] != 0) {
      ce = cudaMemset(p.status, 0, sizeof(status));
      if (ce != cudaSuccess) return cuda_fail(ce, "cudaMemset(status)");
      char buf[128];
      snprintf(buf, sizeof(buf), "kernel gave up in a bounded wait (code %u, block %u)", status[0], status[1]);
      return fail(KCG_E_DEVICE_TIMEOUT, buf);
    }
  }
  return 0;
}

}  // extern "C"
