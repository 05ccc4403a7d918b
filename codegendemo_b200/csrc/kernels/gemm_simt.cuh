// Register-tiled FFMA GEMM ("SIMT variant"): the same algorithm the reference
// generates for its SIMT targets (tiling schedule: src/lib/Conversion/Optimizer.cc:285-469;
// executable twin: matmul.cpp:71-442), written for 32-wide warps. It is kept as the
// measured comparison for the tensor-core kernels and runs the reference's own
// tuning JSONs (small tiles, LOCAL_SPLIT_U, scatter widths) unchanged.
//
//   grid  = (M/BM)*(N/BN) CTAs, rasterised in groups of BLOCK_MAPPING tile rows
//   block = (BM/TM)*(BN/TN)*LOCAL_SPLIT_U threads
//   smem  = smA[BK][BM], smB[BK][BN] (K-major rows), x2 when SHARED_PREFETCH
//   Thread (warp_y, warp_x, lane_y, lane_x) owns TM rows / TN columns scattered
//   in pieces of THREAD_SCATTER_WIDTH inside WARP_SCATTER_WIDTH strips.
//   LOCAL_SPLIT_U: thread group tz handles k == tz (mod LSU) of every K block;
//   partial tiles are summed through shared memory in tz order.
//
// LOAD_CONTINUOUS / REDUCE_C_CONTINUOUS select between thread->element mappings
// that differ only in coalescing on wave64 hardware; here global loads and the
// split-U reduction always use the contiguous mapping.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "gemm_params.h"

namespace kcg {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int W>
struct alignas(sizeof(T) * W) Vec {
  T v[W];
};

template <typename T, int BM, int BN, int BK, int TM, int TN, int BLM, int BLN, int WLM, int WLN,
          int WSWA, int WSWB, int TSWA, int TSWB, int LSU, int GROUP, int GLWA, int GLWB, int GSW,
          int SHMP, int REGP, int ATRANS>
struct SimtGemm {
  static constexpr int BY = BM / TM;
  static constexpr int BX = BN / TN;
  static constexpr int THREADS = BX * BY * LSU;
  static constexpr int WARP = WLM * WLN;  // logical warp of the layout keys
  static constexpr int NBUF = SHMP ? 2 : 1;
  static constexpr int AB_FLOATS = NBUF * (BM + BN) * BK;
  static constexpr int C_FLOATS = (LSU > 1) ? LSU * BM * BN : 0;
  static constexpr int SMEM_FLOATS = AB_FLOATS > C_FLOATS ? AB_FLOATS : C_FLOATS;
  static constexpr int SMEM_BYTES = SMEM_FLOATS * 4;
  static constexpr int A_PER_THREAD = BM * BK / THREADS;
  static constexpr int B_PER_THREAD = BN * BK / THREADS;
  static_assert(BY * TM == BM && BX * TN == BN, "thread tile must divide block tile");
  static_assert(BLM * WLM == BY && BLN * WLN == BX, "warp layout must cover the block");
  static_assert(TM % WSWA == 0 && WSWA % TSWA == 0 && TN % WSWB == 0 && WSWB % TSWB == 0,
                "scatter widths must nest");
  static_assert((BM * BK) % (THREADS * GLWA) == 0 && (BN * BK) % (THREADS * GLWB) == 0,
                "tile loads must split evenly over the threads");
  static_assert(BK % LSU == 0, "LOCAL_SPLIT_U must divide BLOCK_SIZE_K");
  static_assert(ATRANS ? (BM % GLWA == 0) : (BK % GLWA == 0), "A vector width");
  static_assert(BN % GLWB == 0 && TSWB % (GSW < TSWB ? GSW : TSWB) == 0, "B/C vector width");

  // global -> registers (vector loads along the contiguous dimension)
  __device__ static __forceinline__ void load_tiles(const T* __restrict__ A, const T* __restrict__ B,
                                                    int lda, int ldb, int m0, int n0, int k0,
                                                    float (&ta)[A_PER_THREAD], float (&tb)[B_PER_THREAD]) {
    const int tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < A_PER_THREAD / GLWA; ++i) {
      const int e = (tid + i * THREADS) * GLWA;
      Vec<T, GLWA> v;
      if constexpr (ATRANS) {  // A stored K x M: element (k, m), m contiguous
        const int k = e / BM, m = e % BM;
        v = *reinterpret_cast<const Vec<T, GLWA>*>(A + static_cast<size_t>(k0 + k) * lda + m0 + m);
      } else {  // A stored M x K: element (m, k), k contiguous
        const int m = e / BK, k = e % BK;
        v = *reinterpret_cast<const Vec<T, GLWA>*>(A + static_cast<size_t>(m0 + m) * lda + k0 + k);
      }
#pragma unroll
      for (int j = 0; j < GLWA; ++j) ta[i * GLWA + j] = to_f32<T>(v.v[j]);
    }
#pragma unroll
    for (int i = 0; i < B_PER_THREAD / GLWB; ++i) {
      const int e = (tid + i * THREADS) * GLWB;
      const int k = e / BN, n = e % BN;
      const Vec<T, GLWB> v =
          *reinterpret_cast<const Vec<T, GLWB>*>(B + static_cast<size_t>(k0 + k) * ldb + n0 + n);
#pragma unroll
      for (int j = 0; j < GLWB; ++j) tb[i * GLWB + j] = to_f32<T>(v.v[j]);
    }
  }

  // registers -> shared (smA[k][m], smB[k][n])
  __device__ static __forceinline__ void store_tiles(float* smA, float* smB,
                                                     const float (&ta)[A_PER_THREAD],
                                                     const float (&tb)[B_PER_THREAD]) {
    const int tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < A_PER_THREAD / GLWA; ++i) {
      const int e = (tid + i * THREADS) * GLWA;
#pragma unroll
      for (int j = 0; j < GLWA; ++j) {
        if constexpr (ATRANS) {
          smA[e + j] = ta[i * GLWA + j];  // same (k, m) order as global
        } else {
          const int m = e / BK, k = e % BK + j;
          smA[k * BM + m] = ta[i * GLWA + j];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < B_PER_THREAD / GLWB; ++i) {
      const int e = (tid + i * THREADS) * GLWB;
#pragma unroll
      for (int j = 0; j < GLWB; ++j) smB[e + j] = tb[i * GLWB + j];
    }
  }

  // Row (or column) index inside the block tile of the r-th element a thread owns.
  template <int TSZ, int WSW, int TSW, int BL, int WL>
  __device__ static __forceinline__ int owned_index(int r, int warp_c, int lane_c) {
    const int i = r / WSW;          // which warp strip
    const int j = (r % WSW) / TSW;  // which thread piece inside the strip
    const int o = r % TSW;
    return (i * BL + warp_c) * WL * WSW + (j * WL + lane_c) * TSW + o;
  }

  __device__ static __forceinline__ void load_frag(const float* smA, const float* smB, int k,
                                                   int warp_y, int warp_x, int lane_y, int lane_x,
                                                   float (&ra)[TM], float (&rb)[TN]) {
#pragma unroll
    for (int r = 0; r < TM; r += TSWA) {
      const int m = owned_index<TM, WSWA, TSWA, BLM, WLM>(r, warp_y, lane_y);
#pragma unroll
      for (int o = 0; o < TSWA; ++o) ra[r + o] = smA[k * BM + m + o];
    }
#pragma unroll
    for (int r = 0; r < TN; r += TSWB) {
      const int n = owned_index<TN, WSWB, TSWB, BLN, WLN>(r, warp_x, lane_x);
#pragma unroll
      for (int o = 0; o < TSWB; ++o) rb[r + o] = smB[k * BN + n + o];
    }
  }

  __device__ static void run(const KcgGemmParams& p) {
    extern __shared__ __align__(16) float smem_f[];
    const T* A = reinterpret_cast<const T*>(p.A);
    const T* B = reinterpret_cast<const T*>(p.B);
    T* C = reinterpret_cast<T*>(p.C);
    const int tid = threadIdx.x;
    const int tz = tid / (BX * BY);
    const int t2 = tid % (BX * BY);
    const int warp_id = t2 / WARP, lane_id = t2 % WARP;
    const int warp_y = warp_id / BLN, warp_x = warp_id % BLN;
    const int lane_y = lane_id / WLN, lane_x = lane_id % WLN;

    // grouped raster (matmul.cpp:79-86 semantics)
    const int tiles_m = p.M / BM, tiles_n = p.N / BN;
    int by, bx;
    if constexpr (GROUP > 1) {
      const int per_group = GROUP * tiles_n;
      const int g = blockIdx.x / per_group;
      const int first = g * GROUP;
      const int gsz = (tiles_m - first < GROUP) ? (tiles_m - first) : GROUP;
      const int r = blockIdx.x - g * per_group;
      by = first + r % gsz;
      bx = r / gsz;
    } else {
      by = blockIdx.x / tiles_n;
      bx = blockIdx.x % tiles_n;
    }
    const int m0 = by * BM, n0 = bx * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    float ta[A_PER_THREAD], tb[B_PER_THREAD];
    float* smA = smem_f;
    float* smB = smem_f + NBUF * BM * BK;
    const int num_kb = p.K / BK;

    load_tiles(A, B, p.lda, p.ldb, m0, n0, 0, ta, tb);
    store_tiles(smA, smB, ta, tb);
    __syncthreads();

    int buf = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      const bool has_next = kb + 1 < num_kb;
      if (SHMP && has_next) load_tiles(A, B, p.lda, p.ldb, m0, n0, (kb + 1) * BK, ta, tb);
      const float* cA = smA + buf * BM * BK;
      const float* cB = smB + buf * BN * BK;
      if constexpr (REGP) {
        float ra[2][TM], rb[2][TN];
        load_frag(cA, cB, tz, warp_y, warp_x, lane_y, lane_x, ra[0], rb[0]);
#pragma unroll
        for (int kk = 0; kk < BK / LSU; ++kk) {
          const int cur = kk & 1;
          if (kk + 1 < BK / LSU)
            load_frag(cA, cB, (kk + 1) * LSU + tz, warp_y, warp_x, lane_y, lane_x, ra[cur ^ 1],
                      rb[cur ^ 1]);
#pragma unroll
          for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ra[cur][i], rb[cur][j], acc[i][j]);
        }
      } else {
        float ra[TM], rb[TN];
#pragma unroll
        for (int kk = 0; kk < BK / LSU; ++kk) {
          load_frag(cA, cB, kk * LSU + tz, warp_y, warp_x, lane_y, lane_x, ra, rb);
#pragma unroll
          for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ra[i], rb[j], acc[i][j]);
        }
      }
      if (has_next) {
        if constexpr (SHMP) {
          store_tiles(smA + (buf ^ 1) * BM * BK, smB + (buf ^ 1) * BN * BK, ta, tb);
          __syncthreads();
          buf ^= 1;
        } else {
          __syncthreads();
          load_tiles(A, B, p.lda, p.ldb, m0, n0, (kb + 1) * BK, ta, tb);
          store_tiles(smA, smB, ta, tb);
          __syncthreads();
        }
      }
    }

    if constexpr (LSU > 1) {
      // Partial tiles -> smC[tz][BM][BN]; all threads then sum the LSU planes in
      // tz order and store C with GLOB_STORE_WIDTH-wide vectors.
      __syncthreads();
      float* smC = smem_f;
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const int m = owned_index<TM, WSWA, TSWA, BLM, WLM>(i, warp_y, lane_y);
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          const int n = owned_index<TN, WSWB, TSWB, BLN, WLN>(j, warp_x, lane_x);
          smC[(tz * BM + m) * BN + n] = acc[i][j];
        }
      }
      __syncthreads();
      for (int e = tid * GSW; e < BM * BN; e += THREADS * GSW) {
        const int m = e / BN, n = e % BN;
        Vec<T, GSW> out;
        float sv[GSW];
#pragma unroll
        for (int j = 0; j < GSW; ++j) {
          float s = 0.f;
#pragma unroll
          for (int z = 0; z < LSU; ++z) s += smC[(z * BM + m) * BN + n + j];
          sv[j] = s;
        }
        if (p.epi_flags != 0u) epi_span<T, GSW>(p, sv, m0 + m, n0 + n);
#pragma unroll
        for (int j = 0; j < GSW; ++j) out.v[j] = from_f32<T>(sv[j]);
        *reinterpret_cast<Vec<T, GSW>*>(C + static_cast<size_t>(m0 + m) * p.ldc + n0 + n) = out;
      }
    } else {
      constexpr int SW = (GSW < TSWB) ? GSW : TSWB;  // store vector fits one owned piece
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const int m = owned_index<TM, WSWA, TSWA, BLM, WLM>(i, warp_y, lane_y);
#pragma unroll
        for (int j = 0; j < TN; j += SW) {
          const int n = owned_index<TN, WSWB, TSWB, BLN, WLN>(j, warp_x, lane_x);
          Vec<T, SW> out;
          float sv[SW];
#pragma unroll
          for (int o = 0; o < SW; ++o) sv[o] = acc[i][j + o];
          if (p.epi_flags != 0u) epi_span<T, SW>(p, sv, m0 + m, n0 + n);
#pragma unroll
          for (int o = 0; o < SW; ++o) out.v[o] = from_f32<T>(sv[o]);
          *reinterpret_cast<Vec<T, SW>*>(C + static_cast<size_t>(m0 + m) * p.ldc + n0 + n) = out;
        }
      }
    }
  }
};

// One thread per C element; the on-device naive reference (same role as the
// reference's gemm_kernel, matmul.cpp:2327-2337). fp32 accumulate in k order.
template <typename T, int ATRANS>
__device__ void naive_gemm(const KcgGemmParams& p) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= p.M || col >= p.N) return;
  const T* A = reinterpret_cast<const T*>(p.A);
  const T* B = reinterpret_cast<const T*>(p.B);
  float s = 0.f;
  for (int k = 0; k < p.K; ++k) {
    const float a = ATRANS ? to_f32<T>(A[static_cast<size_t>(k) * p.lda + row])
                           : to_f32<T>(A[static_cast<size_t>(row) * p.lda + k]);
    s = fmaf(a, to_f32<T>(B[static_cast<size_t>(k) * p.ldb + col]), s);
  }
  float sv[1] = {s};
  if (p.epi_flags != 0u) epi_span<T, 1>(p, sv, row, col);
  reinterpret_cast<T*>(p.C)[static_cast<size_t>(row) * p.ldc + col] = from_f32<T>(sv[0]);
}

}  // namespace kcg
