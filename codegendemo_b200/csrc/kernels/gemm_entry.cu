// One translation unit = one kernel. The compile entry (kcg_compile_matmul) runs
// nvcc on this file once per tuning config, passing the config as -DKCG_* macros
// and the kernel's symbol as -DKCG_KERNEL_NAME, and loads the resulting cubin
// with the driver API. This replaces the reference's per-config MLIR -> AMDGCN ->
// hsaco pipeline (src/main.cc:250-305) for the GEMM path.
#include <type_traits>

#include "gemm_params.h"

#ifndef KCG_KERNEL_NAME
#error "KCG_KERNEL_NAME must be defined"
#endif
#ifndef KCG_VARIANT
#error "KCG_VARIANT must be defined"
#endif

// REG_PREFETCH of the tuning config: overlap of the accumulator drain with the next tile's main
// loop in the single-pass tcgen05 kernels (gemm_tcgen05.cuh); on unless the config turns it off.
#ifndef KCG_REGP
#define KCG_REGP 1
#endif
#define KCG_ACC_OVERLAP (KCG_REGP ? 1 : 0)
// B stored N x K row-major (single-pass tcgen05 kernels, 16-bit types)
#ifndef KCG_BTRANS
#define KCG_BTRANS 0
#endif
// DATATYPE_C = float32 with 16-bit A and B (single-pass tcgen05 kernels): C keeps the fp32 accumulators
#ifndef KCG_OUT_F32
#define KCG_OUT_F32 0
#endif

#if KCG_DTYPE == KCG_DT_F32
#define KCG_T float
#elif KCG_DTYPE == KCG_DT_F16
#define KCG_T __half
#elif KCG_DTYPE == KCG_DT_BF16
#define KCG_T __nv_bfloat16
#else
#error "unsupported KCG_DTYPE"
#endif

#if KCG_VARIANT == KCG_VARIANT_TCGEN05 && KCG_DTYPE == KCG_DT_F32
#include "gemm_tcgen05_f32x3.cuh"
#ifndef KCG_CHUNK  // K blocks multiplied into one TMEM accumulator before promotion to registers
#define KCG_CHUNK ((128 / KCG_BK) > 0 ? (128 / KCG_BK) : 1)
#endif
using Gemm = kcg::TcGemmF32x3<KCG_BM, KCG_BN, KCG_BK, KCG_STAGES, KCG_ATRANS, KCG_SPLITK, KCG_GROUP, KCG_CHUNK>;
extern "C" __global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == KCG_VARIANT_TCGEN05 || KCG_VARIANT == KCG_VARIANT_TF32X1
#include "gemm_tcgen05.cuh"
using Gemm = kcg::TcGemm<KCG_DTYPE, KCG_BM, KCG_BN, KCG_BK, KCG_STAGES, KCG_ATRANS, KCG_SPLITK, KCG_GROUP, 0, KCG_ACC_OVERLAP, KCG_BTRANS, KCG_OUT_F32>;
extern "C" __global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == KCG_VARIANT_TCGEN05_PAIR && KCG_DTYPE == KCG_DT_F32
#include "gemm_tcgen05_f32x3.cuh"
#ifndef KCG_CHUNK
#define KCG_CHUNK ((128 / KCG_BK) > 0 ? (128 / KCG_BK) : 1)
#endif
using Gemm = kcg::TcGemmF32x3<KCG_BM, KCG_BN, KCG_BK, KCG_STAGES, KCG_ATRANS, KCG_SPLITK, KCG_GROUP, KCG_CHUNK, 1>;
extern "C" __global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == KCG_VARIANT_TCGEN05_PAIR
#include "gemm_tcgen05.cuh"
using Gemm = kcg::TcGemm<KCG_DTYPE, KCG_BM, KCG_BN, KCG_BK, KCG_STAGES, KCG_ATRANS, KCG_SPLITK, KCG_GROUP, 1, KCG_ACC_OVERLAP, KCG_BTRANS, KCG_OUT_F32>;
extern "C" __global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == KCG_VARIANT_TCGEN05_CLUSTERK
#include "gemm_tcgen05_clusterk.cuh"
using Gemm = kcg::TcGemmClusterK<KCG_DTYPE, KCG_BN, KCG_BK, KCG_STAGES, KCG_ATRANS, KCG_SPLITK, KCG_GROUP>;
extern "C" __global__ void __launch_bounds__(Gemm::NUM_THREADS, 1)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == KCG_VARIANT_SIMT
#include "gemm_simt.cuh"
using Gemm = kcg::SimtGemm<KCG_T, KCG_BM, KCG_BN, KCG_BK, KCG_TM, KCG_TN, KCG_BLM, KCG_BLN, KCG_WLM,
                           KCG_WLN, KCG_WSWA, KCG_WSWB, KCG_TSWA, KCG_TSWB, KCG_SPLITK, KCG_GROUP,
                           KCG_GLWA, KCG_GLWB, KCG_GSW, KCG_SHMP, KCG_REGP, KCG_ATRANS>;
extern "C" __global__ void __launch_bounds__(Gemm::THREADS)
KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  Gemm::run(p);
}
#elif KCG_VARIANT == 100  // naive one-thread-per-element device reference
#include "gemm_simt.cuh"
extern "C" __global__ void KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  kcg::naive_gemm<KCG_T, KCG_ATRANS>(p);
}
#elif KCG_VARIANT == 101  // wait probe: exercises the bounded-wait / status-word path
// One CTA waits on an mbarrier that nothing ever signals, with a 20 ms limit instead of the
// kernels' 1 s, records the same status a GEMM role would record and returns. It never spins
// unbounded, traps or touches memory it does not own; C is left untouched.
#undef KCG_WAIT_LIMIT_NS
#define KCG_WAIT_LIMIT_NS 20000000ull
#include "ptx_sm100.cuh"
extern "C" __global__ void KCG_KERNEL_NAME(const __grid_constant__ KcgGemmParams p) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    kcg::mbar_init(&bar, 1);
    abort_flag = 0u;
    kcg::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!kcg::mbar_wait(&bar, 0u, &abort_flag)) {
      if (atomicCAS(p.status, 0u, KCG_ST_TIMEOUT_MMA) == 0u) {
        p.status[1] = blockIdx.x;
        p.status[2] = 0xdeadu;
        p.status[3] = 0u;
      }
    }
  }
}
#else
#error "unknown KCG_VARIANT"
#endif
