// Kernel-argument block and compile-time layout rules shared by the device
// kernels and the host shim. Plain C++ (no torch, no CUDA runtime types beyond
// CUtensorMap), so the host library and every JIT-compiled cubin agree on the
// byte layout of one `__grid_constant__` parameter.
#pragma once
#include <cuda.h>
#include <stdint.h>

// DATATYPE_* values of the tuning config. 2/4/8 are the reference's
// EnumKernelDType byte-size codes (Runtime/python/kcg/Utils.py:198-203);
// 62 is this library's bfloat16 (62 % 30 == 2 bytes keeps the reference's
// sizeof() rule, Utils.py:219-221).
#define KCG_DT_F16 2
#define KCG_DT_F32 4
#define KCG_DT_F64 8
#define KCG_DT_BF16 62

// KERNEL_VARIANT
#define KCG_VARIANT_AUTO 0
#define KCG_VARIANT_SIMT 1     // FFMA register-tiled kernel (fp32)
#define KCG_VARIANT_TCGEN05 2  // TMA + tcgen05/TMEM kernel (bf16, fp16, fp32 as 3xTF32)
#define KCG_VARIANT_TF32X1 3   // tcgen05 single-pass TF32 (fp32 in, reduced accuracy; comparison only)

#define KCG_VARIANT_TCGEN05_PAIR 4  // tcgen05 cta_group::2 on clusters of two CTAs (fp16 / bf16)
// K split over a thread-block cluster of LOCAL_SPLIT_U CTAs, partial tiles reduced through
// distributed shared memory (fp16 / bf16, 128-row tiles): no workspace, no counters
#define KCG_VARIANT_TCGEN05_CLUSTERK 5

#define KCG_MAX_PEERS 7  // other GPUs of one NVSwitch domain of eight

// epi_flags bits
#define KCG_EPI_SCALE 1u  // alpha / beta differ from 1 / 0
#define KCG_EPI_BIAS 2u   // add bias[col]
#define KCG_EPI_RELU 4u   // max(x, 0) last

// Device status word values (status[0]); 0 = ok.
#define KCG_ST_OK 0u
#define KCG_ST_TIMEOUT_PRODUCER 1u
#define KCG_ST_TIMEOUT_MMA 2u
#define KCG_ST_TIMEOUT_EPILOGUE 3u
#define KCG_ST_TIMEOUT_SPLITTER 4u
#define KCG_ST_BAD_SHAPE 5u
#define KCG_ST_TIMEOUT_PUSHER 6u

struct alignas(64) KcgGemmParams {
  CUtensorMap tmA;  // tcgen05 variants: tiled map of A (or of A^T when IS_ATRANS=1)
  CUtensorMap tmB;  // tiled map of B (K x N row-major)
  CUtensorMap tmC;  // C as 32-row x 128-byte boxes (128B swizzle): the TMA-store epilogue
  CUtensorMap tmWs;  // K-split workspace as one tall fp32 matrix of BN columns, 32 x 32 boxes
  const void* A;
  const void* B;
  void* C;
  float* splitk_ws;             // fp32 partial tiles, [slot][BM][BN]; slot = unit - split_first_tile
  unsigned int* tile_counters;  // one per split tile (tile - split_first_tile), zero between launches
  unsigned int* status;         // 4 words: code, blockIdx.x, detail0, detail1
  int M, N, K;
  int lda, ldb, ldc;  // leading dimensions in elements (row-major storage)
  // K splitting over CTAs: tiles [0, split_first_tile) are computed whole, every tile from
  // split_first_tile on is cut into split_factor K ranges. LOCAL_SPLIT_U = S splits every tile
  // (first = 0, factor = S); with LOCAL_SPLIT_U = 1 the launcher splits only the tiles of the last,
  // partially filled wave of the persistent grid (or nothing: factor = 1).
  int split_first_tile, split_factor;
  // Stream-K over the tiles from split_first_tile on (instead of the even split) when > 0: their
  // K blocks, laid end to end, are cut into one contiguous range of sk_per blocks per CTA (pair);
  // the grid then has exactly as many CTAs (pairs) as there are ranges (work_iter.cuh).
  int sk_per;
  // Batched product when > 0: M counts the rows of all batches (A and C stacked by rows), K is one
  // batch's, B holds the batches' K x N matrices one under the other (an A stored K x M likewise),
  // and batch_rows is the M of one batch, a multiple of the tile height.
  int batch_rows;
  // Order of a CTA's units when a launch has both whole tiles and K-split tiles: 1 = the split
  // units (even split or stream-K ranges) come first and the whole tiles after them, so that the
  // partial tiles are written, summed and stored by the epilogue warps while the whole tiles' main
  // loops run, and a CTA ends with an ordinary tile; 0 = whole tiles first, split units last.
  int split_units_first;
  // Fused epilogue, in force when epi_flags != 0: D = act(alpha * (A.B) + beta * C + bias[col]),
  // computed in fp32 before the rounding to C's type. beta * C reads C in place (skipped when
  // beta == 0, so C may then hold anything); bias has N values of C's type.
  float alpha, beta;
  const void* bias;
  unsigned int epi_flags;  // KCG_EPI_*
  // Fused all-gather of an M-sharded product: besides C, every finished tile is also written
  // to the same rows / columns of n_peers more matrices with C's pitch — this rank's slab inside
  // the full C of every other GPU, mapped into this process (coalesced 16-byte stores over NVLink
  // by the kernel's push warps, or by the reducer of a K-split tile; no remote loads, no multicast,
  // no flags between GPUs: the data is in place when every rank's kernel has completed).
  int n_peers;
  void* peerC[KCG_MAX_PEERS];
};

namespace kcg {

constexpr int kc_min(int a, int b) { return a < b ? a : b; }
constexpr int kc_pow2_ceil(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

// Shared-memory / TMA layout of one pipeline stage of the tcgen05 kernels.
// Host (tensor-map construction) and device (descriptors) both derive it from
// the same five config values.
struct TcLayout {
  int eb;          // element bytes
  int umma_k;      // K extent of one MMA instruction
  int atom;        // elements per 128-byte swizzle row
  // A operand
  int a_box_inner, a_box_outer;  // TMA box in elements {contiguous, strided}
  int a_boxes, a_box_bytes, a_bytes;
  int a_tma_swizzle;   // CUtensorMapSwizzle value
  int a_desc_swizzle;  // UMMA descriptor layout type
  int a_lbo, a_sbo;
  // B operand (always MN-major: K x N row-major)
  int b_box_inner, b_box_outer;
  int b_boxes, b_box_bytes, b_bytes;
  int b_tma_swizzle, b_desc_swizzle;
  int b_lbo, b_sbo;
  int stage_hi_bytes;  // one copy of A+B
};

// `btrans` = B is stored N x K row-major (the "NT" product C = A * Bt^T): its tile is then a K-major
// operand laid out exactly like a K-major A tile; 16-bit types only.
constexpr TcLayout make_tc_layout(int dtype, int BM, int BN, int BK, int atrans, int btrans = 0) {
  TcLayout L{};
  L.eb = (dtype == KCG_DT_F32) ? 4 : 2;
  L.umma_k = 32 / L.eb;
  L.atom = 128 / L.eb;
  // MN-major operands: boxes of {atom elements along MN, BK rows of K}.
  // 16-bit: 128B swizzle of 16B units, 8-row repeat; 32-bit: 128B swizzle of
  // 32B units, 4-row repeat (the only MN-major form kind::tf32 accepts).
  const int mn_tma = (L.eb == 4) ? 4 /*128B_ATOM_32B*/ : 3 /*128B*/;
  const int mn_desc = (L.eb == 4) ? 1 : 2;
  const int mn_sbo = (L.eb == 4) ? 512 : 1024;
  if (atrans) {
    L.a_box_inner = L.atom;
    L.a_box_outer = BK;
    L.a_boxes = BM / L.atom;
    L.a_box_bytes = BK * 128;
    L.a_tma_swizzle = mn_tma;
    L.a_desc_swizzle = mn_desc;
    L.a_lbo = BK * 128;
    L.a_sbo = mn_sbo;
  } else {
    const int swb = kc_min(128, BK * L.eb);  // swizzle span = bytes of one K row
    L.a_box_inner = swb / L.eb;
    L.a_box_outer = BM;
    L.a_boxes = (BK * L.eb) / swb;
    L.a_box_bytes = BM * swb;
    L.a_tma_swizzle = (swb == 128) ? 3 : (swb == 64) ? 2 : 1;
    L.a_desc_swizzle = (swb == 128) ? 2 : (swb == 64) ? 4 : 6;
    L.a_lbo = 16;
    L.a_sbo = 8 * swb;
  }
  L.a_bytes = BM * BK * L.eb;
  L.b_box_inner = L.atom;
  L.b_box_outer = BK;
  L.b_boxes = BN / L.atom;
  L.b_box_bytes = BK * 128;
  L.b_bytes = BN * BK * L.eb;
  L.b_tma_swizzle = mn_tma;
  L.b_desc_swizzle = mn_desc;
  L.b_lbo = BK * 128;
  L.b_sbo = mn_sbo;
  if (btrans) {
    const int swb = kc_min(128, BK * L.eb);
    L.b_box_inner = swb / L.eb;
    L.b_box_outer = BN;
    L.b_boxes = (BK * L.eb) / swb;
    L.b_box_bytes = BN * swb;
    L.b_tma_swizzle = (swb == 128) ? 3 : (swb == 64) ? 2 : 1;
    L.b_desc_swizzle = (swb == 128) ? 2 : (swb == 64) ? 4 : 6;
    L.b_lbo = 16;
    L.b_sbo = 8 * swb;
  }
  L.stage_hi_bytes = L.a_bytes + L.b_bytes;
  return L;
}

// Epilogue staging of the single-pass kernel: each of its four epilogue warps owns two
// 32-row x 128-byte buffers from which C leaves through TMA stores. The 3xTF32 kernel
// stores from registers and has none. `x3` only has a meaning for fp32 data: 16-bit data always
// runs on the single-pass kernel.
constexpr int tc_staging_bytes(int dtype, int x3) {
  return (dtype == KCG_DT_F32 && x3) ? 0 : 4 * 2 * 32 * 128;
}

// 3xTF32 kernel: depth of the ring of lo twins beside `stages` TMA-fed hi stages. The kernel
// supports a shorter lo ring, but the splitter has to run several K blocks ahead of the MMAs
// (hand-offs plus two passes over a stage of shared memory), which only equally deep rings give:
// every shorter lo ring measured slower. So the lo ring is as deep as the hi ring.
constexpr int tc_lo_stages(int stages) { return stages; }

// Bytes of the operand rings: single-pass kernel stages * (A + B tile); 3xTF32 adds the lo ring.
constexpr int tc_ring_bytes(int dtype, int BM, int BN, int BK, int stages, int x3) {
  const int eb = (dtype == KCG_DT_F32) ? 4 : 2;
  const int stage = (BM + BN) * BK * eb;
  return stage * (stages + ((eb == 4 && x3) ? tc_lo_stages(stages) : 0));
}

// Shape rules of the tcgen05 kernels; returns 0 when the config is buildable.
constexpr int tc_config_error(int dtype, int BM, int BN, int BK, int stages, int x3) {
  const int eb = (dtype == KCG_DT_F32) ? 4 : 2;
  if (!(dtype == KCG_DT_F32 || dtype == KCG_DT_F16 || dtype == KCG_DT_BF16)) return 1;
  if (!(BM == 128 || BM == 256)) return 2;
  if (BN < 128 / eb || BN > 256 || (BN % (128 / eb)) != 0 || (BN % 16) != 0) return 3;
  if ((BM / 128) * BN > 512) return 4;
  // 3xTF32: two TMEM accumulator buffers and MT*BN/2 register accumulators per epilogue thread
  if (eb == 4 && x3 && ((BM / 128) * BN > 256 || (BN % 64) != 0)) return 9;
  const int rowb = BK * eb;
  if (!(rowb == 32 || rowb == 64 || (rowb % 128) == 0) || rowb > 512) return 5;
  if ((BK % (32 / eb)) != 0 || (BK % 8) != 0) return 6;
  if (eb == 2 && (BK % 16) != 0) return 6;
  if (stages < 2 || stages > 12) return 7;
  if (tc_ring_bytes(dtype, BM, BN, BK, stages, x3) + 2048 + tc_staging_bytes(dtype, x3) > 227 * 1024) return 8;
  return 0;
}

// Cluster split-K kernel (gemm_tcgen05_clusterk.cuh): a 128 x BN tile per cluster of `split` CTAs.
// The operand ring doubles as the exchange buffers of the reduction (a staging copy of the fp32
// accumulator, 128 x BN x 4 bytes, plus a receive slot per other CTA), so it must be at least that
// large; no TMA-store staging.
constexpr int ck_config_error(int dtype, int BN, int BK, int stages, int split) {
  if (!(dtype == KCG_DT_F16 || dtype == KCG_DT_BF16)) return 1;
  if (split < 2 || split > 4) return 2;  // larger clusters do not fit the exchange buffers (nor the GPU: few run at once)
  if (BN < 64 || BN > 256 || (BN % 64) != 0 || BN / 32 < split) return 3;
  const int rowb = BK * 2;
  if (!(rowb == 32 || rowb == 64 || (rowb % 128) == 0) || rowb > 512 || (BK % 16) != 0) return 5;
  if (stages < 2 || stages > 12) return 7;
  const int ring = (128 + BN) * BK * 2 * stages;
  if (ring + 2048 > 227 * 1024) return 8;
  // the ring doubles as exchange buffers: a receive slot per other CTA plus a staging copy of the accumulator
  // of the blocks that belong to other CTAs
  if (ring < ((split - 1) * ((BN / 32 + split - 1) / split) + (BN / 32 - BN / 32 / split)) * 128 * 128) return 10;
  return 0;
}
constexpr int ck_smem_bytes(int BN, int BK, int stages) { return (128 + BN) * BK * 2 * stages + 2048; }

constexpr int tc_smem_bytes(int dtype, int BM, int BN, int BK, int stages, int x3) {
  // +1024 alignment slack, +1024 barriers / TMEM holder / flags, + epilogue staging
  return tc_ring_bytes(dtype, BM, BN, BK, stages, x3) + 2048 + tc_staging_bytes(dtype, x3);
}

}  // namespace kcg
