// Persistent GEMM on CTA pairs: tcgen05.mma.cta_group::2 computes a (256 kMT) x BN
// output tile across two SMs. Each CTA of the pair owns 128 kMT rows of the tile
// (its own TMEM accumulators, its own epilogue) and loads only its 128 x BK slice
// of A and HALF of the B tile (BN/2 columns); the MMA reads the other half from
// the peer's shared memory. Per SM this halves the B traffic of both TMA and UMMA
// operand reads, which is what limits the single-CTA kernel (gemm_tcgen05.cuh).
// No TMA multicast: every load has exactly one destination CTA.
//
// Launch: clusters of 2 along x, grid = 2 * (number of pairs), persistent; a work
// unit is one 256 x BN tile (same grouped raster as the single-CTA kernel).
//
//   warp 0  producer: this CTA's A slice and B half of every K block ->
//           kStages-deep ring; completion bytes of BOTH CTAs are counted on the
//           leader's (even rank) full barrier
//   warp 1  leader only: issues the pair MMAs, releases stages / publishes
//           accumulators to both CTAs with one tcgen05.commit per CTA
//   warps 2..5 epilogue of this CTA's 128 rows (two TMEM accumulator buffers)
//
// All waits are bounded; see ptx_sm100.cuh. Both CTAs always reach the closing
// cluster barrier, after which TMEM is freed.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_params.h"
#include "ptx_sm100.cuh"

namespace kcg {

template <int kDType, int kMT, int kBN, int kBK, int kStages, int kATrans, int kGroup>
struct TcGemmPair {
  // kMT = accumulators (M = 256 pair MMAs) per tile. Two interleaved accumulators keep
  // consecutive MMAs independent, which the tensor pipe needs to stay full (a single
  // accumulator chain measured ~10 % slower).
  static_assert(kMT == 1 || kMT == 2, "one or two accumulators per CTA");
  static constexpr int kBM = 256 * kMT;   // tile rows of the pair
  static constexpr int kRows = 128 * kMT; // rows per CTA
  static constexpr int kHalfN = kBN / 2;
  // Per-CTA operand slices use the single-CTA layout rules with BM = 128, BN = kBN / 2.
  static_assert(tc_config_error(kDType, kRows, kHalfN, kBK, kStages, 0) == 0, "tile not buildable");
  static_assert(kBN % 32 == 0 && kBN <= 256 && kBN >= 64, "pair tile width");
  static constexpr TcLayout L = make_tc_layout(kDType, kRows, kHalfN, kBK, kATrans);
  static constexpr int EB = L.eb;
  static constexpr bool kTf32 = (EB == 4);
  static constexpr int UMMA_K = L.umma_k;
  static constexpr int ACC_COLS = kMT * kBN;
  static constexpr int NACC = (2 * ACC_COLS <= 512) ? 2 : 1;
  static constexpr int TMEM_COLS = kc_pow2_ceil(NACC * ACC_COLS);
  static constexpr int STAGE_BYTES = L.stage_hi_bytes;  // this CTA's share of one stage
  static constexpr int KSTEPS = kBK / UMMA_K;
  static constexpr int NUM_EPI_THREADS = 128;
  static constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS;
  static constexpr int SMEM_BYTES = kStages * STAGE_BYTES + 2048;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
  static constexpr uint32_t FMT = (kDType == KCG_DT_F32)    ? FMT_TF32
                                  : (kDType == KCG_DT_BF16) ? FMT_BF16
                                                            : FMT_F16;
  static constexpr uint32_t IDESC = make_instr_desc(FMT, kATrans ? 1u : 0u, 1u, 256u, kBN);

  struct Barriers {
    uint64_t full[kStages];   // used in the leader only (bytes of both CTAs)
    uint64_t empty[kStages];  // one per CTA, signalled by the leader's commits
    uint64_t tmem_full[2];    // one per CTA
    uint64_t tmem_empty[2];   // used in the leader only: 4 warps x 2 CTAs arrive
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
  };
  static_assert(sizeof(Barriers) <= 1024, "barrier block exceeds its shared-memory slot");

  __device__ static __forceinline__ void tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
    int mb, nb;
    if constexpr (kGroup > 1) {
      const int per_group = kGroup * tiles_n;
      const int g = tile / per_group;
      const int first_m = g * kGroup;
      const int gsz = (tiles_m - first_m < kGroup) ? (tiles_m - first_m) : kGroup;
      const int r = tile - g * per_group;
      mb = first_m + (r % gsz);
      nb = r / gsz;
    } else {
      mb = tile / tiles_n;
      nb = tile - mb * tiles_n;
    }
    m0 = mb * kBM;
    n0 = nb * kBN;
  }

  __device__ static __forceinline__ void report(const KcgGemmParams& p, Barriers* bars, uint32_t code,
                                                uint32_t d0, uint32_t d1) {
    bars->abort_flag = 1u;
    if (atomicCAS(p.status, 0u, code) == 0u) {
      p.status[1] = blockIdx.x;
      p.status[2] = d0;
      p.status[3] = d1;
    }
  }

  template <typename OutT>
  __device__ static __forceinline__ void store_chunk(OutT* dst, const float (&v)[32]) {
    if constexpr (sizeof(OutT) == 4) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = v[8 * i + 2 * j], hi = v[8 * i + 2 * j + 1];
          if constexpr (kDType == KCG_DT_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __half2 h = __floats2half2_rn(lo, hi);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        d4[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }

  __device__ static void run(const KcgGemmParams& p) {
    using OutT = typename std::conditional<kTf32, float,
                 typename std::conditional<kDType == KCG_DT_BF16, __nv_bfloat16, __half>::type>::type;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Both CTAs see the same dynamic shared-memory base offset, so aligned offsets coincide.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();  // 0 = leader
    const uint32_t peer = rank ^ 1u;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + kBN - 1) / kBN;
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&bars->tmem_full[a], 1);
        mbar_init(&bars->tmem_empty[a], 8);  // 4 epilogue warps of each CTA
      }
      bars->abort_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    if (warp == 1) {
      tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
      tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // peer's barriers are initialised before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
      // ------------------------------------------------------------ producer
      if (lane == 0) {
        tma_prefetch_desc(&p.tmA);
        tma_prefetch_desc(&p.tmB);
        uint32_t it = 0;
        bool ok = true;
        for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
          int m0, n0;
          tile_origin(tile, tiles_m, tiles_n, m0, n0);
          const int my_m0 = m0 + static_cast<int>(rank) * kRows;
          const int my_n0 = n0 + static_cast<int>(rank) * kHalfN;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!mbar_wait(&bars->empty[s], ph ^ 1u, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_PRODUCER, it, s);
              ok = false;
              break;
            }
            uint8_t* sa = smem + s * STAGE_BYTES;
            uint8_t* sb = sa + L.a_bytes;
            // completion bytes of both CTAs land on the leader's barrier
            const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[s]), 0u);
            if (rank == 0u) mbar_expect_tx(&bars->full[s], static_cast<uint32_t>(2 * STAGE_BYTES));
            const int k0 = kb * kBK;
#pragma unroll
            for (int j = 0; j < L.a_boxes; ++j) {
              if constexpr (kATrans) {
                tma_load_2d_pair(sa + j * L.a_box_bytes, &p.tmA, full_leader, my_m0 + j * L.atom, k0);
              } else {
                tma_load_2d_pair(sa + j * L.a_box_bytes, &p.tmA, full_leader, k0 + j * L.a_box_inner, my_m0);
              }
            }
#pragma unroll
            for (int j = 0; j < L.b_boxes; ++j) {
              tma_load_2d_pair(sb + j * L.b_box_bytes, &p.tmB, full_leader, my_n0 + j * L.atom, k0);
            }
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------- MMA issuer (leader CTA only)
      if (lane == 0 && rank == 0u) {
        uint32_t it = 0, acc_it = 0;
        bool ok = true;
        for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++acc_it) {
          const uint32_t ab = acc_it % NACC;
          const uint32_t aph = (acc_it / NACC) & 1u;
          if (!mbar_wait(&bars->tmem_empty[ab], aph ^ 1u, &bars->abort_flag)) {
            report(p, bars, KCG_ST_TIMEOUT_MMA, 0x100u + ab, acc_it);
            break;
          }
          tc_fence_after_sync();
          const uint32_t tmem_acc = tmem_base + ab * ACC_COLS;
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!mbar_wait(&bars->full[s], ph, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_MMA, it, s);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
            const uint32_t sb = sa + L.a_bytes;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
              uint32_t a_off;
              if constexpr (kATrans) {
                a_off = ks * UMMA_K * 128;
              } else {
                constexpr int swb = (kBK * EB < 128) ? kBK * EB : 128;
                a_off = ((ks * 32) / swb) * L.a_box_bytes + ((ks * 32) % swb);
              }
              const uint32_t b_off = ks * UMMA_K * 128;
              const uint64_t bdesc = make_smem_desc(sb + b_off, L.b_lbo, L.b_sbo, L.b_desc_swizzle);
#pragma unroll
              for (int t = 0; t < kMT; ++t) {
                // accumulator t: local A rows [128 t, 128 t + 128) of each CTA
                const uint32_t a_t = kATrans ? t * (128 / L.atom) * L.a_box_bytes
                                             : t * 128 * (L.a_box_bytes / kRows);
                const uint64_t adesc = make_smem_desc(sa + a_t + a_off, L.a_lbo, L.a_sbo, L.a_desc_swizzle);
                umma_ss_pair<kTf32>(tmem_acc + t * kBN, adesc, bdesc, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
              }
            }
            // the stage is free in BOTH CTAs once these MMAs retire
            umma_commit_pair(smem_u32(&bars->empty[s]));
            umma_commit_pair(map_to_cta(smem_u32(&bars->empty[s]), 1u));
          }
          if (ok) {
            umma_commit_pair(smem_u32(&bars->tmem_full[ab]));
            umma_commit_pair(map_to_cta(smem_u32(&bars->tmem_full[ab]), 1u));
          }
        }
      }
    } else {
      // ------------------------------------------------------------ epilogue
      const int q = warp & 3;
      const int row_in_acc = q * 32 + lane;
      uint32_t acc_it = 0;
      OutT* Cout = reinterpret_cast<OutT*>(p.C);
      for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++acc_it) {
        int m0, n0;
        tile_origin(tile, tiles_m, tiles_n, m0, n0);
        const uint32_t ab = acc_it % NACC;
        const uint32_t aph = (acc_it / NACC) & 1u;
        const bool got = mbar_wait(&bars->tmem_full[ab], aph, &bars->abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, acc_it, ab);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + ab * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
        for (int t = 0; t < kMT; ++t) {
          const int row = m0 + static_cast<int>(rank) * kRows + t * 128 + row_in_acc;
#pragma unroll 1
          for (int c = 0; c < kBN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem_acc + t * kBN + c * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            const int col = n0 + c * 32;
            if (row < p.M && col < p.N) store_chunk<OutT>(Cout + static_cast<size_t>(row) * p.ldc + col, v);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[ab]), 0u));
      }
    }

    // ------------------------------------------------------------ common exit
    if (bars->abort_flag != 0u) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();  // the peer's shared memory and TMEM stay valid until both are done
    if (warp == 1) {
      __syncwarp();
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
  }
};

}  // namespace kcg
