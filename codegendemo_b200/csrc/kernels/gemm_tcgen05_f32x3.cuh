// fp32 GEMM on the tensor cores with fp32-level accuracy: 3xTF32 split plus
// chunked promotion of the TMEM accumulator into fp32 registers.
//
// Why two extra mechanisms on top of the plain tcgen05 pipeline:
//  * kind::tf32 reads fp32 words and ignores the low 13 mantissa bits, so
//    hi = x needs no work; lo = tf32_rn(x - trunc_tf32(x)) is written by splitter
//    warps into a twin of every landed stage, and each K step issues
//    lo*hi + hi*lo + hi*hi (lo*lo, ~2^-22 relative, is dropped).
//  * The tensor core adds into its fp32 accumulator with truncation, a bias that
//    grows linearly with the number of accumulated K steps (measured: 3e-5
//    normwise at K = 4096). So the MMA warp restarts a fresh accumulator every
//    kChunk K blocks, alternating between two TMEM buffers, and the epilogue
//    warps add each finished chunk into register accumulators with ordinary
//    round-to-nearest FADDs while the next chunk is being multiplied.
//
// Warp roles (512 threads, four warpgroups so that setmaxnreg can move registers
// from the control warps to the accumulating warps):
//   WG0  warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-3 idle
//   WG1  warps 4-7   splitter (lo twin of each stage)
//   WG2/3 warps 8-15 accumulate + epilogue; warp w reads TMEM lane quarter w%4,
//         column half (w-8)/4; kAccPerThread = MT*BN/2 fp32 registers per thread
//
// Same work decomposition, raster, split-K reduction and bounded waits as
// gemm_tcgen05.cuh.
#pragma once
#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"
#include "work_iter.cuh"

namespace kcg {

// kPair = 1 runs the same pipeline on clusters of two CTAs sharing each MMA
// (tcgen05 cta_group::2, M = 256): a CTA then holds kBM/2 rows of the tile and loads and
// splits only half of the B tile (kBN/2 columns); the leader CTA (even rank) issues the
// MMAs once the splitters of BOTH CTAs have arrived, and frees stages / publishes
// accumulators in both CTAs with one commit each. Halving the B operand traffic per SM
// lifts the shared-memory bound of the single-CTA form.
template <int kBM, int kBN, int kBK, int kStages, int kATrans, int kSplitK, int kGroup, int kChunk,
          int kPair = 0>
struct TcGemmF32x3 {
  static constexpr int kDType = KCG_DT_F32;
  static constexpr int NCTA = kPair ? 2 : 1;
  static constexpr int R = kBM / NCTA;     // rows of the tile held by one CTA
  static constexpr int BNL = kBN / NCTA;   // B columns loaded by one CTA
  static_assert(tc_config_error(kDType, R, BNL, kBK, kStages, 1) == 0,
                "config not buildable by the 3xTF32 kernel");
  static constexpr TcLayout L = make_tc_layout(kDType, R, BNL, kBK, kATrans);
  static constexpr int UMMA_K = 8;
  static constexpr int MT = R / 128;
  static constexpr int ACC_COLS = MT * kBN;
  static_assert(2 * ACC_COLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");
  static_assert(kBN % 64 == 0, "each epilogue warp drains whole 32-column pieces of its column half");
  static constexpr int TMEM_COLS = kc_pow2_ceil(2 * ACC_COLS);
  static constexpr int STAGE_HI = L.stage_hi_bytes;
  // Two rings: kStages stages of TMA-landed hi operands (deep, to cover the load latency) and
  // LO_STAGES stages of their lo twins, written just in time by the splitter warps: lo stage
  // it % LO_STAGES is free again as soon as the MMAs of K block it - LO_STAGES have retired.
  static constexpr int LO_STAGES = tc_lo_stages(kStages);
  static constexpr int LO_RING = kStages * STAGE_HI;  // byte offset of the lo ring
  static constexpr int RING_BYTES = (kStages + LO_STAGES) * STAGE_HI;
  static constexpr int KSTEPS = kBK / UMMA_K;
  static constexpr int NUM_THREADS = 512;
  static constexpr int NUM_SPLIT_THREADS = 128;
  static constexpr int NUM_EPI_THREADS = 256;
  static constexpr int HALF_COLS = kBN / 2;
  static constexpr int PIECES = HALF_COLS / 32;
  static constexpr int ACC_PER_THREAD = MT * HALF_COLS;
  static_assert(ACC_PER_THREAD <= 128, "register accumulators per thread");
  static constexpr int SMEM_BYTES = tc_smem_bytes(kDType, R, BNL, kBK, kStages, 1);
  static constexpr uint32_t IDESC = make_instr_desc(FMT_TF32, kATrans ? 1u : 0u, 1u, kPair ? 256u : 128u, kBN);

  struct Barriers {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t split_full[LO_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    uint32_t last_flag;
  };
  static_assert(sizeof(Barriers) <= 1024, "barrier block exceeds its shared-memory slot");

  using Unit = WorkUnit;
  using Iter = WorkIter<kBM, kBN, kGroup, KCG_SERPENTINE>;  // units of this CTA (pair), in order: work_iter.cuh

  __device__ static __forceinline__ void report(const KcgGemmParams& p, Barriers* bars,
                                                uint32_t code, uint32_t d0, uint32_t d1) {
    bars->abort_flag = 1u;
    if (atomicCAS(p.status, 0u, code) == 0u) {
      p.status[1] = blockIdx.x;
      p.status[2] = d0;
      p.status[3] = d1;
    }
  }

  template <int REGS>
  __device__ static __forceinline__ void reg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
  }
  template <int REGS>
  __device__ static __forceinline__ void reg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
  }

  __device__ static void run(const KcgGemmParams& p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + RING_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + kBN - 1) / kBN;
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int first_split = p.split_first_tile;

    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      for (int s = 0; s < LO_STAGES; ++s)
        mbar_init(&bars->split_full[s], 4 * NCTA);  // one arrival per splitter warp of each CTA
      for (int a = 0; a < 2; ++a) {
        mbar_init(&bars->tmem_full[a], 1);
        mbar_init(&bars->tmem_empty[a], 8 * NCTA);  // one arrival per accumulating warp of each CTA
      }
      bars->abort_flag = 0u;
      bars->last_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    if (warp == 1) {
      if constexpr (kPair) {
        tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish_pair();
      } else {
        tmem_alloc(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish();
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t rank = kPair ? cluster_cta_rank() : 0u;  // 0 = leader
    const int unit0 = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int unit_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int row_base = static_cast<int>(rank) * R;     // this CTA's first row inside the tile
    const int bcol_base = static_cast<int>(rank) * BNL;  // this CTA's first B column inside the tile

    if (warp < 4) {
      reg_dec<56>();
      if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- producer
        tma_prefetch_desc(&p.tmA);
        tma_prefetch_desc(&p.tmB);
        griddep_wait();  // the kernel before this one in the stream may have written A or B
        uint32_t it = 0;
        bool ok = true;
        Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
        Unit w;
        while (ok && units.next(w)) {
          for (int kb = 0; kb < w.kbn; ++kb, ++it) {
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            if (!mbar_wait(&bars->empty[s], ph ^ 1u, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_PRODUCER, it, s);
              ok = false;
              break;
            }
            uint8_t* sa = smem + s * STAGE_HI;
            uint8_t* sb = sa + L.a_bytes;
            mbar_expect_tx(&bars->full[s], static_cast<uint32_t>(STAGE_HI));
            const int k0 = (w.kb0 + kb) * kBK;
#pragma unroll
            for (int j = 0; j < L.a_boxes; ++j) {
              if constexpr (kATrans) {  // K x M storage: the batch selects K rows, M counts inside it
                tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s], w.mcol + row_base + j * L.atom,
                            k0 + w.kofs);
              } else {
                tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s],
                            k0 + j * L.a_box_inner, w.m0 + row_base);
              }
            }
#pragma unroll
            for (int j = 0; j < L.b_boxes; ++j) {
              tma_load_2d(sb + j * L.b_box_bytes, &p.tmB, &bars->full[s], w.n0 + bcol_base + j * L.atom,
                          k0 + w.kofs);
            }
          }
        }
        griddep_launch_dependents();  // every load is issued: the stream's next kernel may be brought in
      } else if (warp == 1 && lane == 0 && rank == 0u) {
        // ---------------------------- MMA issuer (in a pair: the leader CTA only)
        uint32_t it = 0, chunk_it = 0;
        bool ok = true;
        Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
        Unit w;
        while (ok && units.next(w)) {
          for (int kb0 = 0; kb0 < w.kbn && ok; kb0 += kChunk, ++chunk_it) {
            const uint32_t ab = chunk_it & 1u;
            const uint32_t aph = (chunk_it >> 1) & 1u;
            if (!mbar_wait(&bars->tmem_empty[ab], aph ^ 1u, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_MMA, 0x100u + ab, chunk_it);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t tmem_acc = tmem_base + ab * ACC_COLS;
            const int kb1 = (kb0 + kChunk < w.kbn) ? kb0 + kChunk : w.kbn;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
              const uint32_t s = it % kStages;
              const uint32_t sl = it % LO_STAGES;
              const uint32_t phl = (it / LO_STAGES) & 1u;
              // the lo twin is written after the hi stage has landed (in both CTAs of a pair)
              if (!mbar_wait(&bars->split_full[sl], phl, &bars->abort_flag)) {
                report(p, bars, KCG_ST_TIMEOUT_MMA, it, s);
                ok = false;
                break;
              }
              tc_fence_after_sync();
              const uint32_t sa = smem_u32(smem + s * STAGE_HI);
              const uint32_t sb = sa + L.a_bytes;
              const uint32_t sa_lo = smem_u32(smem + LO_RING + sl * STAGE_HI);
              const uint32_t sb_lo = sa_lo + L.a_bytes;
#pragma unroll
              for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t a_off;
                if constexpr (kATrans) {
                  a_off = ks * UMMA_K * 128;
                } else {
                  constexpr int swb = (kBK * 4 < 128) ? kBK * 4 : 128;
                  a_off = ((ks * 32) / swb) * L.a_box_bytes + ((ks * 32) % swb);
                }
                const uint32_t b_off = ks * UMMA_K * 128;
                const uint32_t first = (kb > kb0 || ks > 0) ? 1u : 0u;
                const uint64_t bdesc = make_smem_desc(sb + b_off, L.b_lbo, L.b_sbo, L.b_desc_swizzle);
                const uint64_t bdesc_lo =
                    make_smem_desc(sb_lo + b_off, L.b_lbo, L.b_sbo, L.b_desc_swizzle);
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                  const uint32_t a_t = kATrans ? t * (128 / L.atom) * L.a_box_bytes
                                               : t * 128 * (L.a_box_bytes / R);
                  const uint64_t adesc =
                      make_smem_desc(sa + a_t + a_off, L.a_lbo, L.a_sbo, L.a_desc_swizzle);
                  const uint64_t adesc_lo = make_smem_desc(sa_lo + a_t + a_off, L.a_lbo,
                                                           L.a_sbo, L.a_desc_swizzle);
                  const uint32_t d = tmem_acc + t * kBN;
                  if constexpr (kPair) {
                    umma_ss_pair<true>(d, adesc_lo, bdesc, IDESC, first);
                    umma_ss_pair<true>(d, adesc, bdesc_lo, IDESC, 1u);
                    umma_ss_pair<true>(d, adesc, bdesc, IDESC, 1u);
                  } else {
                    umma_ss<true>(d, adesc_lo, bdesc, IDESC, first);
                    umma_ss<true>(d, adesc, bdesc_lo, IDESC, 1u);
                    umma_ss<true>(d, adesc, bdesc, IDESC, 1u);
                  }
                }
              }
              // the hi stage, and with it the lo stage of this K block, is free in both CTAs
              // once these MMAs retire
              if constexpr (kPair) {
                umma_commit_pair(smem_u32(&bars->empty[s]));
                umma_commit_pair(map_to_cta(smem_u32(&bars->empty[s]), 1u));
              } else {
                umma_commit(&bars->empty[s]);
              }
            }
            if (ok) {
              if constexpr (kPair) {
                umma_commit_pair(smem_u32(&bars->tmem_full[ab]));
                umma_commit_pair(map_to_cta(smem_u32(&bars->tmem_full[ab]), 1u));
              } else {
                umma_commit(&bars->tmem_full[ab]);
              }
            }
          }
        }
      }
    } else if (warp < 8) {
      // --------------------------------------------------------------- splitter
      reg_dec<56>();
      const int stid = threadIdx.x - 128;
      uint32_t it = 0;
      bool ok = true;
      Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
      Unit w;
      while (ok && units.next(w)) {
        for (int kb = 0; kb < w.kbn; ++kb, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          const uint32_t sl = it % LO_STAGES;
          // lo stage sl was last read by the MMAs of K block it - LO_STAGES; their retirement is
          // what completes that block's phase of its hi stage's `empty` barrier. The MMA warp
          // never runs ahead of this loop, so that barrier cannot be a whole phase further on.
          bool got = true;
          // (with rings of equal depth the landed hi stage already implies it)
          if (LO_STAGES < kStages && it >= static_cast<uint32_t>(LO_STAGES)) {
            const uint32_t prev = it - LO_STAGES;
            got = mbar_wait(&bars->empty[prev % kStages], (prev / kStages) & 1u, &bars->abort_flag);
          }
          if (got) got = mbar_wait(&bars->full[s], ph, &bars->abort_flag);
          if (!got) {
            if (lane == 0) report(p, bars, KCG_ST_TIMEOUT_SPLITTER, it, s);
            ok = false;
            break;
          }
          const uint4* hi = reinterpret_cast<const uint4*>(smem + s * STAGE_HI);
          uint4* lo = reinterpret_cast<uint4*>(smem + LO_RING + sl * STAGE_HI);
#pragma unroll 4
          for (int i = stid; i < STAGE_HI / 16; i += NUM_SPLIT_THREADS) {
            const uint4 x = hi[i];
            uint4 l;
            l.x = lo_part(x.x);
            l.y = lo_part(x.y);
            l.z = lo_part(x.z);
            l.w = lo_part(x.w);
            lo[i] = l;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              mbar_arrive_cluster(map_to_cta(smem_u32(&bars->split_full[sl]), 0u));
            } else {
              mbar_arrive(&bars->split_full[sl]);
            }
          }
        }
      }
    } else {
      // --------------------------------------------------- accumulate + epilogue
      reg_inc<200>();
      griddep_wait();  // C, the workspace and the counters may still be in use by the kernel before
      const int q = warp & 3;
      const int half = (warp - 8) >> 2;
      const int epi_tid = threadIdx.x - 256;
      const int row_in_acc = q * 32 + lane;
      const int col_half0 = half * HALF_COLS;
      float* Cout = reinterpret_cast<float*>(p.C);
      uint32_t chunk_it = 0;
      bool ok = true;
      Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
      Unit w;
      while (ok && units.next(w)) {
        float acc[ACC_PER_THREAD];
#pragma unroll
        for (int i = 0; i < ACC_PER_THREAD; ++i) acc[i] = 0.f;
        for (int kb0 = 0; kb0 < w.kbn; kb0 += kChunk, ++chunk_it) {
          const uint32_t ab = chunk_it & 1u;
          const uint32_t aph = (chunk_it >> 1) & 1u;
          // A warp whose wait ran out stops reading TMEM but keeps walking the unit's chunks (their
          // waits return at once under the abort flag), so that all eight accumulating warps reach
          // the vote below together.
          if (ok) {
            const bool got = mbar_wait(&bars->tmem_full[ab], aph, &bars->abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
              if (lane == 0) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, chunk_it, ab);
              ok = false;
            }
          }
          if (!ok) continue;
          tc_fence_after_sync();
          const uint32_t tmem_acc =
              tmem_base + ab * ACC_COLS + col_half0 + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
          for (int t = 0; t < MT; ++t) {
#pragma unroll
            for (int c = 0; c < PIECES; ++c) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tmem_acc + t * kBN + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i)
                acc[(t * PIECES + c) * 32 + i] += __uint_as_float(r[i]);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[ab]), 0u));
            } else {
              mbar_arrive(&bars->tmem_empty[ab]);
            }
          }
        }
        // The accumulating warps leave a unit as one (named barrier 2 ANDs their outcomes): the
        // store path below meets on named barrier 1, where a warp that had given up alone would
        // leave the others waiting for its threads for ever.
        ok = named_bar_all(2, NUM_EPI_THREADS, ok);
        if (!ok) break;
        // ---- tile (or split partial) complete in registers: store. A launch with a fused
        // epilogue sends whole-K tiles through the workspace too (every tile is then its own
        // one-way "split": the launcher sets split_first_tile = 0) and applies the epilogue in
        // the reduction loop below, where the accumulators are dead: with all of them live
        // there are no registers left for the bias / C operands.
        const bool via_ws = w.nsplit > 1 || p.epi_flags != 0u;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const int row = w.m0 + row_base + t * 128 + row_in_acc;
#pragma unroll
          for (int c = 0; c < PIECES; ++c) {
            const int col = w.n0 + col_half0 + c * 32;
            if (row < p.M && col < p.N) {
              // A partial is private to this kernel, so it is not stored as a matrix: the CTA's
              // R x kBN floats are laid out [16-byte piece of a thread][thread], which makes every
              // warp store (and the reducer's loads) 512 contiguous bytes. Row-major partials, 16
              // bytes per lane at a 1 KB stride, made L2 merge every sector.
              float4* d4 = via_ws ? reinterpret_cast<float4*>(p.splitk_ws +
                                                             (static_cast<size_t>(w.slot) * kBM + row_base) * kBN) +
                                        (t * PIECES + c) * 8 * NUM_EPI_THREADS + epi_tid
                                  : reinterpret_cast<float4*>(Cout + static_cast<size_t>(row) * p.ldc + col);
              const int step = via_ws ? NUM_EPI_THREADS : 1;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int b = (t * PIECES + c) * 32 + 4 * i;
                d4[i * step] = make_float4(acc[b], acc[b + 1], acc[b + 2], acc[b + 3]);
              }
            }
          }
        }
        if (via_ws) {
          bool reduce_here = true;  // a one-way split reads back what this same thread just wrote
          if (w.nsplit > 1) {
            const int ctr = (w.tile - first_split) * NCTA + static_cast<int>(rank);  // per CTA half
            __threadfence();
            named_bar_sync(1, NUM_EPI_THREADS);
            if (epi_tid == 0) {
              const unsigned int old = atomicAdd(&p.tile_counters[ctr], 1u);
              bars->last_flag = (old == static_cast<unsigned int>(w.nsplit - 1)) ? 1u : 0u;
              if (old == static_cast<unsigned int>(w.nsplit - 1)) p.tile_counters[ctr] = 0u;
            }
            named_bar_sync(1, NUM_EPI_THREADS);
            reduce_here = bars->last_flag != 0u;
          }
          if (reduce_here) {
            __threadfence();
            // One partial at a time: the accumulating warps have no registers to spare for
            // deeper prefetch (more loads in flight made ptxas spill inside the main loop).
#pragma unroll 1
            for (int t = 0; t < MT; ++t) {
              const int row = w.m0 + row_base + t * 128 + row_in_acc;
              if (row >= p.M) continue;
#pragma unroll 1
              for (int c = 0; c < PIECES; ++c) {
                const int col = w.n0 + col_half0 + c * 32;
                if (col >= p.N) continue;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll 1
                for (int s = 0; s < w.nsplit; ++s) {
                  const float4* src =
                      reinterpret_cast<const float4*>(
                          p.splitk_ws + ((static_cast<size_t>(w.slot - w.split) + s) * kBM + row_base) * kBN) +
                      (t * PIECES + c) * 8 * NUM_EPI_THREADS + epi_tid;
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float4 x = __ldcg(src + i * NUM_EPI_THREADS);
                    v[4 * i] += x.x;
                    v[4 * i + 1] += x.y;
                    v[4 * i + 2] += x.z;
                    v[4 * i + 3] += x.w;
                  }
                }
                if (p.epi_flags != 0u) epi_span<float, 32>(p, v, row, col);
                float4* d4 = reinterpret_cast<float4*>(Cout + static_cast<size_t>(row) * p.ldc + col);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
              }
            }
          }
          named_bar_sync(1, NUM_EPI_THREADS);
        }
      }
    }

    // ------------------------------------------------------------ common exit
    // The producer and MMA roles run in one lane; the other lanes of those warps come straight here.
    // Reconverge every warp first: the block-wide barrier below must be executed by whole warps.
    __syncwarp();
    if (bars->abort_flag != 0u) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) {
      __syncwarp();
      cluster_sync_all();  // the peer's shared memory and TMEM stay valid until both CTAs are done
    }
    if (warp == 1) {
      __syncwarp();
      tc_fence_after_sync();
      if constexpr (kPair) {
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
      } else {
        tmem_dealloc(tmem_base, TMEM_COLS);
      }
    }
  }

  // tf32_rn(x - trunc_tf32(x)) on raw bits; the subtraction is exact in fp32.
  __device__ static __forceinline__ uint32_t lo_part(uint32_t xbits) {
    const float x = __uint_as_float(xbits);
    const float hi = __uint_as_float(xbits & 0xffffe000u);
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
    return l;
  }
};

}  // namespace kcg
