// Persistent, warp-specialised GEMM for sm_100a: C[M,N] = A[M,K] * B[K,N].
//
//   warp 0        TMA producer: fills a kStages-deep ring of {A tile, B tile}
//                 in shared memory (cp.async.bulk.tensor, no multicast), one
//                 mbarrier pair (full/empty) per stage.
//   warp 1        MMA issuer: one elected thread issues tcgen05.mma from the
//                 shared-memory descriptors into fp32 accumulators in TMEM and
//                 releases stages / publishes accumulators with tcgen05.commit.
//                 The warp also owns the TMEM allocation.
//   warps 2..5    epilogue: tcgen05.ld the accumulator (one TMEM lane = one C
//                 row per thread), convert, stage 32 x 128-byte blocks in swizzled
//                 shared memory and write C with TMA stores (full 128-byte lines,
//                 asynchronous). K-split partials leave the same way as fp32 blocks
//                 into the workspace; the last contributor of a tile sums them with
//                 coalesced loads. With two accumulator buffers the epilogue overlaps
//                 the next tile's main loop.
//
// fp32 data runs here as ONE TF32 pass (comparison only); the accurate fp32 path
// is gemm_tcgen05_f32x3.cuh.
//
// Config keys -> template parameters (reference meaning: Optimizer.cc:285-469):
//   BLOCK_SIZE_M/N/K -> kBM (128 | 256 = two M=128 accumulators), kBN, kBK
//   SHARED_PREFETCH / NUM_STAGES -> kStages;  LOCAL_SPLIT_U -> kSplitK (K split
//   across CTAs, fp32 partials in a workspace, last arriver reduces in split
//   order so the result is deterministic);  BLOCK_MAPPING -> kGroup (rows of
//   tiles per raster group);  IS_ATRANS -> A stored K x M.
//
// Every mbarrier wait is bounded; on a timeout the role records a status code,
// raises the CTA-wide abort flag and all roles fall through to the common exit
// where TMEM is freed.
#pragma once
#include <cuda_bf16.h>
#ifdef KCG_TIMELINE_PRINT
#include <cstdio>
#endif
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"
#include "work_iter.cuh"

// How long a CTA waits for the other partial tiles of a shared K-split reduction before it hands
// its share to the last arriver.
#ifndef KCG_SHARE_WAIT_NS
#define KCG_SHARE_WAIT_NS 20000ull
#endif

namespace kcg {

//
// kPair = 1 runs the same pipeline on clusters of two CTAs that share every MMA
// (tcgen05 cta_group::2, M = 256): each CTA holds kBM/2 rows of the tile (its own TMEM
// accumulators and epilogue) and loads only its rows of A and HALF of the B tile; the MMA
// reads the other half from the peer's shared memory. The even-ranked CTA (leader) issues
// the MMAs; the completion bytes of BOTH CTAs' loads are counted on the leader's `full`
// barrier; stages are freed and accumulators published in both CTAs with one
// tcgen05.commit per CTA; the peer's epilogue warps release TMEM with a remote arrive. No
// TMA multicast is used: every load has one destination CTA.
//
// kAccOverlap (REG_PREFETCH; the reference's register double buffer, Optimizer.cc:438-447, whose
// purpose is to overlap the drain of one result with the compute of the next) = 1 overlaps the
// epilogue of tile i with the main loop of tile i + 1: through two TMEM accumulator buffers when
// two fit the 512 columns; for the two-accumulator tile that fills all of TMEM (256 rows x 256
// columns per CTA) by releasing the accumulator in halves - the MMA warp runs the first K blocks
// of the next tile into half 0 while the epilogue still drains half 1. 0 = one buffer, released whole.
//
// kBTrans = 1: B is stored N x K row-major (C = A * Bt^T, the "NT" product: Q * K^T of attention
// without a transposed copy of K); the B tile is then a K-major operand like a K-major A tile.
//
// kOutF32 = 1 (DATATYPE_C = float32 with 16-bit A and B): C is written as fp32, the accumulators
// unrounded - e.g. attention scores, whose rounding to bf16 would be amplified by the softmax's exp.
template <int kDType, int kBM, int kBN, int kBK, int kStages, int kATrans, int kSplitK,
          int kGroup, int kPair = 0, int kAccOverlap = 1, int kBTrans = 0, int kOutF32 = 0>
struct TcGemm {
  static constexpr int NCTA = kPair ? 2 : 1;
  static constexpr int R = kBM / NCTA;    // rows of the tile held by one CTA
  static constexpr int BNL = kBN / NCTA;  // B columns loaded by one CTA
  static_assert(tc_config_error(kDType, R, BNL, kBK, kStages, 0) == 0,
                "config not buildable by the tcgen05 kernel");
  static constexpr TcLayout L = make_tc_layout(kDType, R, BNL, kBK, kATrans, kBTrans);
  static constexpr int EB = L.eb;
  static constexpr bool kTf32 = (EB == 4);
  static_assert(!(kBTrans && kTf32), "an N x K stored B is supported for 16-bit types only");
  static constexpr int UMMA_K = L.umma_k;
  static constexpr int MT = R / 128;
  static constexpr int ACC_COLS = MT * kBN;
  static constexpr int NACC = (kAccOverlap && 2 * ACC_COLS <= 512) ? 2 : 1;
  // one buffer of two accumulators, released half by half (tmem_empty[t] = accumulator t is drained)
  static constexpr bool HALF = kAccOverlap && NACC == 1 && MT == 2;
  static constexpr int HALF_KB = kStages - 1;  // K blocks run into half 0 ahead of half 1
  static constexpr int TMEM_COLS = kc_pow2_ceil(NACC * ACC_COLS);
  static constexpr int STAGE_HI = L.stage_hi_bytes;
  static constexpr int STAGE_BYTES = STAGE_HI;
  static constexpr int KSTEPS = kBK / UMMA_K;
  static constexpr int NUM_EPI_THREADS = 128;
  static constexpr int NUM_PUSH_WARPS = 2;  // fused all-gather: copy finished tiles to the peers' C
  static constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS + 32 * NUM_PUSH_WARPS;
  static constexpr int SMEM_BYTES = tc_smem_bytes(kDType, R, BNL, kBK, kStages, 0);
  static constexpr int STG_BYTES = 32 * 128;       // one staging buffer: 32 rows x 128 bytes
  static constexpr bool kOut32 = (kDType == KCG_DT_F32) || kOutF32;  // C holds fp32
  static constexpr int SCOLS = 128 / (kOut32 ? 4 : 2);  // C columns per staging buffer
  static_assert(8 * STG_BYTES == tc_staging_bytes(kDType, 0), "staging size out of step with the host");
  static_assert(kBN % SCOLS == 0, "tile width must be a multiple of the staging width");
  static constexpr uint32_t FMT = (kDType == KCG_DT_F32)    ? FMT_TF32
                                  : (kDType == KCG_DT_BF16) ? FMT_BF16
                                                            : FMT_F16;
  static constexpr uint32_t IDESC =
      make_instr_desc(FMT, kATrans ? 1u : 0u, kBTrans ? 0u : 1u, kPair ? 256u : 128u, kBN);

  struct Barriers {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t red_full;  // partial tiles of a shared reduction have landed in the (idle) operand ring
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    uint32_t last_flag;
    uint32_t push_count;  // epilogue warps that have finished (and completed the stores of) a whole-K tile
#ifdef KCG_TIMELINE
    uint64_t tl[32];  // %globaltimer stamps of CTA 0's phases (experiments only; dumped over C[0, 0..])
#endif
  };
#ifdef KCG_TIMELINE
#define KCG_TL(i) bars->tl[i] = global_timer_ns()
#define KCG_TLC(var) const long long var = clock64()
#define KCG_TLC_ADD(i, var) bars->tl[i] += static_cast<uint64_t>(clock64() - var)
#else
#define KCG_TL(i) ((void)0)
#define KCG_TLC(var) ((void)0)
#define KCG_TLC_ADD(i, var) ((void)0)
#endif
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

  __device__ static void run(const KcgGemmParams& p) {
    using OutT = typename std::conditional<kOut32, float,
                 typename std::conditional<kDType == KCG_DT_BF16, __nv_bfloat16, __half>::type>::type;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Tiles need 1024-byte alignment (128B swizzle repeat); the launch asks for 1 KiB of slack.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * STAGE_BYTES);
#ifdef KCG_TIMELINE
    if (threadIdx.x == 0) {
      for (int i = 10; i < 32; ++i) bars->tl[i] = 0;
    }
    __syncthreads();
#endif
    if (threadIdx.x == 0) KCG_TL(0);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + kBN - 1) / kBN;
    const int num_kb = (p.K + kBK - 1) / kBK;
    const int first_split = p.split_first_tile;

    if (threadIdx.x == 0) {
      // the first TMA instruction needs its descriptor: start fetching the maps before anything else
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&bars->tmem_full[a], 1);
        mbar_init(&bars->tmem_empty[a], 4 * NCTA);  // one arrival per epilogue warp of each CTA
      }
      mbar_init(&bars->red_full, 1);
      bars->abort_flag = 0u;
      bars->last_flag = 0u;
      bars->push_count = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    const uint32_t rank = kPair ? cluster_cta_rank() : 0u;  // 0 = leader
    const int unit0 = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int unit_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const int row_base = static_cast<int>(rank) * R;     // this CTA's first row inside the tile
    const int bcol_base = static_cast<int>(rank) * BNL;  // this CTA's first B column inside the tile

    // ---- producer state (thread 0). The loop below is entered twice: once before the set-up barrier
    // for the FIRST stage only (its `empty` wait passes at once on a fresh barrier, and a single CTA's
    // loads signal only its own barriers, which this very thread has just initialised), so that the
    // first operands are in flight while TMEM is allocated - issuing the whole ring there delayed the
    // barrier by more than it gained -; and again, to the end, as warp 0's role.
    Iter p_units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
    Unit p_w;
    uint32_t p_it = 0;
    int p_kb = 0;
    bool p_have = false, p_ok = true;
    auto produce = [&](uint32_t it_limit) {
      while (p_ok && p_have && p_it < it_limit) {
        if (p_kb >= p_w.kbn) {
          p_kb = 0;
          p_have = p_units.next(p_w);
          continue;
        }
        const uint32_t s = p_it % kStages;
        const uint32_t ph = (p_it / kStages) & 1u;
        KCG_TLC(c_wait);
        if (!mbar_wait(&bars->empty[s], ph ^ 1u, &bars->abort_flag)) {
          report(p, bars, KCG_ST_TIMEOUT_PRODUCER, p_it, s);
          p_ok = false;
          break;
        }
        KCG_TLC_ADD(10, c_wait);
        KCG_TLC(c_issue);
        const Unit& w = p_w;
        uint8_t* sa = smem + s * STAGE_BYTES;
        uint8_t* sb = sa + L.a_bytes;
        const int k0 = (w.kb0 + p_kb) * kBK;
        // K x M storage: the batch selects K rows and M is counted inside the batch
        const int am0 = (kATrans ? w.mcol : w.m0) + row_base, bn0 = w.n0 + bcol_base;
        const int ka = kATrans ? k0 + w.kofs : k0, kb_row = k0 + w.kofs;
        if constexpr (kPair) {
          // completion bytes of both CTAs land on the leader's barrier
          const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[s]), 0u);
          if (rank == 0u) mbar_expect_tx(&bars->full[s], static_cast<uint32_t>(2 * STAGE_HI));
#pragma unroll
          for (int j = 0; j < L.a_boxes; ++j) {
            if constexpr (kATrans) {
              tma_load_2d_pair(sa + j * L.a_box_bytes, &p.tmA, full_leader, am0 + j * L.atom, ka);
            } else {
              tma_load_2d_pair(sa + j * L.a_box_bytes, &p.tmA, full_leader, ka + j * L.a_box_inner, am0);
            }
          }
#pragma unroll
          for (int j = 0; j < L.b_boxes; ++j) {
            if constexpr (kBTrans) {  // N x K storage: the batch selects N rows
              tma_load_2d_pair(sb + j * L.b_box_bytes, &p.tmB, full_leader, k0 + j * L.b_box_inner,
                               bn0 + w.nofs);
            } else {
              tma_load_2d_pair(sb + j * L.b_box_bytes, &p.tmB, full_leader, bn0 + j * L.atom, kb_row);
            }
          }
        } else {
          mbar_expect_tx(&bars->full[s], static_cast<uint32_t>(STAGE_HI));
#pragma unroll
          for (int j = 0; j < L.a_boxes; ++j) {
            if constexpr (kATrans) {
              tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s], am0 + j * L.atom, ka);
            } else {
              tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s], ka + j * L.a_box_inner, am0);
            }
          }
#pragma unroll
          for (int j = 0; j < L.b_boxes; ++j) {
            if constexpr (kBTrans) {
              tma_load_2d(sb + j * L.b_box_bytes, &p.tmB, &bars->full[s], k0 + j * L.b_box_inner, bn0 + w.nofs);
            } else {
              tma_load_2d(sb + j * L.b_box_bytes, &p.tmB, &bars->full[s], bn0 + j * L.atom, kb_row);
            }
          }
        }
        KCG_TLC_ADD(11, c_issue);
        if (p_it == 0) KCG_TL(2);
        ++p_it;
        ++p_kb;
      }
    };
    if (threadIdx.x == 0) {
      griddep_wait();  // the kernel before this one in the stream may have written A or B
      p_have = p_units.next(p_w);
      if constexpr (!kPair) produce(1u);
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
    __syncwarp();  // thread 0 rejoins its warp before the block-wide barrier
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    if (threadIdx.x == 0) KCG_TL(1);

    if (warp == 0) {
      // ------------------------------------------------------------ producer
      if (lane == 0) {
        produce(0xffffffffu);
        // Every load of this CTA is issued: the next kernel of the stream may be brought in as SMs
        // fall free (not earlier: a kernel that took SMs while CTAs of this one still waited for
        // theirs would keep waiting for this one in vain).
        griddep_launch_dependents();
      }
    } else if (warp == 1) {
      // -------------------------- MMA issuer (in a pair: the leader CTA only)
      if (lane == 0 && rank == 0u) {
        uint32_t it = 0, acc_it = 0;
        bool ok = true;
        Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
        Unit w;
        // The MMAs of K block (it, kb) of the unit; accumulators [t0, t1) only.
        auto issue = [&](uint32_t s, int kb, int t0, int t1, uint32_t tmem_acc) {
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + L.a_bytes;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a_off, b_off;
            if constexpr (kATrans) {
              a_off = ks * UMMA_K * 128;
            } else {
              constexpr int swb = (kBK * EB < 128) ? kBK * EB : 128;
              a_off = ((ks * 32) / swb) * L.a_box_bytes + ((ks * 32) % swb);
            }
            if constexpr (kBTrans) {
              constexpr int swb = (kBK * EB < 128) ? kBK * EB : 128;
              b_off = ((ks * 32) / swb) * L.b_box_bytes + ((ks * 32) % swb);
            } else {
              b_off = ks * UMMA_K * 128;
            }
            const uint32_t acc_flag = (kb > 0 || ks > 0) ? 1u : 0u;
            for (int t = t0; t < t1; ++t) {
              // second accumulator: local A rows 128..255. Two accumulators also keep
              // consecutive MMAs independent of each other, which the tensor pipe needs to
              // stay full (a single accumulator chain measured ~10 % slower).
              const uint32_t a_t = kATrans ? t * (128 / L.atom) * L.a_box_bytes
                                           : t * 128 * (L.a_box_bytes / R);
              const uint64_t bdesc = make_smem_desc(sb + b_off, L.b_lbo, L.b_sbo, L.b_desc_swizzle);
              const uint64_t adesc =
                  make_smem_desc(sa + a_t + a_off, L.a_lbo, L.a_sbo, L.a_desc_swizzle);
              const uint32_t d = tmem_acc + t * kBN;
#ifndef KCG_PROBE_NO_MMA  // measurement builds only: loads and barriers run, the products do not
              if constexpr (kPair) {
                umma_ss_pair<kTf32>(d, adesc, bdesc, IDESC, acc_flag);
              } else {
                umma_ss<kTf32>(d, adesc, bdesc, IDESC, acc_flag);
              }
#endif
            }
          }
        };
        // stage reusable (in both CTAs of a pair) once the MMAs issued so far retire
        auto free_stage = [&](uint32_t s) {
          if constexpr (kPair) {
            umma_commit_pair(smem_u32(&bars->empty[s]));
            umma_commit_pair(map_to_cta(smem_u32(&bars->empty[s]), 1u));
          } else {
            umma_commit(&bars->empty[s]);
          }
        };
        for (; ok && units.next(w); ++acc_it) {
          const uint32_t ab = acc_it % NACC;
          const uint32_t aph = (acc_it / NACC) & 1u;
          if (!mbar_wait(&bars->tmem_empty[ab], aph ^ 1u, &bars->abort_flag)) {
            report(p, bars, KCG_ST_TIMEOUT_MMA, 0x100u + ab, acc_it);
            break;
          }
          tc_fence_after_sync();
          const uint32_t tmem_acc = tmem_base + ab * ACC_COLS;
          int kb = 0;
          if constexpr (HALF) {
            // Accumulator 0 is drained (the wait above), accumulator 1 maybe not yet: run the first
            // K blocks into accumulator 0 alone, keeping their stages, then - once the epilogue has
            // let go of accumulator 1 - the same blocks into accumulator 1, and free the stages.
            const int pro = w.kbn < HALF_KB ? w.kbn : HALF_KB;
            for (int j = 0; j < pro; ++j) {
              const uint32_t s = (it + j) % kStages;
              const uint32_t ph = ((it + j) / kStages) & 1u;
              if (!mbar_wait(&bars->full[s], ph, &bars->abort_flag)) {
                report(p, bars, KCG_ST_TIMEOUT_MMA, it + j, s);
                ok = false;
                break;
              }
              tc_fence_after_sync();
              issue(s, j, 0, 1, tmem_acc);
            }
            if (!ok) break;
            if (!mbar_wait(&bars->tmem_empty[1], aph ^ 1u, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_MMA, 0x101u, acc_it);
              break;
            }
            tc_fence_after_sync();
            for (int j = 0; j < pro; ++j) {
              const uint32_t s = (it + j) % kStages;
              issue(s, j, 1, 2, tmem_acc);
              free_stage(s);
            }
            it += pro;
            kb = pro;
          }
          for (; kb < w.kbn; ++kb, ++it) {
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            KCG_TLC(c_wait);
            if (!mbar_wait(&bars->full[s], ph, &bars->abort_flag)) {
              report(p, bars, KCG_ST_TIMEOUT_MMA, it, s);
              ok = false;
              break;
            }
            KCG_TLC_ADD(12, c_wait);
            tc_fence_after_sync();
            if (it == 0) KCG_TL(3);
            KCG_TLC(c_issue);
            issue(s, kb, 0, MT, tmem_acc);
            free_stage(s);
            KCG_TLC_ADD(13, c_issue);
          }
          if (acc_it == 0) KCG_TL(4);
          if (acc_it < 4) KCG_TL(24 + acc_it);  // MMAs of the CTA's first four units issued
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
    } else if (warp >= 6) {
      griddep_wait();
      // ------------------------------------- push warps (fused all-gather only)
      // They walk the same unit sequence; for every whole-K tile they wait until the four epilogue
      // warps have completed its stores, then copy this CTA's rows of the tile from this GPU's C
      // (still in L2) to the same place in every peer's C with coalesced 16-byte loads and
      // stores. They lag behind the epilogue as far as NVLink makes them; nothing waits for them
      // before the end of the kernel. K-split tiles are written to the peers by their reducer.
      if (p.n_peers > 0) {
        const int pw = warp - 6;
        constexpr int ROW_U4 = kBN * static_cast<int>(sizeof(OutT)) / 16;  // 16-byte pieces per tile row
        constexpr int TOTAL = R * ROW_U4;
        constexpr int UNR = 8;
        uint32_t whole = 0;  // whole-K tiles seen so far
        Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
        Unit w;
        bool ok = true;
        while (ok && units.next(w)) {
          if (w.nsplit != 1) continue;
          ++whole;
          const uint32_t want = 4u * whole;
          const uint64_t t0 = global_timer_ns();
          uint32_t spins = 0;
          while (*reinterpret_cast<volatile uint32_t*>(&bars->push_count) < want) {
            if ((++spins & 63u) == 0u) {
              if (bars->abort_flag != 0u || global_timer_ns() - t0 > KCG_WAIT_LIMIT_NS) {
                if (lane == 0 && bars->abort_flag == 0u) report(p, bars, KCG_ST_TIMEOUT_PUSHER, whole, want);
                ok = false;
                break;
              }
              __nanosleep(200);
            }
          }
          if (!ok) break;
          __threadfence();  // acquire: the tile's rows as the epilogue warps published them
          const OutT* src0 = reinterpret_cast<const OutT*>(p.C);
          for (int base = pw * 32 + lane; base < TOTAL; base += 32 * NUM_PUSH_WARPS * UNR) {
            uint4 v[UNR];
            size_t off[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
              const int idx = base + u * 32 * NUM_PUSH_WARPS;
              const int row = w.m0 + row_base + idx / ROW_U4;
              const int col = w.n0 + (idx % ROW_U4) * (16 / static_cast<int>(sizeof(OutT)));
              const bool in = idx < TOTAL && row < p.M && col < p.N;
              off[u] = in ? static_cast<size_t>(row) * p.ldc + col : static_cast<size_t>(-1);
              if (in) v[u] = __ldcg(reinterpret_cast<const uint4*>(src0 + off[u]));
            }
            for (int pe = 0; pe < p.n_peers; ++pe) {
              OutT* dst = reinterpret_cast<OutT*>(p.peerC[pe]);
#pragma unroll
              for (int u = 0; u < UNR; ++u)
                if (off[u] != static_cast<size_t>(-1)) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
            }
          }
        }
        __threadfence_system();  // peer stores ordered before the kernel's completion
      }
    } else {
      // ------------------------------------------------------------ epilogue
      griddep_wait();  // C, the workspace and the counters may still be in use by the kernel before
      const int q = warp & 3;  // TMEM lane quarter this warp may read
      const int epi_tid = (warp - 2) * 32 + lane;
      uint32_t acc_it = 0;
      OutT* Cout = reinterpret_cast<OutT*>(p.C);
      uint8_t* stg = smem + kStages * STAGE_BYTES + 1024 + (warp - 2) * (2 * STG_BYTES);
      uint32_t stg_it = 0;  // staging buffers this warp has filled
      uint32_t red_phase = 0;  // parity of red_full
      if (warp == 2 && lane == 0) tma_prefetch_desc(&p.tmC);
      Iter units(p, unit0, unit_stride, tiles_m, tiles_n, num_kb);
      Unit w;
      for (; units.next(w); ++acc_it) {
        const uint32_t ab = acc_it % NACC;
        const uint32_t aph = (acc_it / NACC) & 1u;
        // The four epilogue warps leave the wait as one (named barrier 2 ANDs their outcomes):
        // tcgen05.ld below is warp-collective, and the K-split path meets on named barrier 1, where
        // a warp that had given up alone - by the abort flag or its own time limit - would leave
        // the other three waiting for its threads for ever.
        const bool got = mbar_wait(&bars->tmem_full[ab], aph, &bars->abort_flag);
        if (!named_bar_all(2, NUM_EPI_THREADS, got)) {
          if (!got) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, acc_it, ab);
          break;
        }
        tc_fence_after_sync();
        if (warp == 2 && lane == 0 && acc_it == 0) KCG_TL(5);
        const uint32_t tmem_acc = tmem_base + ab * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
        // This warp has read all it needs of accumulator buffer (or, in HALF mode, accumulator) `idx`.
        auto release = [&](uint32_t idx) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[idx]), 0u));
            } else {
              mbar_arrive(&bars->tmem_empty[idx]);
            }
          }
        };
        if (w.nsplit == 1) {
          // Whole-K tile: each warp converts 32 rows x 128 bytes at a time into its own
          // staging buffer (16-byte units XOR-swizzled by row, so neither the writes nor the
          // TMA engine's reads conflict on banks) and one lane hands it to a TMA store. Two
          // buffers per warp keep a store in flight while the next block is converted.
#pragma unroll 1
          for (int t = 0; t < MT; ++t) {
            const int row0 = w.m0 + row_base + t * 128 + q * 32;
#pragma unroll 1
            for (int g = 0; g < kBN / SCOLS; ++g, ++stg_it) {
              uint8_t* buf = stg + (stg_it & 1u) * STG_BYTES;
              KCG_TLC(c_e0);
              if (lane == 0) tma_store_wait_read<1>();  // the store that last read `buf` is done
              __syncwarp();
              if (warp == 2 && lane == 0) KCG_TLC_ADD(20, c_e0);
              KCG_TLC(c_e1);
              uint32_t ra[32], rb[32];  // rb: columns 32..63 of a 16-bit block
              tmem_ld_32x32b_x32(tmem_acc + t * kBN + g * SCOLS, ra);
              if constexpr (SCOLS == 64) tmem_ld_32x32b_x32(tmem_acc + t * kBN + g * SCOLS + 32, rb);
              tmem_ld_wait();
              if (warp == 2 && lane == 0) KCG_TLC_ADD(21, c_e1);
              KCG_TLC(c_e2);
              float va[32], vb[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                va[i] = __uint_as_float(ra[i]);
                if constexpr (SCOLS == 64) vb[i] = __uint_as_float(rb[i]);
              }
              if (p.epi_flags != 0u && row0 + lane < p.M) {
                epi_span<OutT, 32>(p, va, row0 + lane, w.n0 + g * SCOLS);
                if constexpr (SCOLS == 64) epi_span<OutT, 32>(p, vb, row0 + lane, w.n0 + g * SCOLS + 32);
              }
              uint8_t* rowp = buf + lane * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint4 o;
                if constexpr (sizeof(OutT) == 4) {
                  o = make_uint4(__float_as_uint(va[4 * j]), __float_as_uint(va[4 * j + 1]),
                                 __float_as_uint(va[4 * j + 2]), __float_as_uint(va[4 * j + 3]));
                } else {
                  uint32_t h[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float lo = (j < 4) ? va[8 * (j & 3) + 2 * i] : vb[8 * (j & 3) + 2 * i];
                    const float hi = (j < 4) ? va[8 * (j & 3) + 2 * i + 1] : vb[8 * (j & 3) + 2 * i + 1];
                    if constexpr (kDType == KCG_DT_BF16) {
                      __nv_bfloat162 x = __floats2bfloat162_rn(lo, hi);
                      h[i] = *reinterpret_cast<uint32_t*>(&x);
                    } else {
                      __half2 x = __floats2half2_rn(lo, hi);
                      h[i] = *reinterpret_cast<uint32_t*>(&x);
                    }
                  }
                  o = make_uint4(h[0], h[1], h[2], h[3]);
                }
                *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = o;
              }
              if (warp == 2 && lane == 0) KCG_TLC_ADD(22, c_e2);
              KCG_TLC(c_e3);
              fence_proxy_async_smem();  // generic-proxy writes visible to the TMA engine
              __syncwarp();
              const int col0 = w.n0 + g * SCOLS;
              if (lane == 0 && row0 < p.M && col0 < p.N) {
                tma_store_2d(&p.tmC, buf, col0, row0);  // rows / columns past the edge are clipped
                tma_store_commit();
              }
              if (warp == 2 && lane == 0) KCG_TLC_ADD(23, c_e3);
            }
            if constexpr (HALF) release(static_cast<uint32_t>(t));
          }
          if (p.n_peers > 0) {
            // Fused all-gather: once this warp's rows of the tile are in C (stores complete, and
            // ordered before generic-proxy reads), tell the push warps, which copy the tile to
            // every peer while the next tiles are computed.
            if (lane == 0) {
              tma_store_wait_all<0>();
              fence_proxy_async_all();
              __threadfence();
              atomicAdd(&bars->push_count, 1u);
            }
            __syncwarp();
          }
        } else {
          // K-split partial: the fp32 accumulators leave through the same staging buffers, as
          // 32-row x 32-column blocks (128 bytes per row), and TMA stores into the workspace,
          // whose slots form one tall matrix of kBN columns. Full 128-byte lines: 16-byte stores
          // straight from each thread's row made L2 read-modify-write every sector and cost
          // tens of microseconds per partial tile.
#pragma unroll 1
          for (int t = 0; t < MT; ++t) {
            const int wrow0 = w.slot * kBM + row_base + t * 128 + q * 32;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c, ++stg_it) {
              uint8_t* buf = stg + (stg_it & 1u) * STG_BYTES;
              if (lane == 0) tma_store_wait_read<1>();
              __syncwarp();
              uint32_t r[32];
              if (w.kbn > 0) {
                tmem_ld_32x32b_x32(tmem_acc + t * kBN + c * 32, r);
                tmem_ld_wait();
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
              }
              uint8_t* rowp = buf + lane * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) =
                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&p.tmWs, buf, c * 32, wrow0);
                tma_store_commit();
              }
            }
            if constexpr (HALF) release(static_cast<uint32_t>(t));
          }
        }
        if constexpr (!HALF) release(ab);
        if (warp == 2 && lane == 0 && acc_it == 0) KCG_TL(6);

        if (w.nsplit > 1) {
          // Publish this split's partial tile; then the partials are summed, always in split order
          // (bitwise reproducible), by one of two protocols on the tile's counter word
          // (arrivals in bits 0-7, shares given up in bits 8-15, shares done in bits 16-23):
          //  * w.share = 0: the last contributor to arrive sums the whole tile;
          //  * w.share > 0: contributors 0 .. share-1 wait a short while for all partials and sum one
          //    share-th of the CTA's rows each, so the reduction runs on several SMs at once
          //    (out of the operand ring when this is the CTA's last unit and the ring is idle,
          //    straight from L2 while the next unit's main loop runs otherwise). A waiter that runs
          //    out of patience (the other CTAs may not be running: another kernel can hold their
          //    SMs while this one holds theirs) records its share as given up and goes on; the last
          //    contributor to arrive - who never waits - sums the shares given up before it came.
          // Whoever finishes the last share zeroes the word for the next launch.
          const int ctr = (w.tile - first_split) * NCTA + static_cast<int>(rank);  // per CTA half
          if (lane == 0) tma_store_wait_all<0>();  // this warp's blocks of the partial are written
          fence_proxy_async_all();                 // ... and ordered before the generic-proxy release below
          __threadfence();
          named_bar_sync(1, NUM_EPI_THREADS);
          const bool sharer = w.split < w.share;
          if (epi_tid == 0) {
            const unsigned int all = static_cast<unsigned int>(w.nsplit);
            const unsigned int old = atomicAdd(&p.tile_counters[ctr], 1u);
            const bool came_last = (old & 0xffu) == all - 1u;
            unsigned int mine = 0u;  // bit s: this CTA sums share s
            if (w.share == 0) {
              if (came_last) {
                mine = 1u;
                p.tile_counters[ctr] = 0u;
              }
            } else {
              if (came_last) mine = (old >> 8) & 0xffu;
              if (sharer) {
                bool go = came_last;
                if (!go) {
                  const uint64_t t0 = global_timer_ns();
                  for (;;) {
                    if ((ld_acquire_gpu(&p.tile_counters[ctr]) & 0xffu) == all) {
                      go = true;
                      break;
                    }
                    if (bars->abort_flag != 0u || global_timer_ns() - t0 > KCG_SHARE_WAIT_NS) break;
                    __nanosleep(40);
                  }
                  if (!go) {
                    // give the share up - unless the last partial came in the meantime: then nobody
                    // has seen the bit, and the share is still this CTA's
                    const unsigned int seen = atomicOr(&p.tile_counters[ctr], 1u << (8 + w.split));
                    go = (seen & 0xffu) == all;
                  }
                }
                if (go) mine |= 1u << w.split;
              }
            }
            bars->last_flag = mine;
          }
          named_bar_sync(1, NUM_EPI_THREADS);
          const unsigned int mine = bars->last_flag;
          if (warp == 2 && lane == 0 && acc_it == 0) KCG_TL(14);
          bool ok = true;
          if (mine != 0u) {
            __threadfence();
            // This CTA's R rows of the tile are contiguous in every partial. 16-byte pieces are
            // summed in K order and written to C by consecutive threads (whole 128-byte lines per
            // quarter warp).
            constexpr int F4_PER_ROW = kBN / 4;
            const size_t slot0 = static_cast<size_t>(w.slot - w.split);
            auto emit = [&](int idx, const float4& sum) {  // idx: piece within this CTA's rows of the tile
              const int row = w.m0 + row_base + idx / F4_PER_ROW;
              const int col = w.n0 + (idx % F4_PER_ROW) * 4;
              if (row >= p.M || col >= p.N) return;
              float o[4] = {sum.x, sum.y, sum.z, sum.w};
              if (p.epi_flags != 0u) epi_span<OutT, 4>(p, o, row, col);
              const size_t off = static_cast<size_t>(row) * p.ldc + col;
              if constexpr (sizeof(OutT) == 4) {
                const float4 out = make_float4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<float4*>(Cout + off) = out;
                for (int pe = 0; pe < p.n_peers; ++pe)
                  *reinterpret_cast<float4*>(reinterpret_cast<OutT*>(p.peerC[pe]) + off) = out;
              } else {
                uint2 out;
                if constexpr (kDType == KCG_DT_BF16) {
                  __nv_bfloat162 l2 = __floats2bfloat162_rn(o[0], o[1]), h2 = __floats2bfloat162_rn(o[2], o[3]);
                  out = make_uint2(*reinterpret_cast<uint32_t*>(&l2), *reinterpret_cast<uint32_t*>(&h2));
                } else {
                  __half2 l2 = __floats2half2_rn(o[0], o[1]), h2 = __floats2half2_rn(o[2], o[3]);
                  out = make_uint2(*reinterpret_cast<uint32_t*>(&l2), *reinterpret_cast<uint32_t*>(&h2));
                }
                *reinterpret_cast<uint2*>(Cout + off) = out;
                for (int pe = 0; pe < p.n_peers; ++pe)
                  *reinterpret_cast<uint2*>(reinterpret_cast<OutT*>(p.peerC[pe]) + off) = out;
              }
            };
            // Sum of blocks [b_lo, b_hi) of the CTA's rows of the tile - 32 rows x one staging buffer's
            // width each, dealt to the four warps in turn - straight from L2, leaving like a whole
            // tile's C: packed into the warp's swizzled staging buffers and written by TMA stores.
            // Used while the operand ring is busy with the next unit.
            constexpr int BLK_PER_ROWBLOCK = kBN / SCOLS;
            constexpr int NBLK = (R / 32) * BLK_PER_ROWBLOCK;
            auto sum_blocks = [&](int b_lo, int b_hi) {
              constexpr int PPR = SCOLS / 4;               // 16-byte pieces of a partial per block row
              constexpr int PIECES = 32 * PPR;             // ... per block
              constexpr int UNR = 8, JB = 2;  // pieces per lane and partials fetched before any is added
              for (int blk = b_lo + (warp - 2); blk < b_hi; blk += 4, ++stg_it) {
                const int rb = blk / BLK_PER_ROWBLOCK, g = blk - rb * BLK_PER_ROWBLOCK;
                uint8_t* buf = stg + (stg_it & 1u) * STG_BYTES;
                if (lane == 0) tma_store_wait_read<1>();  // the store that last read `buf` is done
                __syncwarp();
                const uint32_t buf_s = smem_u32(buf);
#pragma unroll 1
                for (int q0 = 0; q0 < PIECES; q0 += 32 * UNR) {
                  float4 acc[UNR];
#pragma unroll
                  for (int u = 0; u < UNR; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                  for (int s0 = 0; s0 < w.nsplit; s0 += JB) {
                    float4 x[JB][UNR];
#pragma unroll
                    for (int j = 0; j < JB; ++j) {
                      if (s0 + j < w.nsplit) {
                        const float* src = p.splitk_ws + ((slot0 + s0 + j) * kBM + row_base + rb * 32) * kBN + g * SCOLS;
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                          const int q = q0 + u * 32 + lane;
                          x[j][u] = __ldcg(reinterpret_cast<const float4*>(src + (q / PPR) * kBN + (q % PPR) * 4));
                        }
                      }
                    }
#pragma unroll
                    for (int j = 0; j < JB; ++j) {
                      if (s0 + j < w.nsplit) {
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                          acc[u].x += x[j][u].x;
                          acc[u].y += x[j][u].y;
                          acc[u].z += x[j][u].z;
                          acc[u].w += x[j][u].w;
                        }
                      }
                    }
                  }
#pragma unroll
                  for (int u = 0; u < UNR; ++u) {
                    const int q = q0 + u * 32 + lane;
                    const int r = q / PPR, k = q % PPR;
                    float o[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
                    if (p.epi_flags != 0u) {
                      const int row = w.m0 + row_base + rb * 32 + r;
                      if (row < p.M) epi_span<OutT, 4>(p, o, row, w.n0 + g * SCOLS + k * 4);
                    }
                    const uint32_t rowp = buf_s + static_cast<uint32_t>(r) * 128u;
                    if constexpr (sizeof(OutT) == 4) {
                      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(rowp + ((static_cast<uint32_t>(k) ^ (r & 7)) << 4)),
                                   "f"(o[0]), "f"(o[1]), "f"(o[2]), "f"(o[3])
                                   : "memory");
                    } else {
                      uint32_t lo2, hi2;
                      if constexpr (kDType == KCG_DT_BF16) {
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(o[0], o[1]), b2 = __floats2bfloat162_rn(o[2], o[3]);
                        lo2 = *reinterpret_cast<uint32_t*>(&a2);
                        hi2 = *reinterpret_cast<uint32_t*>(&b2);
                      } else {
                        __half2 a2 = __floats2half2_rn(o[0], o[1]), b2 = __floats2half2_rn(o[2], o[3]);
                        lo2 = *reinterpret_cast<uint32_t*>(&a2);
                        hi2 = *reinterpret_cast<uint32_t*>(&b2);
                      }
                      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(rowp + ((static_cast<uint32_t>(k >> 1) ^ (r & 7)) << 4) +
                                                                         static_cast<uint32_t>(k & 1) * 8u),
                                   "r"(lo2), "r"(hi2)
                                   : "memory");
                    }
                  }
                }
                fence_proxy_async_smem();  // generic-proxy writes visible to the TMA engine
                __syncwarp();
                const int row0 = w.m0 + row_base + rb * 32, col0 = w.n0 + g * SCOLS;
                if (lane == 0 && row0 < p.M && col0 < p.N) {
                  tma_store_2d(&p.tmC, buf, col0, row0);  // rows / columns past the edge are clipped
                  tma_store_commit();
                }
              }
            };
            // Shares are runs of such blocks when every split unit of the launch is followed by whole
            // tiles (even split, split units first), else runs of rows (contiguous in a partial: what
            // the bulk copies into the ring want).
            const bool by_blocks = p.split_units_first != 0 && p.sk_per == 0 && first_split > 0;
            const int nshares = w.share > 0 ? w.share : 1;
            const int rows_per = (R + nshares - 1) / nshares;
            for (int s = 0; s < nshares && ok; ++s) {
              if (!((mine >> s) & 1u)) continue;
              const int r_lo = s * rows_per;
              const int r_hi = r_lo + rows_per < R ? r_lo + rows_per : R;
              if (p.n_peers == 0 && (by_blocks || w.share == 0)) {
                sum_blocks(w.share == 0 ? 0 : s * NBLK / nshares, w.share == 0 ? NBLK : (s + 1) * NBLK / nshares);
              } else if (sharer && w.last) {
                // This is the CTA's last unit, so its operand ring is idle (every load has landed
                // and every MMA that read it has retired: the accumulator was seen full). The rows
                // of all partials come in as bulk copies, as many rows at a time as the ring
                // holds - far more bytes in flight than registers could hold, which is what the L2
                // round trip asks for - and are summed out of shared memory.
                constexpr int ROW_BYTES = kBN * 4;
                constexpr int OUT_ROW_BYTES = kBN * static_cast<int>(sizeof(OutT));
                constexpr int RING_BYTES = kStages * STAGE_BYTES;
                const int max_rows = RING_BYTES / (ROW_BYTES * w.nsplit + OUT_ROW_BYTES);
                ok = max_rows > 0;
                // The sums leave as one bulk copy per row of the tile (plain stores from 128 threads
                // reach only a few GB/s: too few of them are in flight for an L2 round trip each):
                // they are packed into the ring behind the partials first. Not for the fused
                // all-gather (the peers get plain stores) nor for a tile that hangs over C's edge.
                const bool bulk_out = p.n_peers == 0 && w.n0 + kBN <= p.N;
                for (int r0 = r_lo; r0 < r_hi && ok; r0 += max_rows) {
                  const int nr = r_hi - r0 < max_rows ? r_hi - r0 : max_rows;
                  const uint32_t bytes = static_cast<uint32_t>(nr) * ROW_BYTES;
                  if (lane == 0) tma_store_wait_read<0>();  // ... also by the bulk copies of the sums
                  named_bar_sync(1, NUM_EPI_THREADS);  // earlier rows have been read out of the ring
                  if (epi_tid == 0) {
                    fence_proxy_async_all();  // the acquire above, before the async-proxy reads of the partials
                    mbar_expect_tx(&bars->red_full, bytes * static_cast<uint32_t>(w.nsplit));
                    for (int j = 0; j < w.nsplit; ++j)
                      bulk_load_1d(smem + static_cast<size_t>(j) * bytes,
                                   p.splitk_ws + ((slot0 + j) * kBM + row_base + r0) * kBN, bytes, &bars->red_full);
                  }
                  const bool got = mbar_wait(&bars->red_full, red_phase, &bars->abort_flag);
                  red_phase ^= 1u;
                  ok = named_bar_all(2, NUM_EPI_THREADS, got);
                  if (!ok) break;
                  if (warp == 2 && lane == 0 && acc_it == 0) KCG_TL(16);
                  const int pieces = nr * F4_PER_ROW;
                  // four pieces per thread at a time: their loads from shared memory are independent,
                  // so a step of the sum costs one load latency, not four
                  constexpr int U = 4;
                  const uint32_t ring = smem_u32(smem);
                  for (int i0 = epi_tid; i0 < pieces; i0 += NUM_EPI_THREADS * U) {
                    float4 sum[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int j = 0; j < w.nsplit; ++j) {
                      const uint32_t src = ring + static_cast<uint32_t>(j) * bytes;
                      float4 x[U];
#pragma unroll
                      for (int u = 0; u < U; ++u) {
                        const int i = i0 + u * NUM_EPI_THREADS;
                        x[u] = ld_shared_f4(src + static_cast<uint32_t>(i < pieces ? i : i0) * 16u);
                      }
#pragma unroll
                      for (int u = 0; u < U; ++u) {
                        sum[u].x += x[u].x;
                        sum[u].y += x[u].y;
                        sum[u].z += x[u].z;
                        sum[u].w += x[u].w;
                      }
                    }
                    if (bulk_out) {
                      const uint32_t out = ring + static_cast<uint32_t>(w.nsplit) * bytes;
#pragma unroll
                      for (int u = 0; u < U; ++u) {
                        const int i = i0 + u * NUM_EPI_THREADS;
                        if (i >= pieces) continue;
                        float o[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
                        if (p.epi_flags != 0u) {
                          const int idx = r0 * F4_PER_ROW + i;
                          epi_span<OutT, 4>(p, o, w.m0 + row_base + idx / F4_PER_ROW, w.n0 + (idx % F4_PER_ROW) * 4);
                        }
                        if constexpr (sizeof(OutT) == 4) {
                          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(out + static_cast<uint32_t>(i) * 16u),
                                       "f"(o[0]), "f"(o[1]), "f"(o[2]), "f"(o[3])
                                       : "memory");
                        } else {
                          uint32_t lo2, hi2;
                          if constexpr (kDType == KCG_DT_BF16) {
                            __nv_bfloat162 a2 = __floats2bfloat162_rn(o[0], o[1]), b2 = __floats2bfloat162_rn(o[2], o[3]);
                            lo2 = *reinterpret_cast<uint32_t*>(&a2);
                            hi2 = *reinterpret_cast<uint32_t*>(&b2);
                          } else {
                            __half2 a2 = __floats2half2_rn(o[0], o[1]), b2 = __floats2half2_rn(o[2], o[3]);
                            lo2 = *reinterpret_cast<uint32_t*>(&a2);
                            hi2 = *reinterpret_cast<uint32_t*>(&b2);
                          }
                          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(out + static_cast<uint32_t>(i) * 8u), "r"(lo2),
                                       "r"(hi2)
                                       : "memory");
                        }
                      }
                    } else {
#pragma unroll
                      for (int u = 0; u < U; ++u) {
                        const int i = i0 + u * NUM_EPI_THREADS;
                        if (i < pieces) emit(r0 * F4_PER_ROW + i, sum[u]);
                      }
                    }
                  }
                  if (bulk_out) {
                    fence_proxy_async_smem();  // the packed sums, before the async-proxy reads of the copies
                    named_bar_sync(1, NUM_EPI_THREADS);
                    if (lane == 0) {
                      const uint32_t out = ring + static_cast<uint32_t>(w.nsplit) * bytes;
                      for (int r = warp - 2; r < nr; r += 4) {
                        const int row = w.m0 + row_base + r0 + r;
                        if (row < p.M)
                          bulk_store_1d(Cout + static_cast<size_t>(row) * p.ldc + w.n0,
                                        out + static_cast<uint32_t>(r) * OUT_ROW_BYTES, OUT_ROW_BYTES);
                      }
                      tma_store_commit();
                    }
                  }
                }
              } else {
                // Rows straight from L2 with plain stores of C (and of the peers' copies of it): the
                // slow way, for the fused all-gather's split tiles and for row shares handed to a
                // last arriver whose ring is busy.
                constexpr int UNR = 2;
                const int hi = r_hi * F4_PER_ROW;
                for (int base = r_lo * F4_PER_ROW + epi_tid; base < hi; base += NUM_EPI_THREADS * UNR) {
                  float4 acc[UNR];
#pragma unroll
                  for (int u = 0; u < UNR; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                  for (int s0 = 0; s0 < w.nsplit; s0 += 4) {
                    float4 x[4][UNR];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      if (s0 + j < w.nsplit) {
                        const float4* src = reinterpret_cast<const float4*>(
                            p.splitk_ws + ((slot0 + s0 + j) * kBM + row_base) * kBN);
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                          const int idx = base + u * NUM_EPI_THREADS;
                          if (idx < hi) x[j][u] = __ldcg(src + idx);
                        }
                      }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      if (s0 + j < w.nsplit) {
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                          acc[u].x += x[j][u].x;
                          acc[u].y += x[j][u].y;
                          acc[u].z += x[j][u].z;
                          acc[u].w += x[j][u].w;
                        }
                      }
                    }
                  }
#pragma unroll
                  for (int u = 0; u < UNR; ++u) {
                    const int idx = base + u * NUM_EPI_THREADS;
                    if (idx < hi) emit(idx, acc[u]);
                  }
                }
              }
            }
          }
          if (!ok) {
            if (epi_tid == 0) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 0x300u + w.split, w.tile);
            break;
          }
          named_bar_sync(1, NUM_EPI_THREADS);  // last_flag is rewritten next unit; every read of the partials is done
          if (warp == 2 && lane == 0 && acc_it == 0 && mine != 0u) KCG_TL(15);
          if (warp == 2 && lane == 0 && acc_it < 4) KCG_TL(28 + acc_it);  // epilogue of the unit (write, wait, sum) done
          if (w.share > 0 && mine != 0u && epi_tid == 0) {
            const unsigned int n = static_cast<unsigned int>(__popc(mine));
            const unsigned int old = atomicAdd(&p.tile_counters[ctr], n << 16);
            if (((old >> 16) & 0xffu) + n == static_cast<unsigned int>(w.share)) p.tile_counters[ctr] = 0u;
          }
        }
      }
      // The staging buffers must have been read before the CTA gives its shared memory back; the
      // writes themselves complete with the kernel (the fused all-gather's push warps are told about
      // written tiles earlier, tile by tile).
      if (lane == 0) tma_store_wait_read<0>();
      if (warp == 2 && lane == 0) KCG_TL(7);
      if (p.n_peers > 0) __threadfence_system();  // peer stores ordered before the kernel's completion
    }

    // ------------------------------------------------------------ common exit
    // The producer and MMA roles run in one lane; the other lanes of those warps come straight here.
    // Reconverge every warp first: the block-wide barrier below must be executed by whole warps.
    __syncwarp();
    if (bars->abort_flag != 0u) {
      // Give copies / MMAs still in flight time to land before shared memory
      // and TMEM are released.
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) {
      __syncwarp();
      cluster_sync_all();  // the peer's shared memory and TMEM stay valid until both CTAs are done
    }
    if (threadIdx.x == 0) KCG_TL(8);
    if (warp == 1) {
      __syncwarp();
      tc_fence_after_sync();
      if constexpr (kPair) {
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
      } else
        tmem_dealloc(tmem_base, TMEM_COLS);
      if (lane == 0) KCG_TL(9);
    }
#ifdef KCG_TIMELINE
    __syncthreads();
    if (threadIdx.x == 0 && blockIdx.x == 0)
      for (int i = 0; i < 16; ++i) reinterpret_cast<uint64_t*>(p.C)[i] = bars->tl[i];
#ifdef KCG_TIMELINE_PRINT  // K-split launches: another CTA's reduction may overwrite the dump in C
    if (threadIdx.x == 0 && blockIdx.x < 4) {
      auto us = [&](int i) { return bars->tl[i] ? (bars->tl[i] - bars->tl[0]) * 1e-3 : 0.0; };
      printf("KCG_TL cta %d (us after entry, first unit): accumulator full %.2f  written %.2f  published / others awaited %.2f  "
             "partials in the ring %.2f  summed %.2f  stores read %.2f  exit %.2f\n",
             static_cast<int>(blockIdx.x), us(5), us(6), us(14), us(16), us(15), us(7), us(8));
      printf("KCG_TL cta %d first four units: MMAs issued %.2f %.2f %.2f %.2f  split-unit epilogues done %.2f %.2f %.2f %.2f\n",
             static_cast<int>(blockIdx.x), us(24), us(25), us(26), us(27), us(28), us(29), us(30), us(31));
      printf("KCG_TL cta %d epilogue cycles (warp 2, all whole tiles): staging buffer free %llu  TMEM read %llu  convert + st.shared %llu  "
             "fence + TMA store issue %llu\n", static_cast<int>(blockIdx.x), bars->tl[20], bars->tl[21], bars->tl[22], bars->tl[23]);
    }
#endif
#endif
  }
};

}  // namespace kcg
