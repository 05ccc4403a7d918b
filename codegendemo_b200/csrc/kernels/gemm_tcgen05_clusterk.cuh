// Split-K GEMM on thread-block clusters for problems with few output tiles (skinny M):
// C[M,N] = A[M,K] * B[K,N], fp16 / bf16, fp32 accumulation.
//
// A cluster of kSplit CTAs owns ONE 128 x kBN output tile. CTA r of the cluster multiplies the
// r-th of kSplit equal K ranges with the usual pipeline (warp 0 TMA producer, warp 1 tcgen05.mma
// issuer, fp32 accumulator in TMEM), so kSplit times as many SMs stream B as there are tiles.
// The partial tiles never touch global memory: the tile's columns are cut into kSplit slices
// (runs of 32-column blocks, lengths differing by at most one, so any kSplit from 2 to 8 works),
// every CTA sends slice j of its accumulator to CTA j through distributed shared memory
// (st.shared::cluster), and CTA j adds the kSplit slices it received in rank order (bitwise
// reproducible) and stores its slice of C. No workspace, no counters, no waits between
// clusters; the hardware co-schedules the CTAs of a cluster, so the waits inside it cannot starve.
//
// This is LOCAL_SPLIT_U of the reference (Optimizer.cc:310-314, 389-411: thread groups of one
// block split K and reduce their partial tiles through shared memory) lifted from the thread
// groups of a block to the CTAs of a cluster.
//
// Receive buffer = the operand ring. A CTA's ring is idle once its own MMAs have retired; it says
// so to every CTA of the cluster (ring_free[r]), and only then do the others write their slices
// into it. Layout of the buffer: [source rank][32-column block][128 rows][128 bytes], the 16-byte
// units of a row XOR-swizzled by (row & 7) so that the remote stores (one row per lane) and the
// adding loop (consecutive threads, consecutive units) are both free of bank conflicts.
//
// One tile per cluster, no persistence: these shapes have fewer tiles than the GPU has SMs.
// Every wait is bounded (ptx_sm100.cuh); on expiry the role records a status code, raises the
// CTA's abort flag and all roles fall through to the common exit, which frees TMEM.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "gemm_params.h"
#include "ptx_sm100.cuh"
#include "work_iter.cuh"

namespace kcg {

template <int kDType, int kBN, int kBK, int kStages, int kATrans, int kSplit, int kGroup>
struct TcGemmClusterK {
  static constexpr int kBM = 128;
  static_assert(ck_config_error(kDType, kBN, kBK, kStages, kSplit) == 0,
                "config not buildable by the cluster split-K kernel");
  static constexpr TcLayout L = make_tc_layout(kDType, kBM, kBN, kBK, kATrans);
  static constexpr int EB = 2;
  static constexpr int UMMA_K = 16;
  static constexpr int KSTEPS = kBK / UMMA_K;
  static constexpr int STAGE_BYTES = L.stage_hi_bytes;
  static constexpr int TMEM_COLS = kc_pow2_ceil(kBN);
  // The tile's kBN / 32 column blocks of 32 are dealt to the kSplit CTAs in contiguous runs whose
  // lengths differ by at most one: block c belongs to CTA c * kSplit / NCH.
  static constexpr int NCH = kBN / 32;
  static constexpr int CB = (NCH + kSplit - 1) / kSplit;  // most 32-column blocks one CTA owns
  static constexpr int BLOCK_BYTES = 128 * 128;           // one 32-column block: 128 rows x 128 bytes
  static constexpr int SLICE_BYTES = CB * BLOCK_BYTES;    // room for one source rank's slice
  __host__ __device__ static constexpr int owner_of(int c) { return c * kSplit / NCH; }
  __host__ __device__ static constexpr int first_block_of(int r) { return (r * NCH + kSplit - 1) / kSplit; }
  static constexpr int NUM_EPI_THREADS = 128;
  static constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS;
  static constexpr int SMEM_BYTES = ck_smem_bytes(kBN, kBK, kStages);
  static_assert(kSplit * SLICE_BYTES <= kStages * STAGE_BYTES, "the ring must hold the received slices");
  static constexpr uint32_t FMT = (kDType == KCG_DT_BF16) ? FMT_BF16 : FMT_F16;
  static constexpr uint32_t IDESC = make_instr_desc(FMT, kATrans ? 1u : 0u, 1u, 128u, kBN);

  struct Barriers {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full;
    uint64_t ring_free[8];  // [r]: CTA r of the cluster no longer touches its operand ring
    uint64_t recv_full;     // all slices for this CTA have arrived (4 warps of each of kSplit CTAs)
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
#ifdef KCG_TIMELINE
    uint64_t tl[16];  // %globaltimer stamps of CTA 0's phases (experiments only; dumped over C[0, 0..])
#endif
  };
#ifdef KCG_TIMELINE
#define KCG_CTL(i) bars->tl[i] = global_timer_ns()
#else
#define KCG_CTL(i) ((void)0)
#endif
  static_assert(sizeof(Barriers) <= 1024, "barrier block exceeds its shared-memory slot");

  __device__ static __forceinline__ void report(const KcgGemmParams& p, Barriers* bars, uint32_t code,
                                                uint32_t d0, uint32_t d1) {
    bars->abort_flag = 1u;
    if (atomicCAS(p.status, 0u, code) == 0u) {
      p.status[1] = blockIdx.x;
      p.status[2] = d0;
      p.status[3] = d1;
    }
  }

  __device__ static void run(const KcgGemmParams& p) {
    using OutT = typename std::conditional<kDType == KCG_DT_BF16, __nv_bfloat16, __half>::type;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * STAGE_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kBM - 1) / kBM;
    const int tiles_n = (p.N + kBN - 1) / kBN;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
      KCG_CTL(0);
      // the first TMA instruction needs its descriptor: start fetching the maps before anything else
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      mbar_init(&bars->tmem_full, 1);
      for (int r = 0; r < 8; ++r) mbar_init(&bars->ring_free[r], 1);
      mbar_init(&bars->recv_full, 4 * kSplit);
      bars->abort_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    const uint32_t rank = cluster_cta_rank();
    // This cluster's tile and this CTA's K range. The raster (and a batched launch's offsets) come
    // from the iterator the other tcgen05 kernels use.
    WorkIter<kBM, kBN, kGroup, KCG_SERPENTINE> raster(p, 0, 1, tiles_m, tiles_n, num_kb);
    WorkUnit w;
    w.tile = static_cast<int>(blockIdx.x) / kSplit;
    raster.origin(w);
    const int per = (num_kb + kSplit - 1) / kSplit;
    const int kb0 = static_cast<int>(rank) * per;
    const int kbn = (kb0 >= num_kb) ? 0 : ((num_kb - kb0 < per) ? num_kb - kb0 : per);

    // Producer (thread 0), entered twice: before the set-up barriers for the first ring of stages - the
    // loads signal only this CTA's own barriers, which this very thread has just initialised, so the first
    // operands are in flight while TMEM is allocated and the cluster synchronises - and again as warp 0's role.
    int p_kb = 0;
    auto produce = [&](int kb_limit) {
      for (; p_kb < kbn && p_kb < kb_limit; ++p_kb) {
        const int kb = p_kb;
        const uint32_t s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1u;
        if (!mbar_wait(&bars->empty[s], ph ^ 1u, &bars->abort_flag)) {
          report(p, bars, KCG_ST_TIMEOUT_PRODUCER, kb, s);
          p_kb = kbn;
          break;
        }
        uint8_t* sa = smem + s * STAGE_BYTES;
        uint8_t* sb = sa + L.a_bytes;
        const int k0 = (kb0 + kb) * kBK;
        const int am0 = kATrans ? w.mcol : w.m0;
        const int ka = kATrans ? k0 + w.kofs : k0, kb_row = k0 + w.kofs;
        mbar_expect_tx(&bars->full[s], static_cast<uint32_t>(STAGE_BYTES));
#pragma unroll
        for (int j = 0; j < L.a_boxes; ++j) {
          if constexpr (kATrans) {
            tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s], am0 + j * L.atom, ka);
          } else {
            tma_load_2d(sa + j * L.a_box_bytes, &p.tmA, &bars->full[s], ka + j * L.a_box_inner, am0);
          }
        }
#pragma unroll
        for (int j = 0; j < L.b_boxes; ++j)
          tma_load_2d(sb + j * L.b_box_bytes, &p.tmB, &bars->full[s], w.n0 + j * L.atom, kb_row);
        if (kb == 0) KCG_CTL(2);
      }
    };
    if (threadIdx.x == 0) produce(kStages);
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
    __syncwarp();  // thread 0 rejoins its warp before the block-wide barrier
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // every CTA's barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;
    if (threadIdx.x == 0) KCG_CTL(1);

    if (warp == 0) {
      // ------------------------------------------------------------ producer
      if (lane == 0) produce(kbn);
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer
      if (lane == 0) {
        bool ok = true;
        for (int kb = 0; kb < kbn; ++kb) {
          const uint32_t s = kb % kStages;
          const uint32_t ph = (kb / kStages) & 1u;
          if (!mbar_wait(&bars->full[s], ph, &bars->abort_flag)) {
            report(p, bars, KCG_ST_TIMEOUT_MMA, kb, s);
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
            const uint64_t adesc = make_smem_desc(sa + a_off, L.a_lbo, L.a_sbo, L.a_desc_swizzle);
            const uint64_t bdesc = make_smem_desc(sb + b_off, L.b_lbo, L.b_sbo, L.b_desc_swizzle);
            umma_ss<false>(tmem_base, adesc, bdesc, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
        }
        KCG_CTL(3);
        if (ok && kbn > 0) umma_commit(&bars->tmem_full);
      }
    } else {
      // ------------------------------------------ epilogue: exchange, add, store
      const int q = warp & 3;  // TMEM lane quarter this warp may read
      const int epi_tid = (warp - 2) * 32 + lane;
      const int row = q * 32 + lane;  // row of the tile this thread holds in TMEM
      bool ok = true;
      if (kbn > 0) ok = mbar_wait(&bars->tmem_full, 0u, &bars->abort_flag);
      // the four warps take every branch below together (named barrier 2 ANDs their outcomes)
      const bool have_acc = named_bar_all(2, NUM_EPI_THREADS, ok);
      if (!have_acc && !ok) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 0u, rank);
      if (have_acc) {
        tc_fence_after_sync();
        if (epi_tid == 0) KCG_CTL(4);
        // This CTA's MMAs have retired (or it had none): its ring is free to receive slices.
        if (epi_tid == 0) {
          for (uint32_t j = 0; j < static_cast<uint32_t>(kSplit); ++j)
            mbar_arrive_cluster(map_to_cta(smem_u32(&bars->ring_free[rank]), j));
        }
        const uint32_t tmem_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        const uint32_t my_slot = smem_u32(smem) + rank * SLICE_BYTES + row * 128;
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          const uint32_t owner = static_cast<uint32_t>(owner_of(c));
          const int cbi = c - first_block_of(static_cast<int>(owner));
          // the owner's ring is idle (its MMAs retired): our slice may overwrite it
          const bool free_ = mbar_wait(&bars->ring_free[owner], 0u, &bars->abort_flag);
          if (!__all_sync(0xffffffffu, free_)) {
            if (lane == 0) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 1u, owner);
            ok = false;
            break;
          }
          uint32_t r[32];
          if (kbn > 0) {
            tmem_ld_32x32b_x32(tmem_acc + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const uint32_t dst = map_to_cta(my_slot + cbi * BLOCK_BYTES, owner);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_cluster_v4(dst + ((j ^ (row & 7)) << 4), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        if (epi_tid == 0) KCG_CTL(5);
        // Publish: every lane's stores are ordered before lane 0's release arrivals.
        fence_acq_rel_cluster();
        __syncwarp();
        if (ok && lane == 0) {
          for (uint32_t j = 0; j < static_cast<uint32_t>(kSplit); ++j)
            mbar_arrive_cluster(map_to_cta(smem_u32(&bars->recv_full), j));
        }
        bool got = ok && mbar_wait_cluster(&bars->recv_full, 0u, &bars->abort_flag);
        const bool all_in = named_bar_all(2, NUM_EPI_THREADS, got);
        if (!all_in && ok && !got) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 2u, rank);
        if (epi_tid == 0) KCG_CTL(6);
        if (all_in) {
          // Add the kSplit slices in rank (= K) order and store this CTA's columns of C.
          OutT* Cout = reinterpret_cast<OutT*>(p.C);
          const int c_first = first_block_of(static_cast<int>(rank));
          const int total = (first_block_of(static_cast<int>(rank) + 1) - c_first) * 128 * 8;  // 16-byte units
#pragma unroll 2
          for (int idx = epi_tid; idx < total; idx += NUM_EPI_THREADS) {
            const int u = idx & 7;
            const int rr = (idx >> 3) & 127;
            const int cbi = idx >> 10;
            const uint8_t* src = smem + cbi * BLOCK_BYTES + rr * 128 + ((u ^ (rr & 7)) << 4);
            float4 acc = *reinterpret_cast<const float4*>(src);
#pragma unroll
            for (int s = 1; s < kSplit; ++s) {
              const float4 x = *reinterpret_cast<const float4*>(src + s * SLICE_BYTES);
              acc.x += x.x;
              acc.y += x.y;
              acc.z += x.z;
              acc.w += x.w;
            }
            const int grow = w.m0 + rr;
            const int gcol = w.n0 + (c_first + cbi) * 32 + u * 4;
            if (grow >= p.M || gcol >= p.N) continue;
            float o[4] = {acc.x, acc.y, acc.z, acc.w};
            if (p.epi_flags != 0u) epi_span<OutT, 4>(p, o, grow, gcol);
            uint2 out;
            if constexpr (kDType == KCG_DT_BF16) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
              out = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
              __half2 lo = __floats2half2_rn(o[0], o[1]), hi = __floats2half2_rn(o[2], o[3]);
              out = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
            *reinterpret_cast<uint2*>(Cout + static_cast<size_t>(grow) * p.ldc + gcol) = out;
          }
        }
      }
    }

    // ------------------------------------------------------------ common exit
    // The producer and MMA roles run in one lane; the other lanes of those warps come straight here.
    // Reconverge every warp first: the block-wide barrier below must be executed by whole warps.
    __syncwarp();
    if (bars->abort_flag != 0u) {
      // Give copies / MMAs still in flight time to land before shared memory and TMEM are released.
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if (threadIdx.x == 64) KCG_CTL(7);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // no CTA leaves while another may still write into its shared memory
    if (warp == 1) {
      __syncwarp();
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, TMEM_COLS);
      if (lane == 0) KCG_CTL(8);
    }
#ifdef KCG_TIMELINE
    __syncthreads();
    if (threadIdx.x == 0 && blockIdx.x == 0)
      for (int i = 0; i < 9; ++i) reinterpret_cast<uint64_t*>(p.C)[i] = bars->tl[i];
#endif
  }
};

}  // namespace kcg
