// Split-K GEMM on thread-block clusters for problems with few output tiles (skinny M):
// C[M,N] = A[M,K] * B[K,N], fp16 / bf16, fp32 accumulation.
//
// A cluster of kSplit CTAs owns ONE 128 x kBN output tile. CTA r of the cluster multiplies the
// r-th of kSplit equal K ranges with the usual pipeline (warp 0 TMA producer, warp 1 tcgen05.mma
// issuer, fp32 accumulator in TMEM), so kSplit times as many SMs stream B as there are tiles.
// The partial tiles never touch global memory: the tile's columns are cut into kSplit slices
// (runs of 32-column blocks, lengths differing by at most one, so kSplit = 3 works as well as 2 and 4),
// every CTA sends slice j of its accumulator to CTA j through distributed shared memory, and CTA j
// adds the kSplit slices in rank order (bitwise reproducible) and stores its slice of C. No workspace, no counters, no waits between
// clusters; the hardware co-schedules the CTAs of a cluster, so the waits inside it cannot starve.
//
// This is LOCAL_SPLIT_U of the reference (Optimizer.cc:310-314, 389-411: thread groups of one
// block split K and reduce their partial tiles through shared memory) lifted from the thread
// groups of a block to the CTAs of a cluster.
//
// Exchange buffers = the operand ring. A CTA's ring is idle once its own MMAs have retired; it says
// so to every CTA of the cluster (ring_free[r]), and only then do the others write into it. The
// ring is then cut in two: a staging area, where the epilogue warps lay down the 32-column blocks
// of the accumulator that belong to OTHER CTAs (tcgen05.ld, one row per lane, 16-byte units of a
// row XOR-swizzled by (row & 7) so that the stores are free of bank conflicts), and a receive area
// [sender][block][128 rows][128 bytes] into which the other CTAs copy theirs. Each warp ships its
// 32 rows of a block - 4 KB, contiguous - with ONE bulk asynchronous copy (cp.async.bulk
// shared::cta -> shared::cluster) that completes on the receiver's mbarrier as transaction bytes;
// plain remote stores, 16 bytes per lane, measured several times slower. The blocks a CTA owns
// never leave its TMEM: each thread adds, for its own row, the received slices and its own
// accumulator in rank order and stores 64 bytes of C.
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
  static constexpr int SLICE_BYTES = CB * BLOCK_BYTES;    // room for one sender's slice
  static constexpr int RECV_BYTES = (kSplit - 1) * SLICE_BYTES;  // receive area: one slot per other CTA
  // staging area: the blocks of the other CTAs, in column order (at least NCH / kSplit blocks are this CTA's own)
  static constexpr int STAGE_OUT_BYTES = (NCH - NCH / kSplit) * BLOCK_BYTES;
  __host__ __device__ static constexpr int owner_of(int c) { return c * kSplit / NCH; }
  __host__ __device__ static constexpr int first_block_of(int r) { return (r * NCH + kSplit - 1) / kSplit; }
  static constexpr int NUM_EPI_THREADS = 128;
  static constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS;
  static constexpr int SMEM_BYTES = ck_smem_bytes(kBN, kBK, kStages);
  static_assert(RECV_BYTES + STAGE_OUT_BYTES <= kStages * STAGE_BYTES, "the ring must hold the exchange buffers");
  static constexpr uint32_t FMT = (kDType == KCG_DT_BF16) ? FMT_BF16 : FMT_F16;
  static constexpr uint32_t IDESC = make_instr_desc(FMT, kATrans ? 1u : 0u, 1u, 128u, kBN);

  struct Barriers {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full;
    uint64_t ring_free[4];  // [r]: CTA r of the cluster no longer touches its operand ring
    uint64_t recv_full;     // all slices for this CTA have arrived (transaction bytes of the bulk copies)
    uint64_t staged[8];     // [f]: the four epilogue warps have laid down the f-th block that leaves this CTA
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
#ifdef KCG_TIMELINE
      for (int i = 0; i < 16; ++i) bars->tl[i] = 0;
#endif
      KCG_CTL(0);
      // the first TMA instruction needs its descriptor: start fetching the maps before anything else
      tma_prefetch_desc(&p.tmA);
      tma_prefetch_desc(&p.tmB);
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&bars->full[s], 1);
        mbar_init(&bars->empty[s], 1);
      }
      mbar_init(&bars->tmem_full, 1);
      for (int r = 0; r < 4; ++r) mbar_init(&bars->ring_free[r], 1);
      mbar_init(&bars->recv_full, 1);
      for (int f = 0; f < 8; ++f) mbar_init(&bars->staged[f], 4);  // one arrival per epilogue warp
      bars->abort_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
      // what the other CTAs will copy in: (kSplit - 1) senders x this CTA's blocks x 16 KB. Posted now;
      // a copy that lands before this CTA looks is simply counted.
      const int r_me = static_cast<int>(cluster_cta_rank());
      const int nb_me = first_block_of(r_me + 1) - first_block_of(r_me);
      mbar_expect_tx(&bars->recv_full, static_cast<uint32_t>((kSplit - 1) * nb_me * BLOCK_BYTES));
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
    // The blocks this CTA owns, and the order in which the others leave it: owner by owner, starting with
    // the next rank (so that the cluster's CTAs do not all write to the same one first). As the owners'
    // runs of blocks are contiguous, the f-th block to leave is simply block (own_end + f) mod NCH.
    const int own_first = first_block_of(static_cast<int>(rank));
    const int own_end = first_block_of(static_cast<int>(rank) + 1);
    const int own_count = own_end - own_first;
    const int foreign = NCH - own_count;
    uint8_t* const stage_out = smem + RECV_BYTES;  // staging area behind the receive area
    auto block_of = [&](int f) { return (own_end + f) % NCH; };
    auto staged_at = [&](int c) {  // where block c waits to leave (the staging area skips the own blocks)
      return stage_out + (c < own_first ? c : c - own_count) * BLOCK_BYTES;
    };
    // Shipping: warps 0 and 1 are idle once the loads and the MMAs are issued; their first lanes send the
    // staged blocks (warp 0 the even ones, warp 1 the odd ones) - 16 KB, contiguous, one bulk copy each -
    // as soon as the four epilogue warps have laid a block down and its owner's ring is idle. Issuing a
    // copy takes the lane about 0.2 us, which the staging warps would otherwise spend between blocks.
    auto ship = [&](int first_f) {
      for (int f = first_f; f < foreign; f += 2) {
        const int c = block_of(f);
        const uint32_t owner = static_cast<uint32_t>(owner_of(c));
        if (!mbar_wait(&bars->staged[f], 0u, &bars->abort_flag)) {
          if (bars->abort_flag == 0u) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 3u, static_cast<uint32_t>(f));
          return;
        }
        if (!mbar_wait(&bars->ring_free[owner], 0u, &bars->abort_flag)) {
          if (bars->abort_flag == 0u) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 1u, owner);
          return;
        }
        const uint32_t slot = rank < owner ? rank : rank - 1u;  // senders in rank order, the owner left out
        const int o_first = first_block_of(static_cast<int>(owner));
        const uint32_t dst_local = smem_u32(smem) + slot * SLICE_BYTES + (c - o_first) * BLOCK_BYTES;
        bulk_copy_to_cta(map_to_cta(dst_local, owner), smem_u32(staged_at(c)), BLOCK_BYTES,
                         map_to_cta(smem_u32(&bars->recv_full), owner));
      }
    };

    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
    // Set-up meeting on named barrier 3. Warp 0 needs nothing from the others (thread 0 initialised the
    // barriers itself, and its loads signal only those), so it merely arrives and starts loading at
    // once; the MMA and epilogue warps wait for the barriers and the TMEM address.
    if (warp == 0) {
      __syncwarp();
      named_bar_arrive(3, NUM_THREADS);
    } else {
      tc_fence_before_sync();
      named_bar_sync(3, NUM_THREADS);
      tc_fence_after_sync();
    }
    // Every CTA's barriers must exist before another CTA signals them - but nothing crosses CTAs before
    // the exchange: arrive on the cluster barrier now (thread 0's fence.mbarrier_init has published the
    // fresh barriers, so the arrival itself needs no ordering), wait for it only there (cluster_wait
    // below), and keep the main loop free of the cluster's start-up skew.
    cluster_arrive_relaxed();
    const uint32_t tmem_base = (warp == 0) ? 0u : bars->tmem_base;
    if (threadIdx.x == 32) KCG_CTL(1);

    if (warp == 0) {
      // ------------------------------------------------------------ producer
      if (lane == 0) {
        griddep_wait();  // the kernel before this one in the stream may have written A or B
        for (int kb = 0; kb < kbn; ++kb) {
          const uint32_t s = kb % kStages;
          const uint32_t ph = (kb / kStages) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u, &bars->abort_flag)) {
            report(p, bars, KCG_ST_TIMEOUT_PRODUCER, kb, s);
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
      }
      __syncwarp();
      if (lane == 0) griddep_launch_dependents();  // every load is issued: the stream's next kernel may be brought in
      cluster_wait();  // set-up phase of the cluster barrier: the other CTAs' barriers exist
      if (lane == 0) {
        ship(0);
        KCG_CTL(5);
      }
      __syncwarp();
      cluster_arrive_relaxed();  // second phase (see the epilogue warps)
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
      __syncwarp();
      cluster_wait();
      if (lane == 0) {
        ship(1);
        KCG_CTL(12);
      }
      __syncwarp();
      cluster_arrive_relaxed();
    } else {
      // ------------------------------------------ epilogue: exchange, add, store
      griddep_wait();  // C may still be in use by the kernel before this one in the stream
      const int q = warp & 3;  // TMEM lane quarter this warp may read
      const int epi_tid = (warp - 2) * 32 + lane;
      const int row = q * 32 + lane;  // row of the tile this thread holds in TMEM
      bool ok = true;
      if (kbn > 0) ok = mbar_wait(&bars->tmem_full, 0u, &bars->abort_flag);
      // the four warps take every branch below together (named barrier 2 ANDs their outcomes)
      const bool have_acc = named_bar_all(2, NUM_EPI_THREADS, ok);
      if (!have_acc && !ok) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 0u, rank);
      cluster_wait();  // the other CTAs' barriers are initialised (all four warps, every lane)
      bool all_in = false;
      if (have_acc) {
        tc_fence_after_sync();
        if (epi_tid == 0) KCG_CTL(4);
        // This CTA's MMAs have retired (or it had none): its ring is free to receive slices. One lane per
        // CTA of the cluster tells it so.
        if (epi_tid < kSplit)
          mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(&bars->ring_free[rank]), static_cast<uint32_t>(epi_tid)));
        if (epi_tid == 0) KCG_CTL(9);
        const uint32_t tmem_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        // ---- stage: the blocks that belong to other CTAs are laid down in this CTA's (idle) ring in the
        // order in which they leave; the TMEM read of the next block is in flight while a block is stored.
        auto load_block = [&](int f, uint32_t (&r)[32]) {
          if (kbn > 0) {
            tmem_ld_32x32b_x32(tmem_acc + block_of(f) * 32, r);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
        };
        auto stage_block = [&](int f, const uint32_t (&r)[32]) {
          uint8_t* rowp = staged_at(block_of(f)) + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          fence_proxy_async_smem();  // generic-proxy writes visible to the bulk copy engine
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->staged[f]);
        };
        {
          uint32_t ra[32], rb[32];
          if (foreign > 0) load_block(0, ra);
#pragma unroll 1
          for (int f = 0; f < foreign; f += 2) {
            tmem_ld_wait();
            if (f + 1 < foreign) load_block(f + 1, rb);
            stage_block(f, ra);
            if (f + 1 < foreign) {
              tmem_ld_wait();
              if (f + 2 < foreign) load_block(f + 2, ra);
              stage_block(f + 1, rb);
            }
          }
        }
        if (epi_tid == 0) KCG_CTL(10);
        bool got = ok && mbar_wait_cluster(&bars->recv_full, 0u, &bars->abort_flag);
        all_in = named_bar_all(2, NUM_EPI_THREADS, got);
        if (!all_in && ok && !got) report(p, bars, KCG_ST_TIMEOUT_EPILOGUE, 2u, rank);
        if (epi_tid == 0) KCG_CTL(6);
      }
      // Second phase of the cluster barrier, which guards the CTAs' lifetimes: this CTA has received
      // everything (or has given up), so no copy into it is in flight any more. Once every CTA of the
      // cluster has said so, all copies have landed and each may leave; the wait is at the common exit,
      // behind the adding and storing below.
      cluster_arrive_relaxed();
      if (all_in) {
        const uint32_t tmem_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        {
          // ---- add: for every block this CTA owns, each thread adds - for its own row - the slices in
          // rank (= K) order, its own from TMEM, and stores 32 values of C
          OutT* Cout = reinterpret_cast<OutT*>(p.C);
          const int c_first = first_block_of(static_cast<int>(rank));
          const int c_end = first_block_of(static_cast<int>(rank) + 1);
          const int grow = w.m0 + row;
#pragma unroll 1
          for (int c = c_first; c < c_end; ++c) {
            const int cbi = c - c_first;
            uint32_t own[32];
            if (kbn > 0) {
              tmem_ld_32x32b_x32(tmem_acc + c * 32, own);
              tmem_ld_wait();
              if (epi_tid == 0 && c == c_first) KCG_CTL(15);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) own[i] = 0u;
            }
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
#pragma unroll
            for (int sdr = 0; sdr < kSplit; ++sdr) {
              if (static_cast<uint32_t>(sdr) == rank) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(own[i]);
              } else {
                const int slot = sdr < static_cast<int>(rank) ? sdr : sdr - 1;
                const uint8_t* src = smem + slot * SLICE_BYTES + cbi * BLOCK_BYTES + row * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float4 x = *reinterpret_cast<const float4*>(src + ((j ^ (row & 7)) << 4));
                  v[4 * j] += x.x;
                  v[4 * j + 1] += x.y;
                  v[4 * j + 2] += x.z;
                  v[4 * j + 3] += x.w;
                }
              }
            }
            if (epi_tid == 0 && c == c_first) KCG_CTL(11);
            const int gcol = w.n0 + c * 32;
            if (grow >= p.M || gcol >= p.N) continue;
            if (p.epi_flags != 0u) epi_span<OutT, 32>(p, v, grow, gcol);
            uint4* dst = reinterpret_cast<uint4*>(Cout + static_cast<size_t>(grow) * p.ldc + gcol);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t h[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if constexpr (kDType == KCG_DT_BF16) {
                  __nv_bfloat162 x = __floats2bfloat162_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                  h[i] = *reinterpret_cast<uint32_t*>(&x);
                } else {
                  __half2 x = __floats2half2_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                  h[i] = *reinterpret_cast<uint32_t*>(&x);
                }
              }
              dst[j] = make_uint4(h[0], h[1], h[2], h[3]);
            }
            if (epi_tid == 0 && c == c_first) KCG_CTL(13);
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
    cluster_wait();  // no CTA leaves while another may still write into its shared memory or read from it
    if (warp == 1) {
      __syncwarp();
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, TMEM_COLS);
      if (lane == 0) KCG_CTL(8);
    }
#ifdef KCG_TIMELINE
    __syncthreads();
    if (threadIdx.x == 0 && blockIdx.x == 0)
      for (int i = 0; i < 16; ++i) reinterpret_cast<uint64_t*>(p.C)[i] = bars->tl[i];
#endif
  }
};

}  // namespace kcg
