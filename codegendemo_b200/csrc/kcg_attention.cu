// Fused attention forward, O = softmax(scale * Q K^T) V per head, for fp16 / bf16 with head dimension 64 or 128:
// the attention-shaped chain (two products around a row softmax, which the reference lists after batched GEMM
// among its next operators, doc/结果汇总.md) as ONE kernel in which scores and probabilities never leave the SM.
// The three-launch form (matmul_op.attention: batched Q K^T with fp32 scores, row softmax, batched P V) stays as
// the path whose parity is pinned to the composition; this kernel is checked against the same composition.
//
// Default form (AttnFwd2): one CTA per (head, 256 query rows) = two query tiles of 128 rows, 320 threads:
//   warp 0    TMA producer: both Q tiles once, then K and V tiles of 128 keys through two-stage rings, shared by
//             the two query tiles
//   warp 1    tcgen05.mma issuer and TMEM owner; per tile t: S_t = Q_t K_j^T (both K-major) into the tile's S
//             buffer, O_t += P_t V_j with P_t read from tensor memory and V as the MN-major operand
//   warps 2-5 softmax of tile 0, warps 6-9 of tile 1, one query row per thread: read S_t from TMEM, running
//             maximum and sum in the exp2 domain, P_t as packed 16-bit pairs over the S columns just read, O_t
//             rescaled in TMEM by exp2(m_old - m_new) only by warps that saw a new maximum; at the end O / sum to
//             global memory
// A tile's chain is serial (scores, softmax, P V, next scores) and the two tiles' chains interleave, so the tensor
// pipe works for one tile while the other is in its softmax. Four single-tile forms are kept for comparison
// (AttnFwd: one query tile per CTA with two S buffers, 64- or 128-key steps, one or two threads per row, P through
// shared or tensor memory; S issued one step ahead - two steps ahead, with a third buffer, measured slower).
// Every wait is bounded (ptx_sm100.cuh); a wait that runs out records a code in a status word the host can read
// (kcg_attention_status), raises the CTA's abort flag and all roles fall through to the exit.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <string>

#include "../../include/kcg_b200.h"
#include "kernels/ptx_sm100.cuh"

extern "C" int kcg_internal_fail(int code, const char* msg);
extern "C" void kcg_internal_count_launch(void);

namespace {

using namespace kcg;

__device__ unsigned int g_attn_status[4];  // {code, block, detail, detail}; 0 = no wait ran out

// 3-D tiled load: {column, row, head}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tm, uint64_t* bar, int32_t c0,
                                            int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// registers -> TMEM: each thread of the warp writes 32 consecutive fp32 columns of its own lane (row)
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem], 16-bit operands: A is read from tensor memory (lane = row, one 32-bit column =
// two consecutive K values), B through a shared-memory descriptor. Issued by ONE thread.
__device__ __forceinline__ void umma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  CUtensorMap tmQ, tmK, tmV;  // {d, rows, heads}, boxes of {64, 128, 1}, 128-byte swizzle
  void* O;                    // heads x sq x d, contiguous
  int sq, sk;
  float scale_log2;           // scale * log2(e): the softmax runs on exp2
};

enum : uint32_t { ATTN_TIMEOUT_PRODUCER = 1, ATTN_TIMEOUT_MMA = 2, ATTN_TIMEOUT_SOFTMAX = 3 };

// kBC = keys per step (64 or 128); kSplit = threads per query row (1 or 2). With 64 keys per step and one
// thread per row a CTA needs 96 KB of shared memory (d = 128), 256 TMEM columns and 192 threads, so TWO CTAs
// share an SM and one's products fill the tensor pipe while the other is in its softmax.
// kPTmem = 1 keeps P in tensor memory: the softmax threads write it (packed pairs) over the columns of the S buffer
// they have just read, and P V takes its A operand from there, so P never crosses the shared-memory port (which
// carries every operand byte of both products and is what bounds this kernel).
template <int kD, bool kBf16, int kBC, int kSplit, int kPTmem>
struct AttnFwd {
  static constexpr int BR = 128;  // query rows per CTA (= TMEM lanes)
  static constexpr int BC = kBC;  // keys per step
  static constexpr int K_STAGES = 2;
  static constexpr int V_STAGES = (kBC == 64) ? 1 : 2;  // V_j is needed a whole softmax later than K_j
  static constexpr int NUM_SOFTMAX_THREADS = 128 * kSplit;
  static constexpr int NUM_THREADS = 64 + NUM_SOFTMAX_THREADS;  // producer, MMA issuer, softmax warps
  static constexpr int BOXES = kD / 64;             // 64 values = 128 bytes per box row
  static constexpr int QBOX_BYTES = BR * 128;       // Q: boxes of 128 rows x 128 bytes
  static constexpr int KVBOX_BYTES = BC * 128;      // K, V: boxes of BC rows x 128 bytes
  static constexpr int Q_BYTES = BR * kD * 2, KV_BYTES = BC * kD * 2, P_BYTES = kPTmem ? 0 : BR * BC * 2;
  static constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + K_STAGES * KV_BYTES, OFF_P = OFF_V + V_STAGES * KV_BYTES;
  static constexpr int RING_BYTES = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = RING_BYTES + 3072;  // 1 KB alignment slack + 2 KB barriers and exchange slots
  static constexpr uint32_t COL_O = 2 * BC;             // S0 [0, BC), S1 [BC, 2 BC), O [2 BC, 2 BC + kD)
  static constexpr uint32_t TMEM_COLS = (2 * BC + kD <= 256) ? 256 : 512;
  static constexpr uint32_t FMT = kBf16 ? FMT_BF16 : FMT_F16;
  // S = Q K^T: both operands K-major (rows x d); O += P V: P K-major (rows x keys), V MN-major (keys x d)
  static constexpr uint32_t IDESC_S = make_instr_desc(FMT, 0u, 0u, 128u, BC);
  static constexpr uint32_t IDESC_O = make_instr_desc(FMT, 0u, 1u, 128u, kD);
  static_assert((kBC == 64 || kBC == 128) && (kSplit == 1 || kSplit == 2) && (kBC / kSplit) % 32 == 0, "shape");
  using T = typename std::conditional<kBf16, __nv_bfloat16, __half>::type;

  struct Barriers {
    uint64_t q_full;
    uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
    uint64_t s_full[2], s_empty[2];
    uint64_t p_full;    // P_j is in shared memory and O is rescaled (every softmax warp arrives)
    uint64_t pv_done;   // P_j V_j has retired: P may be overwritten, O may be read
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
    float exchange[2][128];  // row maxima (and, at the end, row sums) passed between the two threads of a row
  };
  static_assert(sizeof(Barriers) <= 2048, "barrier block exceeds its shared-memory slot");

  __device__ static __forceinline__ void report(Barriers* bars, uint32_t code, uint32_t d0, uint32_t d1) {
    bars->abort_flag = 1u;
    if (atomicCAS(&g_attn_status[0], 0u, code) == 0u) {
      g_attn_status[1] = blockIdx.x;
      g_attn_status[2] = d0;
      g_attn_status[3] = d1;
    }
  }

  __device__ static void run(const AttnParams& p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + RING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = (p.sq + BR - 1) / BR;
    const int head = static_cast<int>(blockIdx.x) / q_tiles;
    const int q0 = (static_cast<int>(blockIdx.x) % q_tiles) * BR;
    const int nkv = (p.sk + BC - 1) / BC;

    if (threadIdx.x == 0) {
      tma_prefetch_desc(&p.tmQ);
      tma_prefetch_desc(&p.tmK);
      tma_prefetch_desc(&p.tmV);
      mbar_init(&bars->q_full, 1);
      for (int s = 0; s < K_STAGES; ++s) {
        mbar_init(&bars->k_full[s], 1);
        mbar_init(&bars->k_empty[s], 1);
      }
      for (int s = 0; s < V_STAGES; ++s) {
        mbar_init(&bars->v_full[s], 1);
        mbar_init(&bars->v_empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bars->s_full[b], 1);
        mbar_init(&bars->s_empty[b], 4 * kSplit);  // one arrival per softmax warp
      }
      mbar_init(&bars->p_full, 4 * kSplit);
      mbar_init(&bars->pv_done, 1);
      bars->abort_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
      // ------------------------------------------------------------------ producer
      if (lane == 0) {
        mbar_expect_tx(&bars->q_full, Q_BYTES);
#pragma unroll
        for (int b = 0; b < BOXES; ++b) tma_load_3d(smem + b * QBOX_BYTES, &p.tmQ, &bars->q_full, b * 64, q0, head);
        for (int j = 0; j < nkv; ++j) {
          const int ks = j % K_STAGES, vs = j % V_STAGES;
          if (!mbar_wait(&bars->k_empty[ks], ((j / K_STAGES) & 1u) ^ 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_PRODUCER, j, 0u);
            break;
          }
          mbar_expect_tx(&bars->k_full[ks], KV_BYTES);
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            tma_load_3d(smem + OFF_K + ks * KV_BYTES + b * KVBOX_BYTES, &p.tmK, &bars->k_full[ks], b * 64, j * BC, head);
          if (!mbar_wait(&bars->v_empty[vs], ((j / V_STAGES) & 1u) ^ 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_PRODUCER, j, 1u);
            break;
          }
          mbar_expect_tx(&bars->v_full[vs], KV_BYTES);
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            tma_load_3d(smem + OFF_V + vs * KV_BYTES + b * KVBOX_BYTES, &p.tmV, &bars->v_full[vs], b * 64, j * BC, head);
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        bool ok = mbar_wait(&bars->q_full, 0u, &bars->abort_flag);
        if (!ok) report(bars, ATTN_TIMEOUT_MMA, 0u, 0u);
        tc_fence_after_sync();
        const uint32_t sq_addr = smem_u32(smem);
        // S_i = Q K_i^T into S buffer i % 2
        auto issue_s = [&](int i) -> bool {
          const int s = i % K_STAGES, b = i & 1;
          if (!mbar_wait(&bars->k_full[s], (i / K_STAGES) & 1u, &bars->abort_flag) ||
              !mbar_wait(&bars->s_empty[b], ((i >> 1) & 1u) ^ 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_MMA, 1u, static_cast<uint32_t>(i));
            return false;
          }
          tc_fence_after_sync();
          const uint32_t sk_addr = smem_u32(smem + OFF_K + s * KV_BYTES);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks) {
            // 16 values of d = 32 bytes of a 128-byte box row; the boxes of 64 values follow one another
            const uint32_t in_row = (ks * 32) % 128, box = (ks * 32) / 128;
            const uint64_t adesc = make_smem_desc(sq_addr + box * QBOX_BYTES + in_row, 16, 1024, SWZ_128B);
            const uint64_t bdesc = make_smem_desc(sk_addr + box * KVBOX_BYTES + in_row, 16, 1024, SWZ_128B);
            umma_ss<false>(tmem_base + b * BC, adesc, bdesc, IDESC_S, ks > 0 ? 1u : 0u);
          }
          umma_commit(&bars->k_empty[s]);
          umma_commit(&bars->s_full[b]);
          return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < nkv && ok; ++j) {
          if (j + 1 < nkv) ok = issue_s(j + 1);
          if (!ok) break;
          const int s = j % V_STAGES;
          if (!mbar_wait(&bars->p_full, j & 1u, &bars->abort_flag) ||
              !mbar_wait(&bars->v_full[s], (j / V_STAGES) & 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_MMA, 2u, static_cast<uint32_t>(j));
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sp_addr = smem_u32(smem + OFF_P);
          const uint32_t sv_addr = smem_u32(smem + OFF_V + s * KV_BYTES);
#pragma unroll
          for (int ks = 0; ks < BC / 16; ++ks) {
            // P: K-major, 128 rows x BC keys in boxes of 64 keys; V: BC keys x d, its 64-value column chunks
            // are boxes of BC key rows (leading-dimension offset = one box), a K step = 16 key rows
            const uint64_t bdesc = make_smem_desc(sv_addr + ks * 16 * 128, KVBOX_BYTES, 1024, SWZ_128B);
            if constexpr (kPTmem) {
              // 16 keys = 8 columns of packed pairs in the S buffer of this step
              umma_ts_f16(tmem_base + COL_O, tmem_base + (j & 1) * BC + ks * 8, bdesc, IDESC_O,
                          (j > 0 || ks > 0) ? 1u : 0u);
            } else {
              const uint32_t a_off = ((ks * 32) / 128) * (BR * 128) + ((ks * 32) % 128);  // boxes of 64 keys
              const uint64_t adesc = make_smem_desc(sp_addr + a_off, 16, 1024, SWZ_128B);
              umma_ss<false>(tmem_base + COL_O, adesc, bdesc, IDESC_O, (j > 0 || ks > 0) ? 1u : 0u);
            }
          }
          umma_commit(&bars->v_empty[s]);
          umma_commit(&bars->pv_done);
        }
      }
    } else {
      // ------------------------------------------------- softmax, correction, epilogue
      // kSplit threads per query row. With two, warps 2-5 take the first half of a step's keys and of O's
      // columns, warps 6-9 the second; the two warps that share a TMEM lane quarter meet on a named barrier
      // of their own to combine their row maxima (the sums stay separate until the end).
      const int q = warp & 3;                // TMEM lane quarter this warp may access
      const int h = (warp - 2) >> 2;         // which part of the keys / of O's columns (0 when kSplit = 1)
      const int row = q * 32 + lane;         // query row of this thread inside the tile
      const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
      constexpr int HC = BC / kSplit;        // keys per thread and step
      constexpr int OC = kD / kSplit;        // O columns per thread
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < nkv; ++j) {
        const int b = j & 1;
        bool got = mbar_wait(&bars->s_full[b], (j >> 1) & 1u, &bars->abort_flag);
        if (!named_bar_all(2, NUM_SOFTMAX_THREADS, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 0u, static_cast<uint32_t>(j));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        float s[HC];
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + b * BC + h * HC + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_empty[b]);  // the MMA warp may overwrite this S buffer
        const int valid = p.sk - j * BC - h * HC;       // keys of this thread's half that exist
        if (valid < HC) {
#pragma unroll
          for (int i = 0; i < HC; ++i)
            if (i >= valid) s[i] = -INFINITY;
        }
        // running maximum of the raw scores (the scale is positive: checked by the host), four chains
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < HC; i += 4) {
          mx4[0] = fmaxf(mx4[0], s[i]);
          mx4[1] = fmaxf(mx4[1], s[i + 1]);
          mx4[2] = fmaxf(mx4[2], s[i + 2]);
          mx4[3] = fmaxf(mx4[3], s[i + 3]);
        }
        float rowmax = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        if constexpr (kSplit == 2) {
          bars->exchange[h][row] = rowmax;
          named_bar_sync(3 + q, 64);  // the two warps of this lane quarter
          rowmax = fmaxf(rowmax, bars->exchange[h ^ 1][row]);
          // (the slot is written again a step later, behind the vote of all softmax warps below: the partner
          // has read it by then)
        }
        const float mx = fmaxf(m, rowmax * p.scale_log2);
        const float alpha = ex2(m - mx);  // 0 on the first step (m = -inf)
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < HC; i += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[i + e] = ex2(fmaf(s[i + e], p.scale_log2, -mx));
            sum4[e] += s[i + e];
          }
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m = mx;
        // Does any row of this warp have a new maximum? Only then is O rescaled (alpha = 1 otherwise).
        const bool rescale = j > 0 && __any_sync(0xffffffffu, alpha != 1.f);
        if constexpr (kPTmem) {
          // P_j goes over the S columns this thread has read: no other step uses them, so it need not wait
          // for the previous product. Two keys per 32-bit column.
          static_assert(HC == 64, "one 32-column store per thread and step");
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if constexpr (kBf16) {
              __nv_bfloat162 v2 = __floats2bfloat162_rn(s[2 * i], s[2 * i + 1]);
              w[i] = *reinterpret_cast<uint32_t*>(&v2);
            } else {
              __half2 v2 = __floats2half2_rn(s[2 * i], s[2 * i + 1]);
              w[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
          }
          tmem_st_32x32b_x32(tmem_base + lane_addr + b * BC + h * (HC / 2), w);
        }
        // P_{j-1} V_{j-1} must have retired before O is touched - and, when P goes through shared memory, before
        // its one buffer is overwritten. (S_j is complete, so every product before P_{j-1} V_{j-1} has retired:
        // the barrier is at most one phase behind and the parity test is unambiguous even after skipped waits.)
        got = (kPTmem && !rescale) ? true : mbar_wait(&bars->pv_done, (j & 1u) ^ 1u, &bars->abort_flag);
        if (!named_bar_all(2, NUM_SOFTMAX_THREADS, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 1u, static_cast<uint32_t>(j));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if constexpr (!kPTmem) {
          // this thread's keys of its row of P: boxes of 64 keys, 16-byte units XOR-swizzled by the row
          constexpr int PBOX_BYTES = BR * 128;
          uint8_t* prow = smem + OFF_P + row * 128;
#pragma unroll
          for (int u = 0; u < HC / 8; ++u) {
            const int unit = (h * HC) / 8 + u;  // 16-byte unit inside the row of BC keys
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if constexpr (kBf16) {
                __nv_bfloat162 v2 = __floats2bfloat162_rn(s[u * 8 + 2 * e], s[u * 8 + 2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&v2);
              } else {
                __half2 v2 = __floats2half2_rn(s[u * 8 + 2 * e], s[u * 8 + 2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&v2);
              }
            }
            *reinterpret_cast<uint4*>(prow + (unit / 8) * PBOX_BYTES + (((unit % 8) ^ (row & 7)) << 4)) =
                make_uint4(w[0], w[1], w[2], w[3]);
          }
          fence_proxy_async_smem();  // P visible to the tensor core's operand reads
        }
        if (rescale) {
          // O <- alpha * O for this thread's columns
#pragma unroll
          for (int c = 0; c < OC / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem_base + lane_addr + COL_O + h * OC + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(tmem_base + lane_addr + COL_O + h * OC + c * 32, r);
          }
        }
        tmem_st_wait();  // P (when it lives in tensor memory) and the rescaled O are written
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full);
      }
      if (ok) {
        bool got = mbar_wait(&bars->pv_done, (nkv - 1) & 1u, &bars->abort_flag);
        if (!named_bar_all(2, NUM_SOFTMAX_THREADS, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 2u, 0u);
          ok = false;
        }
      }
      if (ok) {
        tc_fence_after_sync();
        if constexpr (kSplit == 2) {
          bars->exchange[h][row] = l;  // the row's sum = the two halves' sums (both relative to the same maximum)
          named_bar_sync(3 + q, 64);
          l += bars->exchange[h ^ 1][row];
        }
        const float inv = 1.f / l;
        const int grow = q0 + row;
        T* out = reinterpret_cast<T*>(p.O) + (static_cast<size_t>(head) * p.sq + grow) * kD + h * OC;
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + COL_O + h * OC + c * 32, r);
          tmem_ld_wait();
          if (grow < p.sq) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float a = __uint_as_float(r[u * 8 + 2 * e]) * inv, bb = __uint_as_float(r[u * 8 + 2 * e + 1]) * inv;
                if constexpr (kBf16) {
                  __nv_bfloat162 v2 = __floats2bfloat162_rn(a, bb);
                  w[e] = *reinterpret_cast<uint32_t*>(&v2);
                } else {
                  __half2 v2 = __floats2half2_rn(a, bb);
                  w[e] = *reinterpret_cast<uint32_t*>(&v2);
                }
              }
              *reinterpret_cast<uint4*>(out + c * 32 + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    if (bars->abort_flag != 0u) {
      // give loads / MMAs still in flight time to land before shared memory and TMEM are released
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
};

// Two query tiles per CTA. Tile 0 (rows q0 .. q0 + 127) and tile 1 (the next 128 rows) share the K and V tiles in
// shared memory and take turns on the tensor pipe: while the softmax warps of one tile work on its scores, the
// products of the other run. Each tile owns one S buffer (P is written over it) and one O accumulator in tensor
// memory - S_t [128 t, 128 t + 128), O_t [256 + kD t, ...) - and four softmax warps, one thread per row and 128 keys
// per thread and step. A tile's chain is serial (S, softmax, P V, next S: the next scores overwrite P, and the
// tensor pipe runs its instructions in order), the two chains interleave. The MMA warp serves the tiles in a fixed
// order (serving whichever P is ready first measured no faster).
template <int kD, bool kBf16>
struct AttnFwd2 {
  static constexpr int BR = 128, BC = 128, TILES = 2;
  static constexpr int K_STAGES = 2, V_STAGES = 2;
  static constexpr int NUM_THREADS = 64 + TILES * 128;
  static constexpr int BOXES = kD / 64;
  static constexpr int QBOX_BYTES = BR * 128, KVBOX_BYTES = BC * 128;
  static constexpr int Q_BYTES = BR * kD * 2, KV_BYTES = BC * kD * 2;
  static constexpr int OFF_K = TILES * Q_BYTES, OFF_V = OFF_K + K_STAGES * KV_BYTES;
  static constexpr int RING_BYTES = OFF_V + V_STAGES * KV_BYTES;
  static constexpr int SMEM_BYTES = RING_BYTES + 2048;  // 1 KB alignment slack + barriers
  static constexpr uint32_t COL_O = TILES * BC, TMEM_COLS = 512;
  static constexpr uint32_t FMT = kBf16 ? FMT_BF16 : FMT_F16;
  static constexpr uint32_t IDESC_S = make_instr_desc(FMT, 0u, 0u, 128u, BC);
  static constexpr uint32_t IDESC_O = make_instr_desc(FMT, 0u, 1u, 128u, kD);
  using T = typename std::conditional<kBf16, __nv_bfloat16, __half>::type;

  struct Barriers {
    uint64_t q_full;
    uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
    uint64_t s_full[TILES];   // S_t of the current step is complete
    uint64_t p_full[TILES];   // P_t is in tensor memory and O_t is rescaled (4 warps arrive)
    uint64_t pv_done[TILES];  // P_t V of the current step has retired
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
  };

  __device__ static __forceinline__ void report(Barriers* bars, uint32_t code, uint32_t d0, uint32_t d1) {
    bars->abort_flag = 1u;
    if (atomicCAS(&g_attn_status[0], 0u, code) == 0u) {
      g_attn_status[1] = blockIdx.x;
      g_attn_status[2] = d0;
      g_attn_status[3] = d1;
    }
  }

  __device__ static void run(const AttnParams& p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + RING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_groups = (p.sq + TILES * BR - 1) / (TILES * BR);
    const int head = static_cast<int>(blockIdx.x) / q_groups;
    const int q0 = (static_cast<int>(blockIdx.x) % q_groups) * (TILES * BR);
    const int nkv = (p.sk + BC - 1) / BC;

    if (threadIdx.x == 0) {
      tma_prefetch_desc(&p.tmQ);
      tma_prefetch_desc(&p.tmK);
      tma_prefetch_desc(&p.tmV);
      mbar_init(&bars->q_full, 1);
      for (int s = 0; s < K_STAGES; ++s) {
        mbar_init(&bars->k_full[s], 1);
        mbar_init(&bars->k_empty[s], 1);
      }
      for (int s = 0; s < V_STAGES; ++s) {
        mbar_init(&bars->v_full[s], 1);
        mbar_init(&bars->v_empty[s], 1);
      }
      for (int t = 0; t < TILES; ++t) {
        mbar_init(&bars->s_full[t], 1);
        mbar_init(&bars->p_full[t], 4);
        mbar_init(&bars->pv_done[t], 1);
      }
      bars->abort_flag = 0u;
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
      // ------------------------------------------------------------------ producer
      if (lane == 0) {
        mbar_expect_tx(&bars->q_full, TILES * Q_BYTES);
#pragma unroll
        for (int t = 0; t < TILES; ++t)
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            tma_load_3d(smem + t * Q_BYTES + b * QBOX_BYTES, &p.tmQ, &bars->q_full, b * 64, q0 + t * BR, head);
        for (int j = 0; j < nkv; ++j) {
          const int ks = j % K_STAGES, vs = j % V_STAGES;
          if (!mbar_wait(&bars->k_empty[ks], ((j / K_STAGES) & 1u) ^ 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_PRODUCER, j, 0u);
            break;
          }
          mbar_expect_tx(&bars->k_full[ks], KV_BYTES);
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            tma_load_3d(smem + OFF_K + ks * KV_BYTES + b * KVBOX_BYTES, &p.tmK, &bars->k_full[ks], b * 64, j * BC, head);
          if (!mbar_wait(&bars->v_empty[vs], ((j / V_STAGES) & 1u) ^ 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_PRODUCER, j, 1u);
            break;
          }
          mbar_expect_tx(&bars->v_full[vs], KV_BYTES);
#pragma unroll
          for (int b = 0; b < BOXES; ++b)
            tma_load_3d(smem + OFF_V + vs * KV_BYTES + b * KVBOX_BYTES, &p.tmV, &bars->v_full[vs], b * 64, j * BC, head);
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        bool ok = mbar_wait(&bars->q_full, 0u, &bars->abort_flag);
        if (!ok) report(bars, ATTN_TIMEOUT_MMA, 0u, 0u);
        tc_fence_after_sync();
        // S_t of step i. Issued after P_t V of step i - 1 (program order), which is what has read the P that
        // these scores overwrite; the softmax warps of tile t have read the old scores before they wrote that P.
        auto issue_s = [&](int t, int i) -> bool {
          const int s = i % K_STAGES;
          if (!mbar_wait(&bars->k_full[s], (i / K_STAGES) & 1u, &bars->abort_flag)) {
            report(bars, ATTN_TIMEOUT_MMA, 1u, static_cast<uint32_t>(i));
            return false;
          }
          tc_fence_after_sync();
          const uint32_t sq_addr = smem_u32(smem + t * Q_BYTES);
          const uint32_t sk_addr = smem_u32(smem + OFF_K + s * KV_BYTES);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks) {
            const uint32_t in_row = (ks * 32) % 128, box = (ks * 32) / 128;
            const uint64_t adesc = make_smem_desc(sq_addr + box * QBOX_BYTES + in_row, 16, 1024, SWZ_128B);
            const uint64_t bdesc = make_smem_desc(sk_addr + box * KVBOX_BYTES + in_row, 16, 1024, SWZ_128B);
            umma_ss<false>(tmem_base + t * BC, adesc, bdesc, IDESC_S, ks > 0 ? 1u : 0u);
          }
          if (t == TILES - 1) umma_commit(&bars->k_empty[s]);  // both tiles have read this K tile
          umma_commit(&bars->s_full[t]);
          return true;
        };
        for (int t = 0; t < TILES && ok; ++t) ok = issue_s(t, 0);
        for (int j = 0; j < nkv && ok; ++j) {
          const int vs = j % V_STAGES;
          for (int t = 0; t < TILES && ok; ++t) {
            if (!mbar_wait(&bars->p_full[t], j & 1u, &bars->abort_flag) ||
                !mbar_wait(&bars->v_full[vs], (j / V_STAGES) & 1u, &bars->abort_flag)) {
              report(bars, ATTN_TIMEOUT_MMA, 2u, static_cast<uint32_t>(j));
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t sv_addr = smem_u32(smem + OFF_V + vs * KV_BYTES);
#pragma unroll
            for (int ks = 0; ks < BC / 16; ++ks) {
              const uint64_t bdesc = make_smem_desc(sv_addr + ks * 16 * 128, KVBOX_BYTES, 1024, SWZ_128B);
              umma_ts_f16(tmem_base + COL_O + t * kD, tmem_base + t * BC + ks * 8, bdesc, IDESC_O,
                          (j > 0 || ks > 0) ? 1u : 0u);
            }
            if (t == TILES - 1) umma_commit(&bars->v_empty[vs]);
            umma_commit(&bars->pv_done[t]);
            if (j + 1 < nkv) ok = issue_s(t, j + 1);
          }
        }
      }
    } else {
      // ------------------------------------------------- softmax, correction, epilogue
      const int q = warp & 3;           // TMEM lane quarter this warp may access
      const int t = (warp - 2) >> 2;    // query tile of this warp
      const int row = q * 32 + lane;    // query row of this thread inside its tile
      const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
      const uint32_t col_s = tmem_base + lane_addr + t * BC, col_o = tmem_base + lane_addr + COL_O + t * kD;
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < nkv; ++j) {
        bool got = mbar_wait(&bars->s_full[t], j & 1u, &bars->abort_flag);
        if (!named_bar_all(2 + t, 128, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 0u, static_cast<uint32_t>(j));
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // all four 32-column reads of the row in flight, one wait
        uint32_t sr[BC / 32][32];
#pragma unroll
        for (int c = 0; c < BC / 32; ++c) tmem_ld_32x32b_x32(col_s + c * 32, sr[c]);
        tmem_ld_wait();
        float s[BC];
#pragma unroll
        for (int c = 0; c < BC / 32; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(sr[c][i]);
        const int valid = p.sk - j * BC;
        if (valid < BC) {
#pragma unroll
          for (int i = 0; i < BC; ++i)
            if (i >= valid) s[i] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < BC; i += 4) {
          mx4[0] = fmaxf(mx4[0], s[i]);
          mx4[1] = fmaxf(mx4[1], s[i + 1]);
          mx4[2] = fmaxf(mx4[2], s[i + 2]);
          mx4[3] = fmaxf(mx4[3], s[i + 3]);
        }
        const float mx = fmaxf(m, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2);
        const float alpha = ex2(m - mx);  // 0 on the first step (m = -inf)
        const bool rescale = j > 0 && __any_sync(0xffffffffu, alpha != 1.f);
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        // exponentials and P, 64 keys at a time: packed pairs over the S columns this thread has read
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float e0 = ex2(fmaf(s[half * 64 + 2 * i], p.scale_log2, -mx));
            const float e1 = ex2(fmaf(s[half * 64 + 2 * i + 1], p.scale_log2, -mx));
            sum4[i & 3] += e0 + e1;
            if constexpr (kBf16) {
              __nv_bfloat162 v2 = __floats2bfloat162_rn(e0, e1);
              w[i] = *reinterpret_cast<uint32_t*>(&v2);
            } else {
              __half2 v2 = __floats2half2_rn(e0, e1);
              w[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
          }
          tmem_st_32x32b_x32(col_s + half * 32, w);
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m = mx;
        if (rescale) {
          // O_t <- alpha * O_t for this row: the previous P_t V has retired (the scores of this step were issued
          // behind it), which the barrier confirms
          got = mbar_wait(&bars->pv_done[t], (j & 1u) ^ 1u, &bars->abort_flag);
          if (got) {
            tc_fence_after_sync();
            uint32_t orr[kD / 32][32];
#pragma unroll
            for (int c = 0; c < kD / 32; ++c) tmem_ld_32x32b_x32(col_o + c * 32, orr[c]);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < kD / 32; ++c) {
#pragma unroll
              for (int i = 0; i < 32; ++i) orr[c][i] = __float_as_uint(__uint_as_float(orr[c][i]) * alpha);
              tmem_st_32x32b_x32(col_o + c * 32, orr[c]);
            }
          }
        }
        tmem_st_wait();
        if (!named_bar_all(2 + t, 128, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 1u, static_cast<uint32_t>(j));
          ok = false;
          break;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[t]);
      }
      if (ok) {
        bool got = mbar_wait(&bars->pv_done[t], (nkv - 1) & 1u, &bars->abort_flag);
        if (!named_bar_all(2 + t, 128, got)) {
          if (!got) report(bars, ATTN_TIMEOUT_SOFTMAX, 2u, 0u);
          ok = false;
        }
      }
      if (ok) {
        tc_fence_after_sync();
        const float inv = 1.f / l;
        const int grow = q0 + t * BR + row;
        T* out = reinterpret_cast<T*>(p.O) + (static_cast<size_t>(head) * p.sq + grow) * kD;
#pragma unroll
        for (int c = 0; c < kD / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(col_o + c * 32, r);
          tmem_ld_wait();
          if (grow < p.sq) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float a = __uint_as_float(r[u * 8 + 2 * e]) * inv, bb = __uint_as_float(r[u * 8 + 2 * e + 1]) * inv;
                if constexpr (kBf16) {
                  __nv_bfloat162 v2 = __floats2bfloat162_rn(a, bb);
                  w[e] = *reinterpret_cast<uint32_t*>(&v2);
                } else {
                  __half2 v2 = __floats2half2_rn(a, bb);
                  w[e] = *reinterpret_cast<uint32_t*>(&v2);
                }
              }
              *reinterpret_cast<uint4*>(out + c * 32 + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    if (bars->abort_flag != 0u) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
};

template <int kD, bool kBf16>
__global__ void __launch_bounds__(320, 1) kcg_attention2_kernel(const __grid_constant__ AttnParams p) {
  AttnFwd2<kD, kBf16>::run(p);
}

template <int kD, bool kBf16, int kBC, int kSplit, int kPTmem>
__global__ void __launch_bounds__(64 + 128 * kSplit, (kBC == 64 && kSplit == 1) ? 2 : 1)
kcg_attention_kernel(const __grid_constant__ AttnParams p) {
  AttnFwd<kD, kBf16, kBC, kSplit, kPTmem>::run(p);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
bool g_ready[16][20];  // [device][kernel instance]: dynamic shared memory opted in
std::mutex g_mutex;

int fail(int code, const std::string& msg) { return kcg_internal_fail(code, msg.c_str()); }
int cuda_fail(cudaError_t e, const char* what) {
  return fail(static_cast<int>(e), std::string(what) + ": " + cudaGetErrorString(e));
}

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

// {d, rows, heads} view of a contiguous heads x rows x d tensor; boxes of 64 values x `box_rows` rows of one
// head. Rows past the end of a head read as zero.
int encode3(CUtensorMap* tm, bool bf16, uint64_t ptr, int d, int rows, int heads, int box_rows) {
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads)};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(d) * 2 * static_cast<cuuint64_t>(rows)};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = g_encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                              reinterpret_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(static_cast<int>(r), "cuTensorMapEncodeTiled failed");
  return 0;
}

struct Problem {
  uint64_t Q, K, V, O;
  int heads, sq, sk, d;
  float scale;
  bool bf16;
};

template <int kD, bool kBf16, int kBC, int kSplit, int kPTmem>
int launch(int device, int slot, cudaStream_t st, const Problem& pb) {
  using Kern = AttnFwd<kD, kBf16, kBC, kSplit, kPTmem>;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_ready[device][slot]) {
      const cudaError_t e = cudaFuncSetAttribute(kcg_attention_kernel<kD, kBf16, kBC, kSplit, kPTmem>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Kern::SMEM_BYTES);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
      g_ready[device][slot] = true;
    }
  }
  AttnParams p{};
  if (int r = encode3(&p.tmQ, kBf16, pb.Q, kD, pb.sq, pb.heads, 128)) return r;
  if (int r = encode3(&p.tmK, kBf16, pb.K, kD, pb.sk, pb.heads, kBC)) return r;
  if (int r = encode3(&p.tmV, kBf16, pb.V, kD, pb.sk, pb.heads, kBC)) return r;
  p.O = reinterpret_cast<void*>(pb.O);
  p.sq = pb.sq;
  p.sk = pb.sk;
  p.scale_log2 = pb.scale * 1.4426950408889634f;
  const int grid = pb.heads * ((pb.sq + 127) / 128);
  kcg_attention_kernel<kD, kBf16, kBC, kSplit, kPTmem><<<grid, Kern::NUM_THREADS, Kern::SMEM_BYTES, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attention launch");
  kcg_internal_count_launch();
  return 0;
}

template <int kD, bool kBf16>
int launch2(int device, int slot, cudaStream_t st, const Problem& pb) {
  using Kern = AttnFwd2<kD, kBf16>;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_ready[device][slot]) {
      const cudaError_t e = cudaFuncSetAttribute(kcg_attention2_kernel<kD, kBf16>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Kern::SMEM_BYTES);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
      g_ready[device][slot] = true;
    }
  }
  AttnParams p{};
  if (int r = encode3(&p.tmQ, kBf16, pb.Q, kD, pb.sq, pb.heads, 128)) return r;
  if (int r = encode3(&p.tmK, kBf16, pb.K, kD, pb.sk, pb.heads, 128)) return r;
  if (int r = encode3(&p.tmV, kBf16, pb.V, kD, pb.sk, pb.heads, 128)) return r;
  p.O = reinterpret_cast<void*>(pb.O);
  p.sq = pb.sq;
  p.sk = pb.sk;
  p.scale_log2 = pb.scale * 1.4426950408889634f;
  const int grid = pb.heads * ((pb.sq + 255) / 256);
  kcg_attention2_kernel<kD, kBf16><<<grid, Kern::NUM_THREADS, Kern::SMEM_BYTES, st>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attention launch");
  kcg_internal_count_launch();
  return 0;
}

template <int kBC, int kSplit, int kPTmem>
int launch_shape(int device, int base_slot, cudaStream_t st, const Problem& pb) {
  if (pb.d == 128)
    return pb.bf16 ? launch<128, true, kBC, kSplit, kPTmem>(device, base_slot, st, pb)
                   : launch<128, false, kBC, kSplit, kPTmem>(device, base_slot + 1, st, pb);
  return pb.bf16 ? launch<64, true, kBC, kSplit, kPTmem>(device, base_slot + 2, st, pb)
                 : launch<64, false, kBC, kSplit, kPTmem>(device, base_slot + 3, st, pb);
}

}  // namespace

extern "C" int kcg_attention_fwd(int device, uint64_t stream, uint64_t Q, uint64_t K, uint64_t V, uint64_t O, int dtype,
                                 int heads, int sq, int sk, int d, float scale) {
  if (!Q || !K || !V || !O) return fail(KCG_E_BAD_ARG, "null device pointer");
  if (heads <= 0 || sq <= 0 || sk <= 0) return fail(KCG_E_BAD_ARG, "empty shape");
  if (!(dtype == KCG_DTYPE_BFLOAT16 || dtype == KCG_DTYPE_FLOAT16))
    return fail(KCG_E_BAD_ARG, "the fused attention kernel takes float16 or bfloat16 data");
  if (!(d == 64 || d == 128)) return fail(KCG_E_BAD_CONFIG, "head dimension must be 64 or 128");
  if (!(scale > 0.f) || !std::isfinite(scale)) return fail(KCG_E_BAD_ARG, "scale must be positive and finite");
  if (device < 0 || device >= 16) return fail(KCG_E_BAD_ARG, "device index out of range");
  if (Q % 16 || K % 16 || V % 16 || O % 16) return fail(KCG_E_BAD_ARG, "operands must start on 16-byte boundaries");
  const long long tiles = static_cast<long long>(heads) * ((sq + 127) / 128);
  if (tiles > 0x7fffffffLL) return fail(KCG_E_TOO_LARGE, "too many query tiles for one launch");
  DeviceGuard guard;
  cudaError_t e = guard.enter(device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
        return fail(KCG_E_NO_DRIVER, "cuTensorMapEncodeTiled not available from the driver");
      g_encode = reinterpret_cast<EncodeFn>(fn);
    }
  }
  Problem pb{Q, K, V, O, heads, sq, sk, d, scale, dtype == KCG_DTYPE_BFLOAT16};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Default: two query tiles per CTA that alternate on the tensor pipe (AttnFwd2; the fastest form measured).
  // KCG_ATTN_FORM selects a comparison form with ONE query tile per CTA: 4 = 128-key steps, two threads per row,
  // P in tensor memory; 5 = 64-key steps, one thread per row, two CTAs per SM; 6 and 7 = the same two with P
  // through shared memory.
  static const int form = [] {
    const char* v = getenv("KCG_ATTN_FORM");
    return v ? atoi(v) & 7 : 0;
  }();
  switch (form) {
    case 4: return launch_shape<128, 2, 1>(device, 0, st, pb);
    case 5: return launch_shape<64, 1, 1>(device, 4, st, pb);
    case 6: return launch_shape<128, 2, 0>(device, 8, st, pb);
    case 7: return launch_shape<64, 1, 0>(device, 12, st, pb);
    default:
      if (pb.d == 128) return pb.bf16 ? launch2<128, true>(device, 16, st, pb) : launch2<128, false>(device, 17, st, pb);
      return pb.bf16 ? launch2<64, true>(device, 18, st, pb) : launch2<64, false>(device, 19, st, pb);
  }
}

// Reads (and clears) the status word of the fused attention kernels on `device`: out = {code, block, detail,
// detail}; code 0 = no bounded wait has run out since the last call. Synchronises the device.
extern "C" int kcg_attention_status(int device, uint32_t out[4]) {
  if (!out) return fail(KCG_E_BAD_ARG, "null argument");
  DeviceGuard guard;
  cudaError_t e = guard.enter(device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  e = cudaMemcpyFromSymbol(out, g_attn_status, sizeof(uint32_t) * 4);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol");
  if (out[0] != 0u) {
    const uint32_t zero[4] = {0u, 0u, 0u, 0u};
    e = cudaMemcpyToSymbol(g_attn_status, zero, sizeof(zero));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol");
    return fail(KCG_E_DEVICE_TIMEOUT, "a bounded wait of the attention kernel ran out");
  }
  return 0;
}
