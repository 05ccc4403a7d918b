/* C ABI of libkcg_b200.so: compile, load and launch the B200 (sm_100a) GEMM
 * kernels behind the operator API of Xiebaokang/CodeGenDemo ("KCG").
 *
 * Every function returns 0 on success. A positive value is a CUresult from the
 * CUDA driver, a negative value one of the KCG_E_* codes below; in both cases
 * kcg_last_error() returns a thread-local message that starts with
 * "KCG Error[CUDA]: Code: <n>, Messsage: " — the prefix (typo included) of the
 * reference's loader errors (Runtime/python/kcg/loaderCCode/hip.c:8-21).
 *
 * The library links nothing from the CUDA driver at load time: libcuda.so.1 is
 * opened on the first call that needs a GPU, so the library loads (and the
 * compile entry works) on a machine without one. There is no CPU fallback: a
 * load/launch call without a usable driver fails with KCG_E_NO_DRIVER.
 */
#ifndef KCG_B200_H_
#define KCG_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KCG_NUM_CFG_KEYS 31

/* Positional order of the 31 tuning-config integers. It is the argument order of
 * the reference's compile_kernel_matmul (src/main.cc:64-102, mirrored by
 * Runtime/python/kcg/KCGCompiler.py:14-44). */
enum kcg_cfg_index {
  KCG_CFG_BLOCK_SIZE_M = 0, KCG_CFG_BLOCK_SIZE_N, KCG_CFG_BLOCK_SIZE_K,
  KCG_CFG_THREAD_SIZE_M, KCG_CFG_THREAD_SIZE_N, KCG_CFG_WARP_SIZE,
  KCG_CFG_BLOCK_LAYOUT_M, KCG_CFG_BLOCK_LAYOUT_N, KCG_CFG_WARP_LAYOUT_M, KCG_CFG_WARP_LAYOUT_N,
  KCG_CFG_GLOB_LOAD_WIDTH_A, KCG_CFG_GLOB_LOAD_WIDTH_B,
  KCG_CFG_WARP_SCATTER_WIDTH_A, KCG_CFG_WARP_SCATTER_WIDTH_B,
  KCG_CFG_THREAD_SCATTER_WIDTH_A, KCG_CFG_THREAD_SCATTER_WIDTH_B,
  KCG_CFG_LOCAL_SPLIT_U, KCG_CFG_BLOCK_MAPPING, KCG_CFG_GLOB_STORE_WIDTH,
  KCG_CFG_UNROLL_NUM, KCG_CFG_REG_PREFETCH, KCG_CFG_SHARED_PREFETCH,
  KCG_CFG_LOAD_CONTINUOUS, KCG_CFG_REDUCE_C_CONTINUOUS,
  KCG_CFG_DATATYPE_A, KCG_CFG_DATATYPE_B, KCG_CFG_DATATYPE_C,
  KCG_CFG_M_SIZE, KCG_CFG_N_SIZE, KCG_CFG_K_SIZE, KCG_CFG_IS_ATRANS
};

/* DATATYPE_* values: 2 / 4 are the reference's float16 / float32 codes
 * (Runtime/python/kcg/Utils.py:198-203); 62 is bfloat16 (new; 62 % 30 == 2 bytes). */
#define KCG_DTYPE_FLOAT16 2
#define KCG_DTYPE_FLOAT32 4
#define KCG_DTYPE_BFLOAT16 62

/* Kernel families. AUTO picks TCGEN05 when the tile shape is one the tensor-core
 * kernel can build and SIMT otherwise. */
#define KCG_KERNEL_AUTO 0
#define KCG_KERNEL_SIMT 1     /* FFMA register-tiled kernel */
#define KCG_KERNEL_TCGEN05 2  /* TMA + tcgen05/TMEM; fp32 runs as 3xTF32 */
#define KCG_KERNEL_TF32X1 3   /* fp32 in one TF32 pass (reduced accuracy, comparison only) */
#define KCG_KERNEL_TCGEN05_PAIR 4 /* fp16/bf16 on CTA pairs (tcgen05 cta_group::2), BLOCK_SIZE_M = 256 */
#define KCG_KERNEL_TCGEN05_CLUSTERK 5 /* fp16/bf16 128-row tiles; LOCAL_SPLIT_U (2..4) CTAs of a thread-block
                                         cluster split K and reduce through distributed shared memory */
#define KCG_KERNEL_NAIVE 100  /* one thread per C element, on-device reference */
#define KCG_KERNEL_WAIT_PROBE 101 /* no GEMM: one bounded wait (20 ms) that expires -> KCG_E_DEVICE_TIMEOUT */

/* Error codes (negative; positive values are CUresult). */
#define KCG_E_BAD_CONFIG (-1)      /* config fails the reference's check() rules or the kernel's */
#define KCG_E_COMPILE (-2)         /* nvcc failed; message carries the tail of its log */
#define KCG_E_NO_DRIVER (-3)       /* libcuda.so.1 / a GPU is not available */
#define KCG_E_IO (-4)              /* cubin / cache file could not be read or written */
#define KCG_E_DEVICE_TIMEOUT (-5)  /* a bounded wait inside the kernel ran out (status word) */
#define KCG_E_BAD_ARG (-6)
#define KCG_E_TOO_LARGE (-7)

typedef struct kcg_kernel_info {
  char path[1024];    /* cubin on disk (reference: hsaco path, src/main.cc:343-353) */
  char name[512];     /* kernel symbol, same naming scheme as src/main.cc:119-145 */
  int32_t grid[3];    /* launch dims (reference: func.grid.dim / func.block.dim attrs) */
  int32_t block[3];
  int32_t cluster[3];
  int32_t smem_bytes; /* dynamic shared memory the launch must request */
  int32_t kernel;     /* resolved KCG_KERNEL_* */
  int32_t dtype;      /* DATATYPE_A */
  int32_t bm, bn, bk; /* CTA tile */
  int32_t stages;     /* shared-memory pipeline depth (tcgen05) */
  int32_t splitk;     /* LOCAL_SPLIT_U */
  int32_t group;      /* BLOCK_MAPPING */
  int32_t atrans;     /* IS_ATRANS */
  int32_t m, n, k;
  int32_t reserved[8]; /* [0] persistent grid cap (SMs), [1] b_trans, [2] serpentine,
                          [3] DATATYPE_C when it differs from DATATYPE_A (float32 C over 16-bit operands),
                          [4] accumulator buffers in tensor memory (single-pass tcgen05 kernels: 1 or 2) */
} kcg_kernel_info;

typedef struct kcg_compile_opts {
  int32_t kernel;      /* KCG_KERNEL_*; 0 = auto */
  int32_t num_stages;  /* 0 = derive from SHARED_PREFETCH (0 -> 2 stages, 1 -> as many as fit, max 6) */
  int32_t num_sms;     /* persistent grid size cap; 0 = 148 (B200) */
  int32_t force;       /* 1 = recompile even when the cubin is cached */
  int32_t b_trans;     /* 1 = B is stored N x K row-major (C = A * Bt^T); fp16 / bf16 with KCG_KERNEL_TCGEN05 / _PAIR.
                          The reference stores B as K x N only (src/lib/Operators/Matmul.cc:93-121). */
  int32_t serpentine;  /* 1 = inside a BLOCK_MAPPING group, odd tile columns walk the rows upwards (the reference's
                          serpentine twin, matmul.cpp:1279-1287); tcgen05 kernels, BLOCK_MAPPING >= 2 */
  int32_t reserved[2];
} kcg_compile_opts;

typedef struct kcg_device_props {
  int32_t max_shared_mem;        /* opt-in maximum per block, bytes */
  int32_t multiprocessor_count;
  int32_t sm_clock_rate;         /* kHz */
  int32_t mem_clock_rate;        /* kHz */
  int32_t mem_bus_width;         /* bits */
  int32_t l2_cache_bytes;
  int32_t cc_major, cc_minor;
} kcg_device_props;

/* ---- compile boundary ---------------------------------------------------------
 * Replaces compile_kernel_matmul (src/main.cc:315-357): validates the 31-key config
 * (same rules as KernelArgMatmul.check, Runtime/python/kcg/Operators/matmul.py:180-194),
 * names the kernel, runs `nvcc -cubin -gencode arch=compute_100a,code=sm_100a` on the
 * kernel template with the config as macros (or reuses the cached cubin of that
 * name) and reports path, name and launch dims. Needs no GPU. Reentrant. */
int kcg_compile_matmul(const int32_t cfg[KCG_NUM_CFG_KEYS], kcg_kernel_info* out);
int kcg_compile_matmul_ex(const int32_t cfg[KCG_NUM_CFG_KEYS], const kcg_compile_opts* opts,
                          kcg_kernel_info* out);
/* Writes the kernel symbol the config compiles to (no compilation). */
int kcg_kernel_name(const int32_t cfg[KCG_NUM_CFG_KEYS], const kcg_compile_opts* opts, char* buf,
                    int buf_len);
/* Directory cubins are cached in ($KCG_CACHE_DIR, else <library dir>/_cache). */
const char* kcg_cache_dir(void);

/* ---- load boundary --------------------------------------------------------------
 * Replaces load_binary / get_device_properties of the reference's loader extension
 * (Runtime/python/kcg/loaderCCode/hip.c:60-133 and :44-58). `shared` above 48 KiB
 * opts the function in to that much dynamic shared memory. */
int kcg_load_binary(const char* name, const char* path, int shared, int device, uint64_t* module,
                    uint64_t* function, int* n_regs, int* n_spills);
int kcg_unload(uint64_t module);
int kcg_device_properties(int device, kcg_device_props* out);

/* ---- launch boundary ------------------------------------------------------------
 * Replaces the generated launcher's launch() (Runtime/python/kcg/HIPLauncher.py:189-238):
 * asynchronous on `stream` (a CUstream as integer; 0 = default stream), pointers are
 * device addresses borrowed for the call. Tensor maps for TMA are built (and cached per
 * pointer/shape) inside. Split-K kernels use a per-device workspace the library
 * allocates on first use. C is overwritten (alpha = 1, beta = 0). */
int kcg_launch_gemm(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                    uint64_t A, uint64_t B, uint64_t C);
/* Fused epilogue: C = act(alpha * (A*B) + beta * C + bias[col]), fp32 arithmetic in that order,
 * rounded once to C's type. No counterpart in the reference's launcher (its kernels store A*B
 * only); it covers the bias / ReLU step the reference plans between chained matmuls
 * (doc/重构方案.md). beta * C reads C in place and is skipped when beta == 0 (C may then be
 * uninitialised); `bias` is a device address of N values of C's type, 16-byte aligned, or 0;
 * relu != 0 applies max(x, 0) last. A null `epi` is kcg_launch_gemm. Every kernel family
 * honours it, including the K-split kernels (the reducing CTA applies it once). */
typedef struct kcg_epilogue {
  float alpha;
  float beta;
  uint64_t bias;
  int32_t relu;
  int32_t reserved[3];
} kcg_epilogue;
int kcg_launch_gemm_ex(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                       uint64_t A, uint64_t B, uint64_t C, const kcg_epilogue* epi);
/* ---- batched product ---------------------------------------------------------------
 * C[b] = A[b] * B[b] for b in [0, batch), every operand contiguous over the batches (torch.bmm
 * layout: A is batch x M x K - or batch x K x M with IS_ATRANS - B is batch x K x N, C is batch x M
 * x N), with the cubin compiled for ONE batch's M, N, K. No counterpart in the reference (batched
 * GEMM is on its list of next operators, doc/结果汇总.md). One launch: the persistent kernel
 * walks the tiles of all batches as one tall problem, so small per-batch problems fill the
 * GPU together; tcgen05 kernels only (KERNEL_VARIANT 2, 3, 4). `epi` may be null; a bias is
 * shared by all batches. */
int kcg_launch_gemm_batched(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                            uint64_t A, uint64_t B, uint64_t C, int batch, const kcg_epilogue* epi);

/* ---- strided operands --------------------------------------------------------------
 * kcg_launch_gemm / _ex / _batched with leading dimensions: lda, ldb, ldc are the distances, in
 * elements, between consecutive rows of A, B and C as they are stored (A: M x K, or K x M with
 * IS_ATRANS; B: K x N, or N x K when compiled with b_trans; C: M x N). 0 means contiguous (the row
 * length); a larger value addresses a sub-matrix of a wider row-major array, e.g. a column block of
 * a weight matrix or a head slice of a packed activation. Each must keep rows 16-byte aligned
 * (TMA pitch rule). With batch > 1 the batches follow one another row after row at the same pitch.
 * No counterpart in the reference: its kernels take the row length as the pitch
 * (src/lib/Operators/Matmul.cc:93-121); strided GEMM is on its list of next operators
 * (doc/结果汇总.md). */
int kcg_launch_gemm_strided(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                            uint64_t A, uint64_t B, uint64_t C, int64_t lda, int64_t ldb, int64_t ldc, int batch,
                            const kcg_epilogue* epi);

/* ---- row softmax (middle step of the attention-shaped chain) ---------------------------
 * In place: X[r, :] = softmax(scale * X[r, :]) for r in [0, rows), fp32 arithmetic; X is a
 * row-major matrix of `dtype` (KCG_DTYPE_*) values with `ld` elements between rows (0 = cols).
 * With it, softmax(scale * Q K^T) V runs as three launches on one stream: a batched GEMM compiled
 * with b_trans (S = Q K^T, K stored keys x head_dim), this call, and a batched GEMM (P V). The
 * reference has no such operator yet; it lists the flash-attention-shaped chain after batched
 * GEMM among its next operators (doc/结果汇总.md). Rows must start and end on 16-byte boundaries. */
int kcg_softmax_rows(int device, uint64_t stream, uint64_t X, int64_t rows, int cols, int64_t ld, float scale,
                     int dtype);
/* The same from X into another matrix Y, each with its own type and pitch: fp32 scores in, fp16 / bf16
 * probabilities out (a GEMM compiled with DATATYPE_C = float32 over 16-bit operands writes such scores).
 * cols must be a multiple of 8. Y == X is the in-place call above. */
int kcg_softmax_rows_ex(int device, uint64_t stream, uint64_t X, int dtype_in, int64_t ldx, uint64_t Y,
                        int dtype_out, int64_t ldy, int64_t rows, int cols, float scale);

/* ---- the same chain as ONE kernel ------------------------------------------------------
 * O[h] = softmax(scale * Q[h] K[h]^T) V[h] for h in [0, heads): Q and O are heads x sq x d, K and V
 * heads x sk x d, all contiguous, float16 or bfloat16 (`dtype`), d = 64 or 128. Scores and
 * probabilities stay in tensor memory and shared memory (tcgen05.mma for both products, running
 * maximum and sum per query row); nothing of size sq x sk is written. Asynchronous on `stream`;
 * allocates nothing. `scale` must be positive. The first call per device and data type opts the kernel in
 * to its dynamic shared memory (a function attribute): make it before capturing the stream into a graph.
 * No counterpart in the reference (see the note on kcg_softmax_rows). */
int kcg_attention_fwd(int device, uint64_t stream, uint64_t Q, uint64_t K, uint64_t V, uint64_t O, int dtype,
                      int heads, int sq, int sk, int d, float scale);
/* Synchronises `device` and reads (and clears) the status word of the kernel above: out = {code, block,
 * detail, detail}. Returns KCG_E_DEVICE_TIMEOUT when a bounded wait ran out since the last call, else 0. */
int kcg_attention_status(int device, uint32_t out[4]);

/* ---- M-sharded product with the all-gather of C fused into the kernel ---------------
 * No counterpart in the reference (it has no multi-GPU code). Rank r of G computes rows
 * [r*M/G, (r+1)*M/G) of C with the same cubin as kcg_launch_gemm; `C` is the address of that slab
 * inside this GPU's full C, and peer_c[i] the address of the same slab inside the full C of
 * another GPU, mapped into this process (kcg_peer_open). Every finished tile is written to
 * all of them inside the kernel: the epilogue stores it into this GPU's C and two push warps of
 * the same CTA copy it from there (L2) to the peers with coalesced 16-byte stores over NVLink
 * while later tiles multiply (the reducer of a K-split tile writes the peers itself); no remote
 * loads, no flags or waits between GPUs; the full C is complete on a GPU once the kernels of all
 * ranks have completed (synchronise the streams, then barrier). 16-bit single-pass tcgen05
 * kernels only (KCG_KERNEL_TCGEN05 / _PAIR with fp16 / bf16 data); n_peers = 0 is
 * kcg_launch_gemm_ex. KCG_MAX_PEERS = 7. */
int kcg_launch_gemm_allgather(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                              uint64_t A, uint64_t B, uint64_t C, const kcg_epilogue* epi,
                              const uint64_t* peer_c, int n_peers);
/* Device memory that other processes of the node can map: alloc + 64-byte CUDA IPC handle on
 * the owner, open / close on the others, free on the owner after every peer closed it. */
int kcg_peer_alloc(int device, uint64_t bytes, uint64_t* dptr, uint8_t handle[64]);
int kcg_peer_open(int device, const uint8_t handle[64], uint64_t* dptr);
int kcg_peer_close(int device, uint64_t dptr);
int kcg_peer_free(int device, uint64_t dptr);

/* Reads (and clears) the device status word written by bounded waits; returns
 * KCG_E_DEVICE_TIMEOUT if a kernel gave up since the last check. Synchronises `stream`. */
int kcg_check_status(int device, uint64_t stream);

/* Whole-operator call on HOST buffers: copies A and B to the device (async from the
 * caller's memory, pinned for full speed), runs the kernel and copies C back, ordered
 * after the work already queued on `stream`, then synchronises. Large problems move as
 * up to sixteen row slabs through three internal streams (copy-in, compute, copy-out) so
 * that both transfer directions and the kernels overlap. Device buffers are owned and
 * reused by the library. */
int kcg_matmul_host(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                    const void* hostA, const void* hostB, void* hostC);

/* ---- allocation-free split-K GEMM -------------------------------------------------
 * No counterpart in the reference (its launcher never allocates because its kernels need no
 * workspace). For callers that must not allocate device memory at the point of the GEMM - code
 * running inside a fixed memory pool, a serving loop with a frozen memory budget, a process whose
 * free HBM belongs to another allocator - where the workspace kcg_launch_gemm allocates on first
 * use would fail, stall or synchronise the device. bf16 C = A*B (A is M x K, B is K x N, row-major),
 * K split KCG_NOALLOC_SPLITK ways, tile 128x256x64; same kernel code as the compiled path.
 *
 * The split-K workspace is a fixed array inside the library's device image (about 32 MiB per GPU
 * that loads the library, held until the process exits). Limits: M, N, K multiples of 128, 256, 64;
 * K >= 64*KCG_NOALLOC_SPLITK; KCG_NOALLOC_SPLITK*M*N <= KCG_NOALLOC_MAX_PARTIAL_FLOATS, else
 * KCG_E_TOO_LARGE. That bound on the partial tiles is the one that binds: it allows M*N up to 2 Mi
 * elements, i.e. at most KCG_NOALLOC_MAX_TILES = 64 tiles of 128x256, which is also the number of
 * arrival counters in the array. The call itself calls no cudaMalloc/cudaFree or allocating
 * library routine. The first call on a device resolves the array's device address and raises the
 * kernel's shared-memory limit; under CUDA's default lazy module loading that first call is also
 * what loads the library's device image - the 32 MiB array included - onto the GPU, an implicit
 * device allocation made by the CUDA runtime that can fail when the GPU is already full. So make
 * the first call per device at start-up, while memory is still free and before any stream
 * capture begins; later calls leave the GPU's free memory untouched. The call makes `device`
 * current while it runs and puts the caller's current device back before it returns. All calls on
 * a device share the one array: two calls that overlap on the GPU (different streams, no
 * ordering) race on it and give wrong results; calls ordered on one stream are safe.
 * `synchronize` != 0 waits for the stream and reports a kernel that gave up in a bounded wait as
 * KCG_E_DEVICE_TIMEOUT (and clears the record). With 0 the call is asynchronous and such a record
 * is kept in the array until the next call with `synchronize` != 0 on that device reports it:
 * kcg_check_status does not see it. */
#define KCG_NOALLOC_SPLITK 4
#define KCG_NOALLOC_MAX_PARTIAL_FLOATS (8 * 1024 * 1024)
#define KCG_NOALLOC_MAX_TILES 64
int kcg_gemm_bf16_splitk_noalloc(int device, uint64_t stream, uint64_t A, uint64_t B, uint64_t C, int M, int N,
                                 int K, int synchronize);

/* Number of kernel launches issued through this library since load (all threads). */
uint64_t kcg_launch_count(void);
/* Frees workspaces, device buffers and cached tensor maps of every device. */
int kcg_shutdown(void);
const char* kcg_last_error(void);
const char* kcg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KCG_B200_H_ */
