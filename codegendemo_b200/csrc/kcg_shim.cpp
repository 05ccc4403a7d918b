// Host side of libkcg_b200.so: the C ABI declared in include/kcg_b200.h.
//
//   compile : tuning config -> kernel name -> `nvcc -cubin` of kernels/gemm_entry.cu
//             with the config as macros -> cubin in the cache directory
//   load    : cubin -> CUmodule / CUfunction through the CUDA driver API
//   launch  : tensor maps (cuTensorMapEncodeTiled) + one `__grid_constant__`
//             parameter block -> cuLaunchKernelEx on the caller's stream
//
// libcuda.so.1 is resolved with dlopen on first use, so this library loads on a
// machine without a GPU (the compile entry needs none). Nothing here computes a
// GEMM on the host: without a driver, load/launch fail with KCG_E_NO_DRIVER.
#include <cuda.h>
#include <dirent.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <spawn.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/kcg_b200.h"
#include "kernels/gemm_params.h"

extern char** environ;

namespace {

// --------------------------------------------------------------------- errors
thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[4096];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = "KCG Error[CUDA]: Code: " + std::to_string(code) + ", Messsage: " + buf;
  return code;
}

// --------------------------------------------------------- driver API binding
#define KCG_STR2(x) #x
#define KCG_STR(x) KCG_STR2(x)
#define KCG_DRV_FUNCS(X)                                                                       \
  X(cuInit) X(cuDeviceGet) X(cuDeviceGetCount) X(cuDeviceGetAttribute) X(cuGetErrorString)     \
  X(cuDevicePrimaryCtxRetain) X(cuCtxGetCurrent) X(cuCtxSetCurrent) X(cuModuleLoadData)        \
  X(cuModuleGetFunction) X(cuModuleUnload) X(cuFuncSetAttribute) X(cuFuncGetAttribute)         \
  X(cuLaunchKernelEx) X(cuTensorMapEncodeTiled) X(cuMemAlloc) X(cuMemFree) X(cuMemsetD32)      \
  X(cuMemcpyHtoDAsync) X(cuMemcpyDtoHAsync) X(cuMemcpyDtoH) X(cuMemcpyHtoD)                    \
  X(cuStreamSynchronize) X(cuStreamCreate) X(cuStreamDestroy) X(cuStreamWaitEvent) X(cuEventCreate)        \
  X(cuEventRecord) X(cuEventDestroy) X(cuIpcGetMemHandle) X(cuIpcOpenMemHandle) X(cuIpcCloseMemHandle)

struct Driver {
  void* handle = nullptr;
  bool ok = false;
  std::string why;
#define X(f) decltype(&f) p_##f = nullptr;
  KCG_DRV_FUNCS(X)
#undef X
};

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.handle = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!d.handle) {
      d.why = std::string("cannot open libcuda.so.1: ") + dlerror();
      return;
    }
    bool all = true;
#define X(f)                                                                  \
  d.p_##f = reinterpret_cast<decltype(&f)>(dlsym(d.handle, KCG_STR(f)));      \
  if (!d.p_##f) {                                                             \
    all = false;                                                              \
    d.why += std::string("missing driver symbol ") + KCG_STR(f) + "; ";       \
  }
    KCG_DRV_FUNCS(X)
#undef X
    if (!all) return;
    CUresult r = d.p_cuInit(0);
    if (r != CUDA_SUCCESS) {
      d.why = "cuInit failed with CUresult " + std::to_string(static_cast<int>(r));
      return;
    }
    d.ok = true;
  });
  return d;
}

int drv_fail(CUresult r, const char* what) {
  const char* s = nullptr;
  Driver& d = driver();
  if (d.p_cuGetErrorString) d.p_cuGetErrorString(r, &s);
  return fail(static_cast<int>(r), "%s: %s", what, s ? s : "unknown CUDA error");
}

#define DRV(call)                                             \
  do {                                                        \
    CUresult _r = driver().p_##call;                          \
    if (_r != CUDA_SUCCESS) return drv_fail(_r, #call);       \
  } while (0)

int need_driver() {
  Driver& d = driver();
  if (!d.ok) return fail(KCG_E_NO_DRIVER, "CUDA driver unavailable (%s)", d.why.c_str());
  return 0;
}

// ------------------------------------------------------------- per-device state
// What a launch needs besides its operands - the 4-word status block its bounded waits report
// to, the split-K workspace and the tile counters - belongs to the STREAM it is queued on:
// launches on one stream run in order and may share them, launches on different streams of one
// GPU may overlap and must not. Slots are created on a stream's first launch and recycled
// least-recently-used beyond kMaxStreamSlots (a freed buffer is released with cuMemFree, which
// waits for the work that still uses it).
struct StreamSlot {
  CUstream stream = nullptr;
  CUdeviceptr status = 0;      // 4 x u32
  CUdeviceptr ws = 0;          // split-K partials
  size_t ws_bytes = 0;
  CUdeviceptr counters = 0;    // split-K tile counters
  size_t counters_n = 0;
  uint64_t last_use = 0;
};
constexpr size_t kMaxStreamSlots = 32;

struct DeviceState {
  bool init = false;
  CUcontext ctx = nullptr;
  std::vector<StreamSlot> slots;
  uint64_t use_clock = 0;
  CUdeviceptr hbuf[3] = {0, 0, 0};  // device copies for kcg_matmul_host
  size_t hbuf_bytes[3] = {0, 0, 0};
  CUstream hstream[3] = {nullptr, nullptr, nullptr};  // kcg_matmul_host: copy-in, compute, copy-out
  std::vector<CUevent> hevents;                       // slab hand-off events of kcg_matmul_host
  std::unordered_map<std::string, CUtensorMap> tmaps;
};
constexpr int kMaxDevices = 16;
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mutex;  // guards g_dev[*] (slots, buffers, tensor-map cache)
std::atomic<uint64_t> g_launches{0};

int ensure_device(int device, DeviceState** out) {
  if (int e = need_driver()) return e;
  if (device < 0 || device >= kMaxDevices) return fail(KCG_E_BAD_ARG, "device %d out of range", device);
  DeviceState& s = g_dev[device];
  {
    std::lock_guard<std::mutex> g(g_dev_mutex);
    if (!s.init) {
      CUdevice dev;
      DRV(cuDeviceGet(&dev, device));
      DRV(cuDevicePrimaryCtxRetain(&s.ctx, dev));
      s.slots.reserve(kMaxStreamSlots);
      s.init = true;
    }
  }
  CUcontext cur = nullptr;
  DRV(cuCtxGetCurrent(&cur));
  if (cur != s.ctx) DRV(cuCtxSetCurrent(s.ctx));
  *out = &s;
  return 0;
}

int grow(CUdeviceptr* p, size_t* have, size_t need) {
  if (*have >= need) return 0;
  if (*p) DRV(cuMemFree(*p));
  *p = 0;
  *have = 0;
  DRV(cuMemAlloc(p, need));
  *have = need;
  return 0;
}

int free_slot(StreamSlot& sl) {
  if (sl.status) DRV(cuMemFree(sl.status));
  if (sl.ws) DRV(cuMemFree(sl.ws));
  if (sl.counters) DRV(cuMemFree(sl.counters));
  sl = StreamSlot();
  return 0;
}

// The slot of `stream` on this device (created on first use). Call with g_dev_mutex held.
int slot_for(DeviceState* s, CUstream stream, bool create, StreamSlot** out) {
  *out = nullptr;
  for (StreamSlot& sl : s->slots)
    if (sl.status && sl.stream == stream) {
      sl.last_use = ++s->use_clock;
      *out = &sl;
      return 0;
    }
  if (!create) return 0;
  StreamSlot* dst = nullptr;
  for (StreamSlot& sl : s->slots)
    if (!sl.status) dst = &sl;
  if (!dst && s->slots.size() >= kMaxStreamSlots) {
    dst = &s->slots[0];
    for (StreamSlot& sl : s->slots)
      if (sl.last_use < dst->last_use) dst = &sl;
    if (int e = free_slot(*dst)) return e;
    s->tmaps.clear();  // maps of the freed workspace
  }
  if (!dst) {
    s->slots.emplace_back();
    dst = &s->slots.back();
  }
  dst->stream = stream;
  DRV(cuMemAlloc(&dst->status, 16));
  DRV(cuMemsetD32(dst->status, 0, 4));
  dst->last_use = ++s->use_clock;
  *out = dst;
  return 0;
}

// ----------------------------------------------------------------- config logic
struct Cfg {
  int v[KCG_NUM_CFG_KEYS];
  int operator[](int i) const { return v[i]; }
};

const char* dtype_str(int dt) {
  switch (dt) {
    case KCG_DTYPE_FLOAT16: return "float16";
    case KCG_DTYPE_FLOAT32: return "float32";
    case KCG_DTYPE_BFLOAT16: return "bfloat16";
    default: return nullptr;
  }
}

struct Resolved {
  int kernel = 0;
  int stages = 0;
  int num_sms = 148;
  int btrans = 0;
  int serpentine = 0;
  int out_f32 = 0;  // DATATYPE_C = float32 with 16-bit A and B
};

// The reference's KernelArgMatmul.check() (Operators/matmul.py:180-194) for the
// thread-level keys; the SIMT kernel consumes all of them.
int check_simt(const Cfg& c) {
  const int bm = c[KCG_CFG_BLOCK_SIZE_M], bn = c[KCG_CFG_BLOCK_SIZE_N], bk = c[KCG_CFG_BLOCK_SIZE_K];
  const int tm = c[KCG_CFG_THREAD_SIZE_M], tn = c[KCG_CFG_THREAD_SIZE_N];
  if (tm <= 0 || tn <= 0 || bm % tm || bn % tn) return fail(KCG_E_BAD_CONFIG, "BLOCK_SIZE_M/N not divisible by THREAD_SIZE_M/N");
  if (c[KCG_CFG_BLOCK_LAYOUT_M] * c[KCG_CFG_WARP_LAYOUT_M] != bm / tm ||
      c[KCG_CFG_BLOCK_LAYOUT_N] * c[KCG_CFG_WARP_LAYOUT_N] != bn / tn)
    return fail(KCG_E_BAD_CONFIG, "BLOCK_LAYOUT x WARP_LAYOUT does not cover BLOCK_SIZE / THREAD_SIZE");
  if (c[KCG_CFG_WARP_LAYOUT_M] * c[KCG_CFG_WARP_LAYOUT_N] != c[KCG_CFG_WARP_SIZE])
    return fail(KCG_E_BAD_CONFIG, "WARP_LAYOUT_M * WARP_LAYOUT_N != WARP_SIZE");
  const int lsu = c[KCG_CFG_LOCAL_SPLIT_U] > 0 ? c[KCG_CFG_LOCAL_SPLIT_U] : 1;
  const int threads = (bm / tm) * (bn / tn) * lsu;
  if (threads > 1024) return fail(KCG_E_BAD_CONFIG, "%d threads per block exceed 1024", threads);
  if (bk % lsu) return fail(KCG_E_BAD_CONFIG, "LOCAL_SPLIT_U must divide BLOCK_SIZE_K");
  auto pos = [](int x) { return x > 0 ? x : 1; };
  const int wswa = pos(c[KCG_CFG_WARP_SCATTER_WIDTH_A]), wswb = pos(c[KCG_CFG_WARP_SCATTER_WIDTH_B]);
  const int tswa = pos(c[KCG_CFG_THREAD_SCATTER_WIDTH_A]), tswb = pos(c[KCG_CFG_THREAD_SCATTER_WIDTH_B]);
  if (tm % wswa || wswa % tswa || tn % wswb || wswb % tswb)
    return fail(KCG_E_BAD_CONFIG, "scatter widths must nest: THREAD_SIZE %% WARP_SCATTER %% THREAD_SCATTER");
  const int glwa = pos(c[KCG_CFG_GLOB_LOAD_WIDTH_A]), glwb = pos(c[KCG_CFG_GLOB_LOAD_WIDTH_B]);
  if ((bm * bk) % (threads * glwa) || (bn * bk) % (threads * glwb))
    return fail(KCG_E_BAD_CONFIG, "tile loads do not split evenly over %d threads", threads);
  if ((c[KCG_CFG_IS_ATRANS] ? bm : bk) % glwa || bn % glwb)
    return fail(KCG_E_BAD_CONFIG, "GLOB_LOAD_WIDTH does not divide the contiguous tile extent");
  const int gsw = pos(c[KCG_CFG_GLOB_STORE_WIDTH]);
  if (lsu > 1 ? ((bm * bn) % (threads * gsw) != 0 && (bm * bn) % gsw != 0) : (tswb % (gsw < tswb ? gsw : tswb) != 0))
    return fail(KCG_E_BAD_CONFIG, "GLOB_STORE_WIDTH incompatible with the tile");
  if (lsu > 1 && bn % gsw) return fail(KCG_E_BAD_CONFIG, "GLOB_STORE_WIDTH must divide BLOCK_SIZE_N");
  return 0;
}

int simt_smem_bytes(const Cfg& c) {
  const int bm = c[KCG_CFG_BLOCK_SIZE_M], bn = c[KCG_CFG_BLOCK_SIZE_N], bk = c[KCG_CFG_BLOCK_SIZE_K];
  const int lsu = c[KCG_CFG_LOCAL_SPLIT_U] > 0 ? c[KCG_CFG_LOCAL_SPLIT_U] : 1;
  const int ab = (c[KCG_CFG_SHARED_PREFETCH] ? 2 : 1) * (bm + bn) * bk;
  const int cc = lsu > 1 ? lsu * bm * bn : 0;
  return 4 * (ab > cc ? ab : cc);
}

int resolve(const Cfg& c, const kcg_compile_opts* opts, Resolved* r) {
  const int dt = c[KCG_CFG_DATATYPE_A];
  if (!dtype_str(dt)) return fail(KCG_E_BAD_CONFIG, "unsupported DATATYPE_A %d (2 float16, 4 float32, 62 bfloat16)", dt);
  // A, B and C share one type, with one exception: fp16 / bf16 operands with a float32 C (the fp32
  // accumulators stored unrounded) on the single-pass tcgen05 kernels.
  const bool out_f32 = dt != KCG_DTYPE_FLOAT32 && c[KCG_CFG_DATATYPE_C] == KCG_DTYPE_FLOAT32;
  if (c[KCG_CFG_DATATYPE_B] != dt || (c[KCG_CFG_DATATYPE_C] != dt && !out_f32))
    return fail(KCG_E_BAD_CONFIG, "DATATYPE_A/B/C must be equal (or C float32 with 16-bit A and B)");
  r->out_f32 = out_f32 ? 1 : 0;
  const int bm = c[KCG_CFG_BLOCK_SIZE_M], bn = c[KCG_CFG_BLOCK_SIZE_N], bk = c[KCG_CFG_BLOCK_SIZE_K];
  const int M = c[KCG_CFG_M_SIZE], N = c[KCG_CFG_N_SIZE], K = c[KCG_CFG_K_SIZE];
  if (bm <= 0 || bn <= 0 || bk <= 0 || M <= 0 || N <= 0 || K <= 0)
    return fail(KCG_E_BAD_CONFIG, "sizes must be positive");
  // problem-size check of KernelArgMatmul.check()
  if (M % bm || N % bn || K % bk)
    return fail(KCG_E_BAD_CONFIG, "M,N,K = %d,%d,%d not divisible by BLOCK_SIZE_M,N,K = %d,%d,%d", M, N, K, bm, bn, bk);
  r->num_sms = (opts && opts->num_sms > 0) ? opts->num_sms : 148;
  int want = opts ? opts->kernel : KCG_KERNEL_AUTO;
  const int x3 = (want == KCG_KERNEL_TF32X1) ? 0 : 1;
  auto pick_stages = [&](int x3v) {
    if (opts && opts->num_stages > 0) return opts->num_stages;
    if (!c[KCG_CFG_SHARED_PREFETCH]) return 2;
    int s = 2;
    while (s < 6 && kcg::tc_config_error(dt, bm, bn, bk, s + 1, x3v) == 0) ++s;
    return s;
  };
  if (want == KCG_KERNEL_AUTO) {
    const int st = pick_stages(1);
    want = (kcg::tc_config_error(dt, bm, bn, bk, st, 1) == 0) ? KCG_KERNEL_TCGEN05 : KCG_KERNEL_SIMT;
  }
  r->kernel = want;
  if (r->out_f32 && !(want == KCG_KERNEL_TCGEN05 || want == KCG_KERNEL_TCGEN05_PAIR))
    return fail(KCG_E_BAD_CONFIG, "a float32 C with 16-bit A and B needs a single-pass tcgen05 kernel (KERNEL_VARIANT 2 or 4)");
  r->btrans = (opts && opts->b_trans) ? 1 : 0;
  r->serpentine = (opts && opts->serpentine) ? 1 : 0;
  if (r->serpentine && !(want == KCG_KERNEL_TCGEN05 || want == KCG_KERNEL_TF32X1 || want == KCG_KERNEL_TCGEN05_PAIR ||
                         want == KCG_KERNEL_TCGEN05_CLUSTERK))
    return fail(KCG_E_BAD_CONFIG, "the serpentine raster belongs to the tcgen05 kernels' tile walk");
  if (r->serpentine && c[KCG_CFG_BLOCK_MAPPING] < 2)
    return fail(KCG_E_BAD_CONFIG, "the serpentine raster needs BLOCK_MAPPING >= 2 (rows per group)");
  if (r->btrans) {
    const bool single_pass16 = (want == KCG_KERNEL_TCGEN05 || want == KCG_KERNEL_TCGEN05_PAIR) && dt != KCG_DTYPE_FLOAT32;
    if (!single_pass16)
      return fail(KCG_E_BAD_CONFIG, "a B stored N x K (b_trans) needs a single-pass tcgen05 kernel with fp16 / bf16 data");
    if (K % 8) return fail(KCG_E_BAD_CONFIG, "K must be a multiple of 8 for the TMA row stride of an N x K stored B");
  }
  if (want == KCG_KERNEL_TCGEN05 || want == KCG_KERNEL_TF32X1) {
    if (want == KCG_KERNEL_TF32X1 && dt != KCG_DTYPE_FLOAT32)
      return fail(KCG_E_BAD_CONFIG, "the single-pass TF32 kernel needs float32 data");
    r->stages = pick_stages(x3);
    const int e = kcg::tc_config_error(dt, bm, bn, bk, r->stages, x3);
    if (e) return fail(KCG_E_BAD_CONFIG, "tile %dx%dx%d / %d stages not buildable by the tcgen05 kernel (rule %d)", bm, bn, bk, r->stages, e);
    if (N % 8) return fail(KCG_E_BAD_CONFIG, "N must be a multiple of 8 for TMA row strides");
    const int splitk = c[KCG_CFG_LOCAL_SPLIT_U] > 0 ? c[KCG_CFG_LOCAL_SPLIT_U] : 1;
    if (splitk > K / bk) return fail(KCG_E_BAD_CONFIG, "LOCAL_SPLIT_U %d exceeds the %d K blocks", splitk, K / bk);
  } else if (want == KCG_KERNEL_TCGEN05_PAIR) {
    // CTA pairs: each CTA holds BM/2 rows of the tile and BN/2 columns of B
    const int f32 = (dt == KCG_DTYPE_FLOAT32) ? 1 : 0;
    if (f32 ? (bm != 256 && bm != 512) : (bm != 256 && bm != 512))
      return fail(KCG_E_BAD_CONFIG, "the CTA-pair kernels need BLOCK_SIZE_M = 256 or 512 (128 or 256 rows per CTA)");
    if ((bm / 256) * bn > (f32 ? 256 : 512))
      return fail(KCG_E_BAD_CONFIG, "accumulators of the tile exceed the TMEM columns available");
    const int splitk = c[KCG_CFG_LOCAL_SPLIT_U] > 0 ? c[KCG_CFG_LOCAL_SPLIT_U] : 1;
    if (splitk > K / bk) return fail(KCG_E_BAD_CONFIG, "LOCAL_SPLIT_U %d exceeds the %d K blocks", splitk, K / bk);
    auto ok = [&](int st) { return bn % 2 == 0 && kcg::tc_config_error(dt, bm / 2, bn / 2, bk, st, f32) == 0; };
    int st = (opts && opts->num_stages > 0) ? opts->num_stages : 2;
    if (!(opts && opts->num_stages > 0) && c[KCG_CFG_SHARED_PREFETCH])
      while (st < 7 && ok(st + 1)) ++st;
    if (!ok(st)) return fail(KCG_E_BAD_CONFIG, "tile %dx%dx%d / %d stages not buildable by the CTA-pair kernel", bm, bn, bk, st);
    if (N % 8) return fail(KCG_E_BAD_CONFIG, "N must be a multiple of 8 for TMA row strides");
    r->stages = st;
  } else if (want == KCG_KERNEL_TCGEN05_CLUSTERK) {
    // one 128-row tile per cluster of LOCAL_SPLIT_U CTAs, partial tiles reduced in shared memory
    const int split = c[KCG_CFG_LOCAL_SPLIT_U];
    if (bm != 128) return fail(KCG_E_BAD_CONFIG, "the cluster split-K kernel needs BLOCK_SIZE_M = 128");
    if (split > K / bk) return fail(KCG_E_BAD_CONFIG, "LOCAL_SPLIT_U %d exceeds the %d K blocks", split, K / bk);
    auto ok = [&](int st) { return kcg::ck_config_error(dt, bn, bk, st, split) == 0; };
    int st = (opts && opts->num_stages > 0) ? opts->num_stages : 2;
    if (!(opts && opts->num_stages > 0)) {
      while (st < 8 && !ok(st)) ++st;                                   // the ring must hold the received slices
      if (c[KCG_CFG_SHARED_PREFETCH]) while (st < 8 && ok(st + 1)) ++st;  // then as deep as fits
    }
    if (!ok(st))
      return fail(KCG_E_BAD_CONFIG,
                  "tile 128x%dx%d / %d stages / LOCAL_SPLIT_U %d not buildable by the cluster split-K kernel (rule %d: "
                  "fp16 / bf16, split 2..4 and at most BLOCK_SIZE_N / 32, ring large enough for the exchange buffers)",
                  bn, bk, st, split, kcg::ck_config_error(dt, bn, bk, st, split));
    if (N % 8) return fail(KCG_E_BAD_CONFIG, "N must be a multiple of 8 for TMA row strides");
    r->stages = st;
  } else if (want == KCG_KERNEL_SIMT) {
    if (int e = check_simt(c)) return e;
    r->stages = c[KCG_CFG_SHARED_PREFETCH] ? 2 : 1;
    if (simt_smem_bytes(c) > 227 * 1024) return fail(KCG_E_BAD_CONFIG, "shared memory %d B exceeds 227 KiB", simt_smem_bytes(c));
  } else if (want == KCG_KERNEL_NAIVE || want == KCG_KERNEL_WAIT_PROBE) {
    r->stages = 1;
  } else {
    return fail(KCG_E_BAD_CONFIG, "unknown kernel family %d", want);
  }
  return 0;
}

// Same scheme as MatmulParams::getKernelName (src/main.cc:119-145) plus the two
// keys this library adds (stages, kernel family).
std::string kernel_name(const Cfg& c, const Resolved& r) {
  std::ostringstream ss;
  ss << "GEMM_MNK" << c[KCG_CFG_M_SIZE] << "x" << c[KCG_CFG_N_SIZE] << "x" << c[KCG_CFG_K_SIZE] << "_";
  ss << "DTabc" << dtype_str(c[KCG_CFG_DATATYPE_A]) << "x" << dtype_str(c[KCG_CFG_DATATYPE_B]) << "x"
     << dtype_str(c[KCG_CFG_DATATYPE_C]) << "_";
  ss << "AT" << (c[KCG_CFG_IS_ATRANS] ? 1 : 0) << "_";
  ss << "TTmn" << c[KCG_CFG_THREAD_SIZE_M] << "x" << c[KCG_CFG_THREAD_SIZE_N] << "_";
  ss << "BTmnk" << c[KCG_CFG_BLOCK_SIZE_M] << "x" << c[KCG_CFG_BLOCK_SIZE_N] << "x" << c[KCG_CFG_BLOCK_SIZE_K] << "_";
  ss << "BLmn" << c[KCG_CFG_BLOCK_LAYOUT_M] << "x" << c[KCG_CFG_BLOCK_LAYOUT_N] << "_";
  ss << "WLmn" << c[KCG_CFG_WARP_LAYOUT_M] << "x" << c[KCG_CFG_WARP_LAYOUT_N] << "_";
  ss << "GLWab" << c[KCG_CFG_GLOB_LOAD_WIDTH_A] << "x" << c[KCG_CFG_GLOB_LOAD_WIDTH_B] << "_";
  ss << "GSW" << c[KCG_CFG_GLOB_STORE_WIDTH] << "_";
  ss << "WSWab" << c[KCG_CFG_WARP_SCATTER_WIDTH_A] << "x" << c[KCG_CFG_WARP_SCATTER_WIDTH_B] << "_";
  ss << "TSWab" << c[KCG_CFG_THREAD_SCATTER_WIDTH_A] << "x" << c[KCG_CFG_THREAD_SCATTER_WIDTH_B] << "_";
  ss << "LSU" << c[KCG_CFG_LOCAL_SPLIT_U] << "_";
  ss << "BM" << c[KCG_CFG_BLOCK_MAPPING] << "_";
  ss << "UNROLL" << c[KCG_CFG_UNROLL_NUM] << "_";
  ss << "REGP" << c[KCG_CFG_REG_PREFETCH] << "_";
  ss << "SHMP" << c[KCG_CFG_SHARED_PREFETCH] << "_";
  ss << "LC" << c[KCG_CFG_LOAD_CONTINUOUS] << "_";
  ss << "RC" << c[KCG_CFG_REDUCE_C_CONTINUOUS] << "_";
  ss << "ST" << r.stages << "_V" << r.kernel;
  if (r.btrans) ss << "_BT1";
  if (r.serpentine) ss << "_SP1";
  return ss.str();
}

std::string lib_dir() {
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&lib_dir), &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    const size_t slash = p.rfind('/');
    if (slash != std::string::npos) return p.substr(0, slash);
  }
  return ".";
}

std::string kernel_src_dir() {
  const char* e = getenv("KCG_KERNEL_SRC_DIR");
  return (e && *e) ? std::string(e) : lib_dir() + "/csrc/kernels";
}

// Tag of the kernel sources a cubin was built from: FNV-1a over the names and contents of the
// files in the kernel source directory, in name order. Cubins live in a sub-directory named
// after it, so an edit of any kernel header can never be served by a cubin of the old source.
// Without sources (a deployment that ships cubins only) the newest tagged sub-directory is used.
std::string source_tag(const std::string& cache_base) {
  static std::mutex mu;
  static std::string tag;
  std::lock_guard<std::mutex> g(mu);
  if (!tag.empty()) return tag;
  std::vector<std::string> names;
  const std::string dir = kernel_src_dir();
  if (DIR* d = opendir(dir.c_str())) {
    while (struct dirent* ent = readdir(d)) {
      const std::string n = ent->d_name;
      if (n.size() > 2 && n[0] != '.' &&
          (n.rfind(".cu") == n.size() - 3 || n.rfind(".cuh") == n.size() - 4 || n.rfind(".h") == n.size() - 2))
        names.push_back(n);
    }
    closedir(d);
  }
  if (names.empty()) {
    std::string best;
    time_t best_t = 0;
    if (DIR* d = opendir(cache_base.c_str())) {
      while (struct dirent* ent = readdir(d)) {
        const std::string n = ent->d_name;
        struct stat st;
        if (n.rfind("src-", 0) == 0 && stat((cache_base + "/" + n).c_str(), &st) == 0 && S_ISDIR(st.st_mode) &&
            (best.empty() || st.st_mtime > best_t)) {
          best = n;
          best_t = st.st_mtime;
        }
      }
      closedir(d);
    }
    tag = best.empty() ? "src-none" : best;
    return tag;
  }
  std::sort(names.begin(), names.end());
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](const char* p, size_t n) {
    for (size_t i = 0; i < n; ++i) {
      h ^= static_cast<unsigned char>(p[i]);
      h *= 1099511628211ull;
    }
  };
  for (const std::string& n : names) {
    mix(n.data(), n.size() + 1);
    std::ifstream f(dir + "/" + n, std::ios::binary);
    std::string body((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    mix(body.data(), body.size());
  }
  char buf[32];
  snprintf(buf, sizeof(buf), "src-%012llx", static_cast<unsigned long long>(h & 0xffffffffffffull));
  tag = buf;
  return tag;
}

std::string cache_dir() {
  const char* e = getenv("KCG_CACHE_DIR");
  const std::string base = (e && *e) ? std::string(e) : lib_dir() + "/_cache";
  mkdir(base.c_str(), 0755);
  const std::string d = base + "/" + source_tag(base);
  mkdir(d.c_str(), 0755);
  return d;
}

std::string find_nvcc() {
  const char* e = getenv("KCG_NVCC");
  if (e && *e) return e;
  if (access("/usr/local/cuda/bin/nvcc", X_OK) == 0) return "/usr/local/cuda/bin/nvcc";
  const char* path = getenv("PATH");
  if (path) {
    std::stringstream ss(path);
    std::string dir;
    while (std::getline(ss, dir, ':')) {
      const std::string cand = dir + "/nvcc";
      if (access(cand.c_str(), X_OK) == 0) return cand;
    }
  }
  return "";
}

bool file_exists(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && st.st_size > 0;
}

std::string tail_of(const std::string& path, size_t n) {
  std::ifstream f(path);
  std::stringstream ss;
  ss << f.rdbuf();
  std::string s = ss.str();
  return s.size() > n ? s.substr(s.size() - n) : s;
}

std::vector<std::string> macro_flags(const Cfg& c, const Resolved& r, const std::string& name) {
  auto pos = [](int x) { return x > 0 ? x : 1; };
  std::vector<std::string> f;
  auto D = [&](const char* k, int v) { f.push_back(std::string("-DKCG_") + k + "=" + std::to_string(v)); };
  f.push_back("-DKCG_KERNEL_NAME=" + name);
  D("VARIANT", r.kernel);
  D("DTYPE", c[KCG_CFG_DATATYPE_A]);
  D("BM", c[KCG_CFG_BLOCK_SIZE_M]);
  D("BN", c[KCG_CFG_BLOCK_SIZE_N]);
  D("BK", c[KCG_CFG_BLOCK_SIZE_K]);
  D("STAGES", r.stages);
  D("ATRANS", c[KCG_CFG_IS_ATRANS] ? 1 : 0);
  D("SPLITK", pos(c[KCG_CFG_LOCAL_SPLIT_U]));
  D("GROUP", c[KCG_CFG_BLOCK_MAPPING] > 0 ? c[KCG_CFG_BLOCK_MAPPING] : 0);
  if (r.kernel == KCG_KERNEL_SIMT) {
    D("TM", c[KCG_CFG_THREAD_SIZE_M]);
    D("TN", c[KCG_CFG_THREAD_SIZE_N]);
    D("BLM", c[KCG_CFG_BLOCK_LAYOUT_M]);
    D("BLN", c[KCG_CFG_BLOCK_LAYOUT_N]);
    D("WLM", c[KCG_CFG_WARP_LAYOUT_M]);
    D("WLN", c[KCG_CFG_WARP_LAYOUT_N]);
    D("WSWA", pos(c[KCG_CFG_WARP_SCATTER_WIDTH_A]));
    D("WSWB", pos(c[KCG_CFG_WARP_SCATTER_WIDTH_B]));
    D("TSWA", pos(c[KCG_CFG_THREAD_SCATTER_WIDTH_A]));
    D("TSWB", pos(c[KCG_CFG_THREAD_SCATTER_WIDTH_B]));
    D("GLWA", pos(c[KCG_CFG_GLOB_LOAD_WIDTH_A]));
    D("GLWB", pos(c[KCG_CFG_GLOB_LOAD_WIDTH_B]));
    D("GSW", pos(c[KCG_CFG_GLOB_STORE_WIDTH]));
    D("SHMP", c[KCG_CFG_SHARED_PREFETCH] ? 1 : 0);
  }
  // SIMT: register double buffer of the fragments; single-pass tcgen05 kernels: overlap of the
  // accumulator drain with the next tile's main loop
  D("REGP", c[KCG_CFG_REG_PREFETCH] ? 1 : 0);
  D("BTRANS", r.btrans);
  D("SERPENTINE", r.serpentine);
  D("OUT_F32", r.out_f32);
  return f;
}

int run_nvcc(const std::string& nvcc, const std::vector<std::string>& flags, const std::string& out,
             const std::string& log) {
  std::vector<std::string> args = {nvcc, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
                                   "-std=c++17", "-lineinfo", "-I" + kernel_src_dir()};
  args.insert(args.end(), flags.begin(), flags.end());
  // KCG_NVCC_FLAGS: extra flags for experiments (e.g. -DKCG_TIMELINE=1 -Xptxas -v). The cubin cache is
  // keyed by kernel name and source text only, so point KCG_CACHE_DIR elsewhere when using it.
  if (const char* extra = getenv("KCG_NVCC_FLAGS")) {
    std::stringstream es(extra);
    std::string tok;
    while (es >> tok) args.push_back(tok);
  }
  args.push_back("-o");
  args.push_back(out);
  args.push_back(kernel_src_dir() + "/gemm_entry.cu");
  std::vector<char*> argv;
  for (auto& a : args) argv.push_back(const_cast<char*>(a.c_str()));
  argv.push_back(nullptr);
  posix_spawn_file_actions_t fa;
  posix_spawn_file_actions_init(&fa);
  posix_spawn_file_actions_addopen(&fa, 1, log.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  posix_spawn_file_actions_adddup2(&fa, 1, 2);
  pid_t pid;
  const int rc = posix_spawn(&pid, nvcc.c_str(), &fa, nullptr, argv.data(), environ);
  posix_spawn_file_actions_destroy(&fa);
  if (rc != 0) return -1;
  int status = 0;
  if (waitpid(pid, &status, 0) < 0) return -1;
  return (WIFEXITED(status) && WEXITSTATUS(status) == 0) ? 0 : 1;
}

int fill_info(const Cfg& c, const Resolved& r, const std::string& name, const std::string& path,
              kcg_kernel_info* out) {
  memset(out, 0, sizeof(*out));
  if (path.size() >= sizeof(out->path) || name.size() >= sizeof(out->name))
    return fail(KCG_E_TOO_LARGE, "path or kernel name too long");
  strcpy(out->path, path.c_str());
  strcpy(out->name, name.c_str());
  const int bm = c[KCG_CFG_BLOCK_SIZE_M], bn = c[KCG_CFG_BLOCK_SIZE_N], bk = c[KCG_CFG_BLOCK_SIZE_K];
  const int M = c[KCG_CFG_M_SIZE], N = c[KCG_CFG_N_SIZE], K = c[KCG_CFG_K_SIZE];
  const int lsu = c[KCG_CFG_LOCAL_SPLIT_U] > 0 ? c[KCG_CFG_LOCAL_SPLIT_U] : 1;
  const int tiles = (M / bm) * (N / bn);
  out->grid[1] = out->grid[2] = out->block[1] = out->block[2] = 1;
  out->cluster[0] = out->cluster[1] = out->cluster[2] = 1;
  if (r.kernel == KCG_KERNEL_TCGEN05 || r.kernel == KCG_KERNEL_TF32X1) {
    const int x3 = (r.kernel == KCG_KERNEL_TCGEN05) ? 1 : 0;
    const int units = tiles * lsu;
    out->grid[0] = units < r.num_sms ? units : r.num_sms;  // persistent CTAs
    // single-pass kernel: producer, MMA, four epilogue warps, two push warps (fused all-gather)
    out->block[0] = (c[KCG_CFG_DATATYPE_A] == KCG_DTYPE_FLOAT32 && x3) ? 512 : 256;
    out->smem_bytes = kcg::tc_smem_bytes(c[KCG_CFG_DATATYPE_A], bm, bn, bk, r.stages, x3);
  } else if (r.kernel == KCG_KERNEL_TCGEN05_PAIR) {
    const int f32 = (c[KCG_CFG_DATATYPE_A] == KCG_DTYPE_FLOAT32) ? 1 : 0;
    const int units = tiles * lsu;
    const int pairs = units < r.num_sms / 2 ? units : r.num_sms / 2;
    out->grid[0] = 2 * pairs;  // persistent clusters of two CTAs
    out->cluster[0] = 2;
    out->block[0] = f32 ? 512 : 256;
    out->smem_bytes = kcg::tc_smem_bytes(c[KCG_CFG_DATATYPE_A], bm / 2, bn / 2, bk, r.stages, f32);
  } else if (r.kernel == KCG_KERNEL_TCGEN05_CLUSTERK) {
    out->grid[0] = tiles * lsu;  // one cluster of LOCAL_SPLIT_U CTAs per tile
    out->cluster[0] = lsu;
    out->block[0] = 192;  // producer, MMA, four epilogue warps
    out->smem_bytes = kcg::ck_smem_bytes(bn, bk, r.stages);
  } else if (r.kernel == KCG_KERNEL_SIMT) {
    // grid/block as the reference derives them (Optimizer.cc:20,336; Rewriter.cc:726-761)
    out->grid[0] = tiles;
    out->block[0] = (bm / c[KCG_CFG_THREAD_SIZE_M]) * (bn / c[KCG_CFG_THREAD_SIZE_N]) * lsu;
    out->smem_bytes = simt_smem_bytes(c);
  } else {
    out->grid[0] = (N + 15) / 16;
    out->grid[1] = (M + 15) / 16;
    out->block[0] = 16;
    out->block[1] = 16;
    out->smem_bytes = 0;
  }
  out->kernel = r.kernel;
  out->dtype = c[KCG_CFG_DATATYPE_A];
  out->bm = bm;
  out->bn = bn;
  out->bk = bk;
  out->stages = r.stages;
  out->splitk = (r.kernel == KCG_KERNEL_NAIVE || r.kernel == KCG_KERNEL_WAIT_PROBE) ? 1 : lsu;
  if (r.kernel == KCG_KERNEL_WAIT_PROBE) {
    out->grid[0] = out->grid[1] = 1;
    out->block[0] = 32;
    out->block[1] = 1;
  }
  out->group = c[KCG_CFG_BLOCK_MAPPING];
  out->atrans = c[KCG_CFG_IS_ATRANS] ? 1 : 0;
  out->m = M;
  out->n = N;
  out->k = K;
  out->reserved[0] = r.num_sms;
  out->reserved[1] = r.btrans;
  out->reserved[2] = r.serpentine;
  out->reserved[3] = r.out_f32 ? KCG_DTYPE_FLOAT32 : 0;
  {
    // accumulator buffers of the single-pass tcgen05 kernels: two when REG_PREFETCH is on and two
    // copies of a CTA's accumulator fit the 512 TMEM columns (gemm_tcgen05.cuh: NACC)
    const int rows = bm / (r.kernel == KCG_KERNEL_TCGEN05_PAIR ? 2 : 1);
    const int acc_cols = (rows / 128 > 0 ? rows / 128 : 1) * bn;
    out->reserved[4] = (c[KCG_CFG_REG_PREFETCH] && 2 * acc_cols <= 512) ? 2 : 1;
  }
  return 0;
}

int encode_map(DeviceState* s, CUtensorMap* out, int dtype, uint64_t ptr, uint64_t inner, uint64_t outer,
               uint64_t row_bytes, int box_inner, int box_outer, int swizzle) {
  char key[160];
  snprintf(key, sizeof(key), "%d:%llx:%llu:%llu:%llu:%d:%d:%d", dtype, (unsigned long long)ptr,
           (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_bytes, box_inner,
           box_outer, swizzle);
  auto it = s->tmaps.find(key);  // the caller holds g_dev_mutex
  if (it != s->tmaps.end()) {
    *out = it->second;
    return 0;
  }
  const CUtensorMapDataType dt = dtype == KCG_DTYPE_FLOAT32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == KCG_DTYPE_FLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {row_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  if (ptr % 16 || row_bytes % 16)
    return fail(KCG_E_BAD_ARG, "TMA needs 16-byte aligned base (%llx) and row pitch (%llu)", (unsigned long long)ptr,
                (unsigned long long)row_bytes);
  DRV(cuTensorMapEncodeTiled(out, dt, 2, reinterpret_cast<void*>(ptr), gdim, gstride, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(swizzle),
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  if (s->tmaps.size() > 4096) s->tmaps.clear();
  s->tmaps[key] = *out;
  return 0;
}

// How a tcgen05 launch cuts its tiles into work units (see kernels/work_iter.cuh).
struct SplitPlan {
  int tiles, first, factor, sk_per, sk_ranges, units_at_once, units_first;
};

SplitPlan plan_split(const kcg_kernel_info* info, bool fused_epilogue, int batch = 1) {
  const int M = info->m * batch, N = info->n, K = info->k;  // a batched product is one tall problem
  const bool pair = info->kernel == KCG_KERNEL_TCGEN05_PAIR;
  const bool x3 = info->dtype == KCG_DTYPE_FLOAT32 && info->kernel != KCG_KERNEL_TF32X1;
  // K splitting. LOCAL_SPLIT_U > 1 splits every tile evenly. Otherwise the tiles that do not fill
  // a wave of the persistent grid (the remainder) can be split over the CTAs so that every SM works
  // for about the same time:
  //  * even split (the default): each remainder tile is cut into floor(G / remainder) K ranges. In
  //    the single-pass kernels these split units run FIRST and the whole tiles after them: all
  //    contributors of a tile start with the kernel and finish together, their partial tiles are
  //    written, summed (a share each) and stored by the epilogue warps while the main loops of the
  //    whole tiles run, and the kernel ends with ordinary tiles. The 3xTF32 kernel, whose epilogue
  //    warps are busy during the main loop, keeps the split units last.
  //  * stream-K (KCG_TAIL_SPLIT=1): the remainder's K blocks - together with the full wave before
  //    it when it is less than half a wave - laid end to end and cut into one contiguous range per
  //    CTA (pair), after the whole tiles; tiles that fall into several ranges are reduced like an
  //    even split. Measured slower than the even split on every benchmarked shape (ranges straddle
  //    tile borders, so contributors finish at different times); kept for comparison.
  // KCG_TAIL_SPLIT=0 turns the split off, =2 selects the even split, =3 / =4 stream-K / the even
  // split without the cost gate, =5 stream-K over the remainder alone BEFORE the whole tiles (the
  // last arriver sums a tile; no gate; an experiment that measured no consistent gain).
  const int T = (M / info->bm) * (N / info->bn);
  const int num_kb = K / info->bk;
  const int nsm = info->reserved[0] > 0 ? info->reserved[0] : 148;
  const int G = pair ? nsm / 2 : nsm;  // work units that run at once (CTAs, or CTA pairs)
  int first = T, factor = 1, sk_per = 0, sk_ranges = 0;
  int units_first = 0;
  if (info->splitk > 1) {
    first = 0;
    factor = info->splitk;
  } else {
    const char* e = getenv("KCG_TAIL_SPLIT");
    const bool sk_first = e && e[0] == '5' && !x3;  // stream-K ranges before the whole tiles, no gate
    const bool ungated = e && (e[0] == '3' || e[0] == '4' || e[0] == '5');
    const int mode = (e && e[0] == '0') ? 0 : (e && (e[0] == '1' || e[0] == '3' || e[0] == '5')) ? 1 : 2;
    units_first = (!x3 && (mode == 2 || sk_first)) ? 1 : 0;
    const int rem = T % G;
    if (mode != 0 && rem > 0) {
      // Worth it only when the time saved exceeds the cost of the split. A tile's main-loop time is
      // estimated from a per-SM rate in MFLOP per microsecond: 10 for 16-bit data, 1.4 useful for fp32
      // as 3xTF32, 4.5 for the single TF32 pass.
      const double mflop_per_us = (info->dtype == KCG_DTYPE_FLOAT32 && info->kernel != KCG_KERNEL_TF32X1) ? 1.4
                                  : (info->dtype == KCG_DTYPE_FLOAT32)                                     ? 4.5
                                                                                                           : 10.0;
      const double tile_us =
          2.0 * (info->bm / (pair ? 2 : 1)) * info->bn * static_cast<double>(K) / 1e6 / mflop_per_us;
      const double partial_kb = (info->bm / (pair ? 2 : 1)) * static_cast<double>(info->bn) * 4.0 / 1024.0;
      // What a split costs, fitted to in-kernel timelines (128 KB partials: 3.4 us to write one,
      // ~4.6 us for a contributor to sum its share of a tile straight from L2, ~12 us for the whole
      // exchange at the end of a kernel when the contributors sum their shares out of their idle
      // operand rings; ~4.6 us per partial when the last arriver sums a tile alone):
      //  * hidden (whole tiles follow, single-pass kernels): a pipeline refill, plus whatever of
      //    the write + shared sum does not fit behind one whole tile's main loop;
      //  * exposed, shared (no whole tiles follow): 6 us + 0.05 us per KB of partial;
      //  * exposed, summed by the last arriver (3xTF32): 5 us + 0.18 us per KB of partial.
      const bool hidden = units_first != 0 && T > G;
      auto overhead_us = [&](int contrib) {
        if (hidden) {
          const double fix = 1.5 + partial_kb * (contrib <= 8 ? 0.063 : 0.027 + 0.036 * contrib);
          return 3.0 + (fix > tile_us ? fix - tile_us : 0.0);
        }
        return !x3 ? 6.0 + 0.05 * partial_kb : 5.0 + 0.18 * partial_kb;
      };
      const double margin = ungated ? 0.0 : 1.25;
      if (mode == 2) {
        // Cut each remainder tile into f K ranges; the rem * f units take ceil(rem * f / G) rounds
        // of 1/f of a tile's time. One round (f <= G / rem) always qualifies; several rounds - a
        // remainder of more than half a wave cut into quarters runs as three rounds, 3/4 of a
        // tile instead of a whole one - only when the units run first, whole tiles follow and the
        // kernel has two accumulator buffers (the MMAs of the next unit must not wait for the
        // epilogue warps, who are busy with the previous unit's partial tile): every unit's
        // write-and-sum (with the waits for partners a round apart, ~1.5 us + 0.14 us per KB
        // on the timelines) must fit behind the main loops that are still to come.
        double best_gain = 0.0;
        for (int f = 2; f <= 8 && f <= num_kb; ++f) {
          if (((num_kb + f - 1) / f) * (f - 1) >= num_kb) continue;  // the last range would be empty
          const int rounds = (rem * f + G - 1) / G;
          if (rounds > 1 && (!hidden || info->reserved[4] < 2)) break;  // needs a spare accumulator to run ahead
          double cost;
          // several rounds: a unit's write-and-sum must be over before the next unit's accumulator is
          // full, or the epilogue warps fall behind (1024x8192x8192 in quarters, 12 us units against
          // ~19 us: 4 % slower than unsplit; 2048x11008x11008 in thirds, 21 us units: 5 % faster)
          if (!ungated && rounds > 1 && tile_us / f < 1.5 + 0.14 * partial_kb) continue;
          if (hidden) {
            const double fix = rounds * (1.5 + 0.14 * partial_kb);
            const double room = tile_us * (1.0 + static_cast<double>(rounds - 1) / f);
            cost = 3.0 * rounds + (fix > room ? fix - room : 0.0);
          } else {
            cost = overhead_us(f);
          }
          const double gain = tile_us * (1.0 - static_cast<double>(rounds) / f) - margin * cost;
          if (gain > best_gain || (ungated && factor == 1 && rounds == 1)) {
            best_gain = gain > best_gain ? gain : best_gain;
            first = T - rem;
            factor = f;
          }
        }
      } else {
        // Tiles handed to stream-K: the remainder, together with the full wave before it when the
        // remainder is less than half a wave.
        const int R = (!sk_first && T > G && 2 * rem < G) ? rem + G : rem;
        const long long blocks = static_cast<long long>(R) * num_kb;
        const double waves_without = static_cast<double>((R + G - 1) / G);
        double best_gain = 0.0;
        for (int cap = 7; cap >= 2; --cap) {  // at most cap + 1 contributors per tile (eight can share a sum)
          long long ranges = G;
          if (ranges > static_cast<long long>(cap) * R) ranges = static_cast<long long>(cap) * R;
          if (ranges > blocks) ranges = blocks;
          const long long per = (blocks + ranges - 1) / ranges;
          ranges = (blocks + per - 1) / per;  // no empty range
          const int contrib = static_cast<int>((num_kb + per - 1) / per) + 1;
          const double saved_us = tile_us * (waves_without - static_cast<double>(R) / static_cast<double>(ranges));
          const double gain = saved_us - margin * overhead_us(contrib < cap + 1 ? contrib : cap + 1);
          if (gain > best_gain || (ungated && sk_per == 0)) {
            best_gain = gain > best_gain ? gain : best_gain;
            first = T - R;
            sk_per = static_cast<int>(per);
            sk_ranges = static_cast<int>(ranges);
          }
        }
      }
    }
  }
  // The 3xTF32 kernel applies a fused epilogue in its reduction loop only (its register file is
  // full of accumulators at the direct store), so a fused launch sends every tile through the
  // workspace as a one-way split; the tail split is not combined with it.
  const bool ws_epilogue = x3 && fused_epilogue;
  if (ws_epilogue && info->splitk <= 1) {
    first = 0;
    factor = 1;
    sk_per = 0;
  }
  return SplitPlan{T, first, factor, sk_per, sk_ranges, G, units_first};
}

}  // namespace

// ============================================================================ C ABI
extern "C" {

// Internal (not part of the ABI): lets the library's other translation units report through
// kcg_last_error() and count their launches.
int kcg_internal_fail(int code, const char* msg) { return fail(code, "%s", msg); }
void kcg_internal_count_launch(void) { g_launches.fetch_add(1); }
// Internal (tests): the work decomposition a launch of `info` would use:
// {tiles, split_first_tile, split_factor, sk_per, stream-K ranges, units that run at once, split units first}.
int kcg_internal_plan_split(const kcg_kernel_info* info, int fused_epilogue, int batch, int out[7]) {
  if (!info || !out || batch < 1) return fail(KCG_E_BAD_ARG, "null argument");
  const SplitPlan pl = plan_split(info, fused_epilogue != 0, batch);
  out[0] = pl.tiles;
  out[1] = pl.first;
  out[2] = pl.factor;
  out[3] = pl.sk_per;
  out[4] = pl.sk_ranges;
  out[5] = pl.units_at_once;
  out[6] = pl.units_first;
  return 0;
}

const char* kcg_last_error(void) { return g_last_error.c_str(); }
const char* kcg_version(void) { return "kcg-b200 0.1 (sm_100a)"; }
uint64_t kcg_launch_count(void) { return g_launches.load(); }

const char* kcg_cache_dir(void) {
  static thread_local std::string d;
  d = cache_dir();
  return d.c_str();
}

int kcg_kernel_name(const int32_t cfg[KCG_NUM_CFG_KEYS], const kcg_compile_opts* opts, char* buf, int buf_len) {
  if (!cfg || !buf || buf_len <= 0) return fail(KCG_E_BAD_ARG, "null argument");
  Cfg c;
  memcpy(c.v, cfg, sizeof(c.v));
  Resolved r;
  if (int e = resolve(c, opts, &r)) return e;
  const std::string n = kernel_name(c, r);
  if (static_cast<int>(n.size()) >= buf_len) return fail(KCG_E_TOO_LARGE, "buffer too small for kernel name");
  strcpy(buf, n.c_str());
  return 0;
}

int kcg_compile_matmul_ex(const int32_t cfg[KCG_NUM_CFG_KEYS], const kcg_compile_opts* opts, kcg_kernel_info* out) {
  if (!cfg || !out) return fail(KCG_E_BAD_ARG, "null argument");
  Cfg c;
  memcpy(c.v, cfg, sizeof(c.v));
  Resolved r;
  if (int e = resolve(c, opts, &r)) return e;
  const std::string name = kernel_name(c, r);
  const std::string dir = cache_dir();
  const std::string path = dir + "/" + name + ".cubin";
  if (int e = fill_info(c, r, name, path, out)) return e;
  if (file_exists(path) && !(opts && opts->force)) return 0;
  const std::string nvcc = find_nvcc();
  if (nvcc.empty())
    return fail(KCG_E_COMPILE, "no nvcc found (set KCG_NVCC) and no prebuilt cubin %s", path.c_str());
  const std::string tmp = dir + "/" + name + "." + std::to_string(getpid()) + ".tmp.cubin";
  const std::string log = dir + "/" + name + "." + std::to_string(getpid()) + ".log";
  const int rc = run_nvcc(nvcc, macro_flags(c, r, name), tmp, log);
  if (rc != 0) {
    const std::string t = tail_of(log, 1500);
    unlink(tmp.c_str());
    return fail(KCG_E_COMPILE, "nvcc failed for %s:\n%s", name.c_str(), t.c_str());
  }
  unlink(log.c_str());
  if (rename(tmp.c_str(), path.c_str()) != 0) return fail(KCG_E_IO, "cannot move cubin to %s", path.c_str());
  return 0;
}

int kcg_compile_matmul(const int32_t cfg[KCG_NUM_CFG_KEYS], kcg_kernel_info* out) {
  return kcg_compile_matmul_ex(cfg, nullptr, out);
}

int kcg_device_properties(int device, kcg_device_props* out) {
  if (!out) return fail(KCG_E_BAD_ARG, "null argument");
  if (int e = need_driver()) return e;
  CUdevice dev;
  DRV(cuDeviceGet(&dev, device));
  int v = 0;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN, dev));
  out->max_shared_mem = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dev));
  out->multiprocessor_count = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_CLOCK_RATE, dev));
  out->sm_clock_rate = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MEMORY_CLOCK_RATE, dev));
  out->mem_clock_rate = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_GLOBAL_MEMORY_BUS_WIDTH, dev));
  out->mem_bus_width = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE, dev));
  out->l2_cache_bytes = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, dev));
  out->cc_major = v;
  DRV(cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, dev));
  out->cc_minor = v;
  return 0;
}

int kcg_load_binary(const char* name, const char* path, int shared, int device, uint64_t* module,
                    uint64_t* function, int* n_regs, int* n_spills) {
  if (!name || !path || !module || !function) return fail(KCG_E_BAD_ARG, "null argument");
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  std::ifstream f(path, std::ios::binary);
  if (!f) return fail(KCG_E_IO, "cannot open cubin %s", path);
  std::vector<char> image((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  if (image.empty()) return fail(KCG_E_IO, "empty cubin %s", path);
  image.push_back(0);
  CUmodule mod;
  CUfunction fn;
  DRV(cuModuleLoadData(&mod, image.data()));
  CUresult r = driver().p_cuModuleGetFunction(&fn, mod, name);
  if (r != CUDA_SUCCESS) {
    driver().p_cuModuleUnload(mod);
    return drv_fail(r, "cuModuleGetFunction");
  }
  if (shared > 48 * 1024) {
    r = driver().p_cuFuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, shared);
    if (r != CUDA_SUCCESS) {
      driver().p_cuModuleUnload(mod);
      return drv_fail(r, "cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
    }
  }
  int regs = 0, local = 0;
  driver().p_cuFuncGetAttribute(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, fn);
  driver().p_cuFuncGetAttribute(&local, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, fn);
  if (n_regs) *n_regs = regs;
  if (n_spills) *n_spills = local / 4;
  *module = reinterpret_cast<uint64_t>(mod);
  *function = reinterpret_cast<uint64_t>(fn);
  return 0;
}

int kcg_unload(uint64_t module) {
  if (int e = need_driver()) return e;
  DRV(cuModuleUnload(reinterpret_cast<CUmodule>(module)));
  return 0;
}

int kcg_launch_gemm(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                    uint64_t B, uint64_t C) {
  return kcg_launch_gemm_ex(function, info, device, stream, A, B, C, nullptr);
}

int kcg_launch_gemm_ex(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                       uint64_t B, uint64_t C, const kcg_epilogue* epi) {
  return kcg_launch_gemm_allgather(function, info, device, stream, A, B, C, epi, nullptr, 0);
}

// ---- peer buffers: device memory another process of the same node can map (CUDA IPC)
int kcg_peer_alloc(int device, uint64_t bytes, uint64_t* dptr, uint8_t handle[64]) {
  if (!dptr || !handle || bytes == 0) return fail(KCG_E_BAD_ARG, "null argument");
  static_assert(sizeof(CUipcMemHandle) == 64, "IPC handle size");
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  CUdeviceptr d = 0;
  DRV(cuMemAlloc(&d, bytes));
  CUipcMemHandle h;
  CUresult r = driver().p_cuIpcGetMemHandle(&h, d);
  if (r != CUDA_SUCCESS) {
    driver().p_cuMemFree(d);
    return drv_fail(r, "cuIpcGetMemHandle");
  }
  memcpy(handle, &h, 64);
  *dptr = static_cast<uint64_t>(d);
  return 0;
}

int kcg_peer_open(int device, const uint8_t handle[64], uint64_t* dptr) {
  if (!dptr || !handle) return fail(KCG_E_BAD_ARG, "null argument");
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  CUipcMemHandle h;
  memcpy(&h, handle, 64);
  CUdeviceptr d = 0;
  DRV(cuIpcOpenMemHandle(&d, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
  *dptr = static_cast<uint64_t>(d);
  return 0;
}

int kcg_peer_close(int device, uint64_t dptr) {
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  DRV(cuIpcCloseMemHandle(static_cast<CUdeviceptr>(dptr)));
  return 0;
}

int kcg_peer_free(int device, uint64_t dptr) {
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  DRV(cuMemFree(static_cast<CUdeviceptr>(dptr)));
  return 0;
}

struct LeadingDims {
  int64_t lda = 0, ldb = 0, ldc = 0;  // elements between rows as stored; 0 = contiguous
};
static int launch_impl(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                       uint64_t B, uint64_t C, const kcg_epilogue* epi, const uint64_t* peer_c, int n_peers, int batch,
                       const LeadingDims& ld = LeadingDims());

int kcg_launch_gemm_allgather(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                              uint64_t B, uint64_t C, const kcg_epilogue* epi, const uint64_t* peer_c, int n_peers) {
  return launch_impl(function, info, device, stream, A, B, C, epi, peer_c, n_peers, 1);
}

int kcg_launch_gemm_batched(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                            uint64_t B, uint64_t C, int batch, const kcg_epilogue* epi) {
  if (batch < 1) return fail(KCG_E_BAD_ARG, "batch must be at least 1");
  return launch_impl(function, info, device, stream, A, B, C, epi, nullptr, 0, batch);
}

int kcg_launch_gemm_strided(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                            uint64_t B, uint64_t C, int64_t lda, int64_t ldb, int64_t ldc, int batch,
                            const kcg_epilogue* epi) {
  if (batch < 1) return fail(KCG_E_BAD_ARG, "batch must be at least 1");
  if (lda < 0 || ldb < 0 || ldc < 0) return fail(KCG_E_BAD_ARG, "leading dimensions must not be negative");
  LeadingDims ld;
  ld.lda = lda;
  ld.ldb = ldb;
  ld.ldc = ldc;
  return launch_impl(function, info, device, stream, A, B, C, epi, nullptr, 0, batch, ld);
}

static int launch_impl(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream, uint64_t A,
                       uint64_t B, uint64_t C, const kcg_epilogue* epi, const uint64_t* peer_c, int n_peers, int batch,
                       const LeadingDims& ld) {
  if (!function || !info || !A || !B || !C) return fail(KCG_E_BAD_ARG, "null argument");
  if (batch > 1) {
    const bool tc = info->kernel == KCG_KERNEL_TCGEN05 || info->kernel == KCG_KERNEL_TCGEN05_PAIR ||
                    info->kernel == KCG_KERNEL_TF32X1 || info->kernel == KCG_KERNEL_TCGEN05_CLUSTERK;
    if (!tc) return fail(KCG_E_BAD_CONFIG, "batched launches need a tcgen05 kernel (KERNEL_VARIANT 2, 3, 4 or 5)");
    if (static_cast<int64_t>(info->m) * batch > 0x7fffffff || static_cast<int64_t>(info->k) * batch > 0x7fffffff)
      return fail(KCG_E_TOO_LARGE, "batch * M and batch * K must fit 31 bits");
  }
  if (n_peers < 0 || n_peers > KCG_MAX_PEERS || (n_peers > 0 && !peer_c))
    return fail(KCG_E_BAD_ARG, "n_peers must be 0..%d with their addresses", KCG_MAX_PEERS);
  if (n_peers > 0) {
    const bool staged = (info->kernel == KCG_KERNEL_TCGEN05 && info->dtype != KCG_DTYPE_FLOAT32) ||
                        (info->kernel == KCG_KERNEL_TCGEN05_PAIR && info->dtype != KCG_DTYPE_FLOAT32) ||
                        info->kernel == KCG_KERNEL_TF32X1;
    if (!staged)
      return fail(KCG_E_BAD_CONFIG, "the fused all-gather needs a single-pass tcgen05 kernel (bf16 / fp16)");
    for (int i = 0; i < n_peers; ++i)
      if (!peer_c[i] || peer_c[i] % 16) return fail(KCG_E_BAD_ARG, "peer address %d is null or not 16-byte aligned", i);
  }
  if (epi && (epi->bias % 16) != 0) return fail(KCG_E_BAD_ARG, "bias must be 16-byte aligned");
  if (epi && info->kernel == KCG_KERNEL_WAIT_PROBE) return fail(KCG_E_BAD_ARG, "the wait probe has no epilogue");
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  // Held up to the launch: the stream's slot (status, workspace, counters) and the tensor-map
  // cache must not move under a launch another thread is putting together.
  std::lock_guard<std::mutex> guard(g_dev_mutex);
  StreamSlot* slot = nullptr;
  if (int e = slot_for(s, reinterpret_cast<CUstream>(stream), true, &slot)) return e;
  KcgGemmParams p;
  memset(&p, 0, sizeof(p));
  // A batched product runs as one tall problem: M counts the rows of all batches
  const int Mb = info->m, M = info->m * batch, N = info->n, K = info->k;
  const int eb = (info->dtype == KCG_DTYPE_FLOAT32) ? 4 : 2;
  p.A = reinterpret_cast<const void*>(A);
  p.B = reinterpret_cast<const void*>(B);
  p.C = reinterpret_cast<void*>(C);
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch_rows = batch > 1 ? Mb : 0;
  // Rows as stored: A is M x K (K x M when IS_ATRANS), B is K x N (N x K when compiled with b_trans),
  // C is M x N. A leading dimension larger than the row length addresses a sub-matrix of a wider
  // array; in a batched launch the batches still follow one another row after row at that pitch.
  const int btrans = info->reserved[1] ? 1 : 0;
  const int dtype_c = info->reserved[3] ? info->reserved[3] : info->dtype;  // C may be float32 over 16-bit operands
  const int eb_c = (dtype_c == KCG_DTYPE_FLOAT32) ? 4 : 2;
  const int64_t row_a = info->atrans ? Mb : K, row_b = btrans ? K : N, row_c = N;
  const int64_t lda = ld.lda ? ld.lda : row_a, ldb = ld.ldb ? ld.ldb : row_b, ldc = ld.ldc ? ld.ldc : row_c;
  if (lda < row_a || ldb < row_b || ldc < row_c)
    return fail(KCG_E_BAD_ARG, "leading dimensions %lld, %lld, %lld are below the row lengths %lld, %lld, %lld",
                (long long)lda, (long long)ldb, (long long)ldc, (long long)row_a, (long long)row_b, (long long)row_c);
  if (lda > 0x7fffffff || ldb > 0x7fffffff || ldc > 0x7fffffff)
    return fail(KCG_E_TOO_LARGE, "leading dimensions must fit 31 bits");
  if ((lda * eb) % 16 || (ldb * eb) % 16 || (ldc * eb_c) % 16)
    return fail(KCG_E_BAD_ARG, "leading dimensions must keep every row 16-byte aligned");
  if ((ld.lda || ld.ldb || ld.ldc) && n_peers > 0)
    return fail(KCG_E_BAD_ARG, "the fused all-gather takes contiguous operands");
  p.lda = static_cast<int>(lda);
  p.ldb = static_cast<int>(ldb);
  p.ldc = static_cast<int>(ldc);
  p.status = reinterpret_cast<unsigned int*>(slot->status);
  p.split_first_tile = (M / (info->bm > 0 ? info->bm : 1)) * (N / (info->bn > 0 ? info->bn : 1));
  p.split_factor = 1;
  p.alpha = 1.f;
  if (epi) {
    p.alpha = epi->alpha;
    p.beta = epi->beta;
    p.bias = reinterpret_cast<const void*>(epi->bias);
    p.epi_flags = ((epi->alpha != 1.f || epi->beta != 0.f) ? KCG_EPI_SCALE : 0u) | (epi->bias ? KCG_EPI_BIAS : 0u) |
                  (epi->relu ? KCG_EPI_RELU : 0u);
  }
  p.n_peers = n_peers;
  for (int i = 0; i < n_peers; ++i) p.peerC[i] = reinterpret_cast<void*>(peer_c[i]);
  int grid0 = info->grid[0];
  const bool pair = info->kernel == KCG_KERNEL_TCGEN05_PAIR;
  // Tensor maps of A and B for a tcgen05 kernel whose per-CTA operand slices have layout L.
  auto encode_operands = [&](const kcg::TcLayout& L) -> int {
    if (info->atrans) {
      // K x M storage: the batches' matrices lie one under the other, K rows each
      if (int e = encode_map(s, &p.tmA, info->dtype, A, Mb, static_cast<uint64_t>(K) * batch,
                             static_cast<uint64_t>(lda) * eb, L.a_box_inner, L.a_box_outer, L.a_tma_swizzle))
        return e;
    } else {
      if (int e = encode_map(s, &p.tmA, info->dtype, A, K, M, static_cast<uint64_t>(lda) * eb, L.a_box_inner,
                             L.a_box_outer, L.a_tma_swizzle))
        return e;
    }
    if (btrans)  // N x K storage: the batches' matrices lie one under the other, N rows each
      return encode_map(s, &p.tmB, info->dtype, B, K, static_cast<uint64_t>(N) * batch,
                        static_cast<uint64_t>(ldb) * eb, L.b_box_inner, L.b_box_outer, L.b_tma_swizzle);
    return encode_map(s, &p.tmB, info->dtype, B, N, static_cast<uint64_t>(K) * batch, static_cast<uint64_t>(ldb) * eb,
                      L.b_box_inner, L.b_box_outer, L.b_tma_swizzle);
  };
  if (info->kernel == KCG_KERNEL_TCGEN05_CLUSTERK) {
    // One cluster per tile; the K split and its reduction stay inside the cluster (no workspace).
    if (int e = encode_operands(kcg::make_tc_layout(info->dtype, info->bm, info->bn, info->bk, info->atrans))) return e;
    grid0 = (M / info->bm) * (N / info->bn) * info->splitk;
  }
  if (info->kernel == KCG_KERNEL_TCGEN05 || info->kernel == KCG_KERNEL_TF32X1 || pair) {
    // the pair kernel loads per-CTA slices: BM/2 rows of A, BN/2 columns of B
    if (int e = encode_operands(pair ? kcg::make_tc_layout(info->dtype, info->bm / 2, info->bn / 2, info->bk,
                                                           info->atrans, btrans)
                                     : kcg::make_tc_layout(info->dtype, info->bm, info->bn, info->bk, info->atrans,
                                                           btrans)))
      return e;
    // The single-pass kernel writes C with TMA stores of 32-row x 128-byte boxes taken from
    // 128B-swizzled staging buffers; the 3xTF32 kernel stores from registers.
    const bool x3 = eb == 4 && info->kernel != KCG_KERNEL_TF32X1;
    if (!x3) {
      if (int e = encode_map(s, &p.tmC, dtype_c, C, N, M, static_cast<uint64_t>(ldc) * eb_c, 128 / eb_c, 32,
                             3 /*CU_TENSOR_MAP_SWIZZLE_128B*/))
        return e;
    }
    const SplitPlan plan = plan_split(info, p.epi_flags != 0u, batch);
    const int T = plan.tiles, first = plan.first, factor = plan.factor, sk_per = plan.sk_per,
              sk_ranges = plan.sk_ranges, G = plan.units_at_once;
    const bool ws_epilogue = x3 && p.epi_flags != 0u;
    // Under stream-K the whole tiles before the tail are walked with the grid as stride: the grid
    // stays at every unit that runs at once even when the tail is cut into fewer ranges (the CTAs
    // beyond the last range then simply have no tail piece).
    const int units = sk_per > 0 ? (first > 0 ? G : sk_ranges) : first + (T - first) * factor;
    grid0 = (units < G ? units : G) * (pair ? 2 : 1);
    p.split_first_tile = first;
    p.split_factor = factor;
    p.sk_per = sk_per;
    p.split_units_first = plan.units_first;
    if (factor > 1 || ws_epilogue || sk_per > 0) {
      // slots: one per (tile, split) of an even split; range index + tile index under stream-K
      const size_t slots = sk_per > 0 ? static_cast<size_t>(sk_ranges) + (T - first)
                                      : static_cast<size_t>(T - first) * factor;
      const size_t need = slots * info->bm * info->bn * sizeof(float);
      if (slot->ws_bytes < need) {
        s->tmaps.clear();  // drops the maps of the workspace that is about to move
        if (int e = grow(&slot->ws, &slot->ws_bytes, need)) return e;
      }
      const size_t tiles = static_cast<size_t>(T - first) * (pair ? 2 : 1);  // one counter per CTA half
      if (slot->counters_n < tiles) {
        size_t have = slot->counters_n * 4;
        slot->counters_n = 0;
        if (int e = grow(&slot->counters, &have, tiles * 4)) return e;
        slot->counters_n = tiles;
        DRV(cuMemsetD32(slot->counters, 0, tiles));
      }
      p.splitk_ws = reinterpret_cast<float*>(slot->ws);
      p.tile_counters = reinterpret_cast<unsigned int*>(slot->counters);
    }
    if (!x3 && (factor > 1 || sk_per > 0)) {
      // The single-pass kernel writes its partial tiles with TMA stores: the workspace as one tall
      // fp32 matrix of BN columns (every row the buffer holds, so that the map is reused while the
      // buffer is), 32 x 32 boxes with the 128B swizzle of the staging buffers.
      const uint64_t row_bytes = static_cast<uint64_t>(info->bn) * 4;
      if (int e = encode_map(s, &p.tmWs, KCG_DTYPE_FLOAT32, static_cast<uint64_t>(slot->ws), info->bn,
                             slot->ws_bytes / row_bytes, row_bytes, 32, 32, 3))
        return e;
    }
  }
  void* args[1] = {&p};
  CUlaunchConfig cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDimX = grid0;
  cfg.gridDimY = info->grid[1];
  cfg.gridDimZ = info->grid[2];
  cfg.blockDimX = info->block[0];
  cfg.blockDimY = info->block[1];
  cfg.blockDimZ = info->block[2];
  cfg.sharedMemBytes = info->smem_bytes;
  cfg.hStream = reinterpret_cast<CUstream>(stream);
  CUlaunchAttribute attr[2];
  cfg.numAttrs = 0;
  cfg.attrs = attr;
  if (info->cluster[0] * info->cluster[1] * info->cluster[2] > 1) {
    attr[cfg.numAttrs].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr[cfg.numAttrs].value.clusterDim.x = info->cluster[0];
    attr[cfg.numAttrs].value.clusterDim.y = info->cluster[1];
    attr[cfg.numAttrs].value.clusterDim.z = info->cluster[2];
    ++cfg.numAttrs;
  }
  // Programmatic dependent launch for the kernels that guard their global-memory accesses with
  // griddepcontrol.wait (every tcgen05 kernel; not the SIMT comparison kernel): after another such
  // launch in the same stream, the CTAs of this one are brought onto SMs as that kernel's CTAs leave,
  // set themselves up and wait there for its completion, instead of being launched only then.
  // KCG_PDL=0 turns it off.
  {
    static const bool pdl_on = [] {
      const char* e = getenv("KCG_PDL");
      return !(e && e[0] == '0');
    }();
    const bool guarded = info->kernel == KCG_KERNEL_TCGEN05 || info->kernel == KCG_KERNEL_TCGEN05_PAIR ||
                         info->kernel == KCG_KERNEL_TF32X1 || info->kernel == KCG_KERNEL_TCGEN05_CLUSTERK;
    if (pdl_on && guarded) {
      attr[cfg.numAttrs].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
      attr[cfg.numAttrs].value.programmaticStreamSerializationAllowed = 1;
      ++cfg.numAttrs;
    }
  }
  DRV(cuLaunchKernelEx(&cfg, reinterpret_cast<CUfunction>(function), args, nullptr));
  g_launches.fetch_add(1);
  return 0;
}

// Reads (and clears) the status block of a stream's slot after synchronising the stream.
// Call with g_dev_mutex held.
static int read_status(StreamSlot* sl) {
  unsigned int st[4] = {0, 0, 0, 0};
  DRV(cuMemcpyDtoH(st, sl->status, sizeof(st)));
  if (st[0] != 0) {
    DRV(cuMemsetD32(sl->status, 0, 4));
    // a timed-out split-K launch may leave counters mid-count
    if (sl->counters) DRV(cuMemsetD32(sl->counters, 0, sl->counters_n));
    static const char* role[] = {"", "TMA producer", "MMA issuer", "epilogue", "splitter", "shape", "push warp"};
    return fail(KCG_E_DEVICE_TIMEOUT, "kernel gave up in a bounded wait: role %s (code %u), block %u, detail %u/%u",
                st[0] < 7 ? role[st[0]] : "?", st[0], st[1], st[2], st[3]);
  }
  return 0;
}

int kcg_check_status(int device, uint64_t stream) {
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  DRV(cuStreamSynchronize(reinterpret_cast<CUstream>(stream)));
  std::lock_guard<std::mutex> guard(g_dev_mutex);
  StreamSlot* sl = nullptr;
  if (int e = slot_for(s, reinterpret_cast<CUstream>(stream), false, &sl)) return e;
  if (!sl) return 0;  // nothing was ever launched on this stream
  return read_status(sl);
}

int kcg_matmul_host(uint64_t function, const kcg_kernel_info* info, int device, uint64_t stream,
                    const void* hostA, const void* hostB, void* hostC) {
  if (!info || !hostA || !hostB || !hostC) return fail(KCG_E_BAD_ARG, "null argument");
  DeviceState* s = nullptr;
  if (int e = ensure_device(device, &s)) return e;
  const size_t eb = (info->dtype == KCG_DTYPE_FLOAT32) ? 4 : 2;
  const size_t eb_c = (info->reserved[3] == KCG_DTYPE_FLOAT32) ? 4 : eb;
  const size_t bytes[3] = {static_cast<size_t>(info->m) * info->k * eb, static_cast<size_t>(info->k) * info->n * eb,
                           static_cast<size_t>(info->m) * info->n * eb_c};
  {
    std::lock_guard<std::mutex> g(g_dev_mutex);
    for (int i = 0; i < 3; ++i)
      if (int e = grow(&s->hbuf[i], &s->hbuf_bytes[i], bytes[i])) return e;
  }
  CUstream st = reinterpret_cast<CUstream>(stream);
  // Row slabs of A / C move through three streams (copy-in, compute, copy-out) so that the
  // transfers in both directions and the kernels overlap; B goes in first. Tiles do not straddle
  // slabs: a slab is a multiple of BLOCK_SIZE_M rows.
  const int bm = info->bm > 0 ? info->bm : 1;
  const int tiles_m = info->m / bm;
  const bool tensor_core = info->kernel == KCG_KERNEL_TCGEN05 || info->kernel == KCG_KERNEL_TF32X1 ||
                           info->kernel == KCG_KERNEL_TCGEN05_PAIR;
  int nslabs = 1;
  if (tensor_core && !info->atrans && bytes[0] + bytes[2] >= (64u << 20) && tiles_m >= 4) {
    // up to 16 slabs, none smaller than ~16 MiB of A + C: what is not overlapped is the first
    // slab's copy-in and the last slab's kernel and copy-out, so more slabs shorten both ends
    size_t want = (bytes[0] + bytes[2]) / (16u << 20);
    if (want < 4) want = 4;
    if (want > 16) want = 16;
    nslabs = tiles_m < static_cast<int>(want) ? tiles_m : static_cast<int>(want);
  }
  // The kernels report an expired wait to the status block of the stream they ran on.
  auto kernel_status = [&](CUstream ran_on) -> int {
    std::lock_guard<std::mutex> g(g_dev_mutex);
    StreamSlot* sl = nullptr;
    if (int e = slot_for(s, ran_on, false, &sl)) return e;
    return sl ? read_status(sl) : 0;
  };
  if (nslabs == 1) {
    DRV(cuMemcpyHtoDAsync(s->hbuf[0], hostA, bytes[0], st));
    DRV(cuMemcpyHtoDAsync(s->hbuf[1], hostB, bytes[1], st));
    int rc = kcg_launch_gemm(function, info, device, stream, s->hbuf[0], s->hbuf[1], s->hbuf[2]);
    if (rc == 0) {
      const CUresult r = driver().p_cuMemcpyDtoHAsync(hostC, s->hbuf[2], bytes[2], st);
      if (r != CUDA_SUCCESS) rc = drv_fail(r, "cuMemcpyDtoHAsync");
    }
    // also on an error path: nothing of this call is left in flight on the caller's buffers
    const CUresult rs = driver().p_cuStreamSynchronize(st);
    if (rc == 0 && rs != CUDA_SUCCESS) rc = drv_fail(rs, "cuStreamSynchronize");
    return rc ? rc : kernel_status(st);
  }
  {
    std::lock_guard<std::mutex> g(g_dev_mutex);
    for (int i = 0; i < 3; ++i)
      if (!s->hstream[i]) DRV(cuStreamCreate(&s->hstream[i], CU_STREAM_NON_BLOCKING));
    while (s->hevents.size() < static_cast<size_t>(2 * nslabs + 2)) {
      CUevent ev;
      DRV(cuEventCreate(&ev, CU_EVENT_DISABLE_TIMING));
      s->hevents.push_back(ev);
    }
  }
  CUstream s_in = s->hstream[0], s_exec = s->hstream[1], s_out = s->hstream[2];
  CUevent ev_begin = s->hevents[2 * nslabs], ev_end = s->hevents[2 * nslabs + 1];
  // Every step of the pipeline runs through `step`; after the first failure the rest is skipped
  // and the three internal streams are drained before the error is returned, so that no copy or
  // kernel of this call still touches the caller's buffers (or the library's) afterwards.
  int rc = 0;
  auto step = [&](CUresult r, const char* what) {
    if (rc == 0 && r != CUDA_SUCCESS) rc = drv_fail(r, what);
    return rc == 0;
  };
  Driver& d = driver();
  step(d.p_cuEventRecord(ev_begin, st), "cuEventRecord");  // work already queued on the caller's stream comes first
  if (rc == 0) step(d.p_cuStreamWaitEvent(s_in, ev_begin, 0), "cuStreamWaitEvent");
  if (rc == 0) step(d.p_cuStreamWaitEvent(s_exec, ev_begin, 0), "cuStreamWaitEvent");
  if (rc == 0) step(d.p_cuStreamWaitEvent(s_out, ev_begin, 0), "cuStreamWaitEvent");
  if (rc == 0) step(d.p_cuMemcpyHtoDAsync(s->hbuf[1], hostB, bytes[1], s_in), "cuMemcpyHtoDAsync(B)");
  const int base_tiles = tiles_m / nslabs, extra = tiles_m % nslabs;
  size_t row0 = 0;
  for (int i = 0; i < nslabs && rc == 0; ++i) {
    const size_t rows = static_cast<size_t>(base_tiles + (i < extra ? 1 : 0)) * bm;
    const size_t a_off = row0 * info->k * eb, c_off = row0 * info->n * eb_c;
    if (!step(d.p_cuMemcpyHtoDAsync(s->hbuf[0] + a_off, static_cast<const char*>(hostA) + a_off, rows * info->k * eb,
                                    s_in), "cuMemcpyHtoDAsync(A)"))
      break;
    if (!step(d.p_cuEventRecord(s->hevents[2 * i], s_in), "cuEventRecord")) break;
    if (!step(d.p_cuStreamWaitEvent(s_exec, s->hevents[2 * i], 0), "cuStreamWaitEvent")) break;
    kcg_kernel_info slab = *info;  // same cubin: the kernels take M from the launch parameters
    slab.m = static_cast<int32_t>(rows);
    rc = kcg_launch_gemm(function, &slab, device, reinterpret_cast<uint64_t>(s_exec), s->hbuf[0] + a_off, s->hbuf[1],
                         s->hbuf[2] + c_off);
    if (rc != 0) break;
    if (!step(d.p_cuEventRecord(s->hevents[2 * i + 1], s_exec), "cuEventRecord")) break;
    if (!step(d.p_cuStreamWaitEvent(s_out, s->hevents[2 * i + 1], 0), "cuStreamWaitEvent")) break;
    if (!step(d.p_cuMemcpyDtoHAsync(static_cast<char*>(hostC) + c_off, s->hbuf[2] + c_off, rows * info->n * eb_c, s_out),
              "cuMemcpyDtoHAsync(C)"))
      break;
    row0 += rows;
  }
  if (rc == 0) step(d.p_cuEventRecord(ev_end, s_out), "cuEventRecord");
  if (rc == 0) step(d.p_cuStreamWaitEvent(st, ev_end, 0), "cuStreamWaitEvent");
  // drain (also after a failure)
  const CUresult r_in = d.p_cuStreamSynchronize(s_in), r_exec = d.p_cuStreamSynchronize(s_exec),
                 r_out = d.p_cuStreamSynchronize(s_out), r_st = d.p_cuStreamSynchronize(st);
  step(r_in, "cuStreamSynchronize");
  step(r_exec, "cuStreamSynchronize");
  step(r_out, "cuStreamSynchronize");
  step(r_st, "cuStreamSynchronize");
  return rc ? rc : kernel_status(s_exec);
}

int kcg_shutdown(void) {
  Driver& d = driver();
  if (!d.ok) return 0;
  std::lock_guard<std::mutex> g(g_dev_mutex);
  for (int i = 0; i < kMaxDevices; ++i) {
    DeviceState& s = g_dev[i];
    if (!s.init) continue;
    d.p_cuCtxSetCurrent(s.ctx);
    for (StreamSlot& sl : s.slots) {
      if (sl.status) d.p_cuMemFree(sl.status);
      if (sl.ws) d.p_cuMemFree(sl.ws);
      if (sl.counters) d.p_cuMemFree(sl.counters);
    }
    for (int j = 0; j < 3; ++j) {
      if (s.hbuf[j]) d.p_cuMemFree(s.hbuf[j]);
      if (s.hstream[j]) d.p_cuStreamDestroy(s.hstream[j]);
    }
    for (CUevent ev : s.hevents) d.p_cuEventDestroy(ev);
    s = DeviceState();
  }
  return 0;
}

}  // extern "C"
