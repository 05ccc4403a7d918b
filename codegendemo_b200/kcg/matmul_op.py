"""Convenience wrappers over the reference-style flow
``KernelArgMatmul -> KCGCompiler.compileKernel -> UserInputs -> CompiledKernelFactory.getKernel``
(the sequence of SerialCompileTask._task_compile_kernel, Runtime/python/kcg/KCGTask.py:275-297)."""
from codegendemo_b200.kcg.CompiledKernelFactory import CompiledKernelFactory, EnumOperator, UserInputs
from codegendemo_b200.kcg.KCGCompiler import KCGCompiler
from codegendemo_b200.kcg.Operators.matmul import KernelArgMatmul
from codegendemo_b200.kcg.Utils import EnumKernelDType, FromTorchType


def default_config(M: int, N: int, K: int, dtype: EnumKernelDType, **keys) -> KernelArgMatmul:
    """A tensor-core config for the NN case (A is M x K row-major) with sensible B200 defaults;
    any tuning key can be overridden by keyword (attribute names of KernelArgMatmul)."""
    kpm = KernelArgMatmul(M, N, K, dtype, dtype, dtype)
    eb = int(dtype) % 30
    kpm.BLOCK_SIZE_M = 128
    kpm.BLOCK_SIZE_N = 256 if N % 256 == 0 else 128 if N % 128 == 0 else 64
    kpm.BLOCK_SIZE_K = 128 // eb
    kpm.THREAD_SIZE_M, kpm.THREAD_SIZE_N = 8, kpm.BLOCK_SIZE_N // 16
    kpm.WARP_SIZE = 32
    kpm.WARP_LAYOUT_M, kpm.WARP_LAYOUT_N = 4, 8
    kpm.BLOCK_LAYOUT_M, kpm.BLOCK_LAYOUT_N = 4, 2
    kpm.isATranspose = 0
    kpm.LOCAL_SPLIT_U = 1
    kpm.BLOCK_MAPPING = 8
    kpm.SHARED_PREFETCH = 1
    kpm.REG_PREFETCH = 1
    kpm.GLOB_LOAD_WIDTH_A = kpm.GLOB_LOAD_WIDTH_B = kpm.GLOB_STORE_WIDTH = 4
    kpm.WARP_SCATTER_WIDTH_A = kpm.THREAD_SCATTER_WIDTH_A = kpm.THREAD_SIZE_M
    kpm.WARP_SCATTER_WIDTH_B = kpm.THREAD_SCATTER_WIDTH_B = kpm.THREAD_SIZE_N
    kpm.UNROLL_NUM = 4
    for k, v in keys.items():
        if not hasattr(kpm, k):
            raise KeyError(f"unknown tuning key {k}")
        setattr(kpm, k, v)
    return kpm


def tuned_config(M: int, N: int, K: int, dtype: EnumKernelDType, isATranspose: int = 0, db=None) -> KernelArgMatmul:
    """Best known config of a shape: the kernel database's entry when the shape was tuned, else a
    rule of thumb from the B200 measurements (CTA-pair kernels once their larger tiles still fill
    the 74 pairs for several waves, single-CTA 256x256 / 128x256 tiles otherwise)."""
    from codegendemo_b200.kcg.InfoDb import KernelDb
    db = db if db is not None else KernelDb()
    hit = db.lookup(M, N, K, int(dtype), isATranspose)
    if hit is not None:
        return KernelArgMatmul.fromJson(hit["config"])
    pairs = 74
    if int(dtype) == int(EnumKernelDType.float32):
        if M % 256 == 0 and N % 256 == 0 and K % 32 == 0 and (M // 256) * (N // 256) >= pairs:
            return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256,
                                  BLOCK_SIZE_K=32, NUM_STAGES=3, isATranspose=isATranspose)
        if N % 256 == 0 and K % 16 == 0:
            return default_config(M, N, K, dtype, BLOCK_SIZE_N=256, BLOCK_SIZE_K=16, NUM_STAGES=4,
                                  isATranspose=isATranspose)
        return default_config(M, N, K, dtype, BLOCK_SIZE_N=128 if N % 128 == 0 else 64, isATranspose=isATranspose)
    if M % 512 == 0 and N % 256 == 0 and K % 64 == 0 and (M // 512) * (N // 256) >= 6 * pairs:
        return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64,
                              NUM_STAGES=4, isATranspose=isATranspose)
    tiles256 = (M // 256) * (N // 256) if M % 256 == 0 and N % 256 == 0 else 0
    if K <= 512 and K % 64 == 0 and N % 256 == 0:
        # short K: the epilogue weighs as much as the main loop, so take the tile whose two TMEM accumulator
        # buffers overlap them (batched 256 x (256x256x256): 489 vs 405 TFLOP/s with the pair tile)
        return default_config(M, N, K, dtype, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, isATranspose=isATranspose)
    if K % 64 == 0 and pairs <= tiles256 < 6 * pairs:
        # one to six waves of 256x256 pair tiles: the pair kernel with a stream-K tail measured best on the
        # rectangular shapes (512 and 2048 rows x 11008^2), with 128-wide K blocks once K is long
        return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256,
                              BLOCK_SIZE_K=128 if (K % 128 == 0 and K >= 8192) else 64, isATranspose=isATranspose)
    if K % 64 == 0 and tiles256 >= 148:
        return default_config(M, N, K, dtype, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, NUM_STAGES=3,
                              isATranspose=isATranspose)
    if N % 128 == 0 and K % 128 == 0 and K >= 1024:
        # few tiles: small tiles with long K blocks (best on the 128- and 512-row shapes)
        return default_config(M, N, K, dtype, BLOCK_SIZE_N=128, BLOCK_SIZE_K=128, isATranspose=isATranspose)
    return default_config(M, N, K, dtype, isATranspose=isATranspose)


def build_kernel(kpm: KernelArgMatmul, deviceId: int = 0):
    """Compile (or fetch from the cubin cache) and wrap one config; returns (UserInputs, CompiledKernel)."""
    kpm.check()
    compiler = KCGCompiler()
    path, name, gx, gy, gz, bx, by, bz = compiler.compileKernel(kpm)[0]
    inConfig = UserInputs(path, name, kpm, compiler.lastInfo)
    inConfig.m_gridDims = [gx, gy, gz]
    inConfig.m_blockDims = [bx, by, bz]
    inConfig.operatorKind = EnumOperator.Matmul
    return inConfig, CompiledKernelFactory.getKernel(inConfig, deviceId)


_KERNELS = {}


def matmul(a, b, c=None, alpha=1.0, beta=0.0, bias=None, relu=False, **keys):
    """``c = a @ b`` on the current CUDA device through the kernel database's config for the shape
    (or a default config tuned by keyword). ``alpha``, ``beta``, ``bias`` (N values of c's dtype) and
    ``relu`` fuse ``c = act(alpha * a @ b + beta * c + bias)`` into the kernel's store. Compiled and
    loaded kernels are kept per (shape, dtype, device, keys)."""
    import torch
    M, K = a.shape
    K2, N = b.shape
    assert K == K2 and a.is_contiguous() and b.is_contiguous()
    if c is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs the c to scale")
        c = torch.empty((M, N), dtype=a.dtype, device=a.device)
    dt = FromTorchType(a.dtype)
    dev = a.device.index or 0
    key = (M, N, K, int(dt), dev, tuple(sorted(keys.items())))
    kern = _KERNELS.get(key)
    if kern is None:
        kpm = default_config(M, N, K, dt, **keys) if keys else tuned_config(M, N, K, dt)
        _, kern = build_kernel(kpm, dev)
        _KERNELS[key] = kern
    kern.run(a, b, c, alpha=alpha, beta=beta, bias=bias, relu=relu)
    return c


def bmm(a, b, c=None, alpha=1.0, beta=0.0, bias=None, relu=False, **keys):
    """``c[i] = a[i] @ b[i]`` (``torch.bmm`` layout: a is batch x M x K, b is batch x K x N, both
    contiguous) as ONE launch of the kernel compiled for a single batch's M, N, K: the persistent grid
    walks the tiles of all batches, so that small per-batch problems fill the GPU together. The
    epilogue keywords are those of ``matmul`` (a bias is shared by the batches)."""
    import torch
    batch, M, K = a.shape
    batch2, K2, N = b.shape
    assert batch == batch2 and K == K2 and a.is_contiguous() and b.is_contiguous()
    if c is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs the c to scale")
        c = torch.empty((batch, M, N), dtype=a.dtype, device=a.device)
    dt = FromTorchType(a.dtype)
    dev = a.device.index or 0
    key = (M, N, K, int(dt), dev, tuple(sorted(keys.items())), 0 if keys else batch)
    kern = _KERNELS.get(key)
    if kern is None:
        if keys:
            kpm = default_config(M, N, K, dt, **keys)
        else:
            # the launch walks all batches' tiles as one tall problem: pick the tile for that much work,
            # as long as a batch holds a whole number of tile rows
            kpm = tuned_config(batch * M, N, K, dt)
            if M % kpm.BLOCK_SIZE_M:
                kpm = tuned_config(M, N, K, dt)
            kpm.M = M
        _, kern = build_kernel(kpm, dev)
        _KERNELS[key] = kern
    kern.run(a, b, c, alpha=alpha, beta=beta, bias=bias, relu=relu, batch=batch)
    return c
