"""Convenience wrappers over the reference-style flow
``KernelArgMatmul -> KCGCompiler.compileKernel -> UserInputs -> CompiledKernelFactory.getKernel``
(the sequence of SerialCompileTask._task_compile_kernel, Runtime/python/kcg/KCGTask.py:275-297)."""
from codegendemo_b200.kcg.CompiledKernelFactory import CompiledKernelFactory, EnumOperator, UserInputs
from codegendemo_b200.kcg.KCGCompiler import KCGCompiler
from codegendemo_b200.kcg.Operators.matmul import KernelArgMatmul
from codegendemo_b200.kcg.Utils import EnumKernelDType, FromTorchType


def default_config(M: int, N: int, K: int, dtype: EnumKernelDType, out_dtype=None, **keys) -> KernelArgMatmul:
    """A tensor-core config for the NN case (A is M x K row-major) with sensible B200 defaults;
    any tuning key can be overridden by keyword (attribute names of KernelArgMatmul). ``out_dtype`` =
    float32 with fp16 / bf16 operands stores the fp32 accumulators unrounded."""
    kpm = KernelArgMatmul(M, N, K, dtype, dtype, dtype if out_dtype is None else out_dtype)
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
    tiles256 = (M // 256) * (N // 256) if M % 256 == 0 and N % 256 == 0 else 0
    if K <= 512 and K % 64 == 0 and N % 256 == 0:
        # short K: the epilogue weighs as much as the main loop, so take the tile whose two TMEM accumulator
        # buffers overlap them
        return default_config(M, N, K, dtype, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64, isATranspose=isATranspose)
    if M % 512 == 0 and N % 256 == 0 and K % 64 == 0 and (M // 512) * (N // 256) >= 6 * pairs:
        # six waves and more of 512x256 pair tiles: the largest tile (fewest operand bytes per flop through
        # L2), its accumulator released in halves. Measured in short bursts at full clock (how the benchmark
        # runs) it leads; under a sustained power cap the 256x256x128 tile below overtakes it by a few percent.
        return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64,
                              NUM_STAGES=4, isATranspose=isATranspose)
    if K % 128 == 0 and tiles256 >= pairs:
        # one to twelve waves of 256x256 pair tiles: CTA pairs with 128-wide K blocks (half as many stage
        # hand-offs per byte as 64-wide ones, two accumulator buffers, remainder split run first); best or within 2 % of
        # the best on every such shape measured, from 512 x 11008 x 4096 to 4096 x 8192 x 8192
        return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256,
                              BLOCK_SIZE_K=128, isATranspose=isATranspose)
    if K % 64 == 0 and tiles256 >= pairs:
        return default_config(M, N, K, dtype, KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256,
                              BLOCK_SIZE_K=64, isATranspose=isATranspose)
    pick = clusterk_choice(M, N, K)
    if pick is not None:
        # fewer 128-row tiles than SMs: K is split over the CTAs of a cluster (KERNEL_VARIANT 5, reduction in
        # shared memory) so that two to four times as many SMs stream the operands
        bn, bk, split = pick
        return default_config(M, N, K, dtype, KERNEL_VARIANT=5, BLOCK_SIZE_N=bn, BLOCK_SIZE_K=bk,
                              LOCAL_SPLIT_U=split, isATranspose=isATranspose)
    if N % 128 == 0 and K % 128 == 0 and K >= 1024:
        # few tiles: small tiles with long K blocks (best on the 128- and 512-row shapes)
        return default_config(M, N, K, dtype, BLOCK_SIZE_N=128, BLOCK_SIZE_K=128, isATranspose=isATranspose)
    return default_config(M, N, K, dtype, isATranspose=isATranspose)


def clusterk_choice(M: int, N: int, K: int, sms: int = 148):
    """(BLOCK_SIZE_N, BLOCK_SIZE_K, LOCAL_SPLIT_U) of the cluster split-K kernel for a 16-bit problem with fewer
    128-row tiles than SMs, or None when it does not apply. Of the tile widths 128 and 256, each with the largest
    split of 2..4 whose CTAs still fit one wave, the one that occupies more SMs wins; at equal count the wider
    tile (fewer operand bytes through each SM, less to exchange). Measured: 128 x 4096 x 4096 -> 128 wide, split 4;
    128 x 11008 x K -> 256 wide, split 3; 512 x 4096 x K -> 256 wide, split 2, each ahead of the whole-K kernels."""
    if M % 128 != 0 or M > 512 or K < 2048:
        return None
    best = None
    for bn, bk in ((128, 128), (256, 64)):
        if N % bn != 0 or K % bk != 0:
            continue
        tiles = (M // 128) * (N // bn)
        split = min(4, sms // tiles) if tiles > 0 else 0
        if split < 2 or (K // bk) < 4 * split:
            continue
        ctas = tiles * split
        if best is None or ctas >= best[0]:
            best = (ctas, bn, bk, split)
    return None if best is None else best[1:]


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


def _row_pitch(t, what: str) -> int:
    """Leading dimension (elements between rows) of a 2-D tensor whose rows are contiguous: a plain
    matrix or a column block / row block view of a wider row-major one."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{what} must be a 2-D tensor with contiguous rows (a view with a row pitch is fine)")
    return int(t.stride(0)) if t.shape[0] > 1 else int(t.shape[1])


def matmul(a, b, c=None, alpha=1.0, beta=0.0, bias=None, relu=False, b_transposed=False, **keys):
    """``c = a @ b`` on the current CUDA device through the kernel database's config for the shape
    (or a default config tuned by keyword). ``alpha``, ``beta``, ``bias`` (N values of c's dtype) and
    ``relu`` fuse ``c = act(alpha * a @ b + beta * c + bias)`` into the kernel's store. The operands may
    be views with a row pitch (column or row blocks of wider row-major tensors): their leading dimensions go
    to the strided launch entry, nothing is copied. ``b_transposed=True`` takes ``b`` stored N x K and computes
    ``a @ b.T`` (16-bit dtypes). Compiled and loaded kernels are kept per (shape, dtype, device, keys)."""
    import torch
    M, K = a.shape
    if b_transposed:
        N, K2 = b.shape
    else:
        K2, N = b.shape
    assert K == K2
    lda, ldb = _row_pitch(a, "a"), _row_pitch(b, "b")
    if c is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs the c to scale")
        c = torch.empty((M, N), dtype=a.dtype, device=a.device)
    ldc = _row_pitch(c, "c")
    dt = FromTorchType(a.dtype)
    dev = a.device.index or 0
    key = (M, N, K, int(dt), dev, tuple(sorted(keys.items())), bool(b_transposed))
    kern = _KERNELS.get(key)
    if kern is None:
        kpm = default_config(M, N, K, dt, **keys) if keys else tuned_config(M, N, K, dt)
        if b_transposed:
            kpm = _single_pass_16bit(kpm, M, N, K, dt)
            kpm.IS_BTRANS = 1
        _, kern = build_kernel(kpm, dev)
        _KERNELS[key] = kern
    contiguous = lda == K and ldb == (K if b_transposed else N) and ldc == N
    if contiguous:
        kern.run(a, b, c, alpha=alpha, beta=beta, bias=bias, relu=relu)
    else:
        kern.run(a, b, c, alpha=alpha, beta=beta, bias=bias, relu=relu, lda=lda, ldb=ldb, ldc=ldc)
    return c


def _single_pass_16bit(kpm, M, N, K, dt):
    """An N x K stored B runs on the single-pass tcgen05 kernels (variants 2 and 4) only: keep a tuned config of
    those families, else fall back to the default tile."""
    if kpm.KERNEL_VARIANT in (2, 4) or (kpm.KERNEL_VARIANT == 0 and kpm.usesTensorCores()):
        if kpm.KERNEL_VARIANT == 0:
            kpm.KERNEL_VARIANT = 2
        return kpm
    return default_config(M, N, K, dt, KERNEL_VARIANT=2)


def attention(q, k, v, scale=None, out=None):
    """``softmax(scale * q @ k^T) @ v`` per head, the attention-shaped chain, as three launches on the current
    stream: a batched product with k taken as stored (keys x head_dim, no transposed copy) whose epilogue applies
    ``scale`` and which stores the scores as fp32; a row softmax (fp32 arithmetic) from the scores into
    probabilities of the inputs' dtype; a batched product with v. ``q`` is (heads, Sq, d), ``k`` and ``v`` are
    (heads, Sk, d), all contiguous fp16 / bf16; ``heads`` may be batch * heads flattened. The Sq x Sk score and
    probability matrices are materialised; Sk must be a multiple of 8. Returns (heads, Sq, d)."""
    import ctypes
    import math
    import torch
    from codegendemo_b200 import _lib
    from codegendemo_b200.kcg.Utils import DeviceInfo
    H, Sq, D = q.shape
    H2, Sk, D2 = k.shape
    assert H == H2 and D == D2 and tuple(v.shape) == (H, Sk, D)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dt = FromTorchType(q.dtype)
    dev = q.device.index or 0
    key = ("attn", H, Sq, Sk, D, int(dt), dev)
    kerns = _KERNELS.get(key)
    if kerns is None:
        def tile_for(m, n, kk, scores_step):
            kpm = tuned_config(H * m, n, kk, dt)
            if m % kpm.BLOCK_SIZE_M or kpm.KERNEL_VARIANT not in (0, 2, 4):
                kpm = default_config(m, n, kk, dt)
            kpm.M = m
            if scores_step:
                # q k^T with k as stored; the scores leave as fp32: rounded to 16 bits first, their error
                # (up to 2^-9 of a score of several units) would be amplified by the softmax's exp
                kpm = _single_pass_16bit(kpm, m, n, kk, dt)
                kpm.IS_BTRANS = 1
                kpm.setOutputDtype(EnumKernelDType.float32)
            return build_kernel(kpm, dev)[1]
        kerns = (tile_for(Sq, Sk, D, True), tile_for(Sq, D, Sk, False))
        _KERNELS[key] = kerns
    scores = torch.empty((H, Sq, Sk), dtype=torch.float32, device=q.device)
    probs = torch.empty((H, Sq, Sk), dtype=q.dtype, device=q.device)
    if out is None:
        out = torch.empty((H, Sq, D), dtype=q.dtype, device=q.device)
    kerns[0].run(q, k, scores, alpha=float(scale), batch=H)
    _lib.check(_lib.get_lib().kcg_softmax_rows_ex(dev, ctypes.c_uint64(DeviceInfo.get_cuda_stream(dev)),
                                                  ctypes.c_uint64(scores.data_ptr()), int(EnumKernelDType.float32), 0,
                                                  ctypes.c_uint64(probs.data_ptr()), int(dt), 0, H * Sq, Sk, 1.0))
    kerns[1].run(probs, v, out, batch=H)
    return out


def attention_fused(q, k, v, scale=None, out=None):
    """``softmax(scale * q @ k^T) @ v`` per head as ONE kernel (``kcg_attention_fwd``): scores and probabilities
    stay in tensor memory and shared memory. ``q`` is (heads, Sq, d), ``k`` and ``v`` are (heads, Sk, d), all
    contiguous fp16 / bf16 with d = 64 or 128; any Sq and Sk. Returns (heads, Sq, d). ``attention`` above is the
    three-launch form of the same chain."""
    import ctypes
    import math
    import torch
    from codegendemo_b200 import _lib
    from codegendemo_b200.kcg.Utils import DeviceInfo
    H, Sq, D = q.shape
    H2, Sk, D2 = k.shape
    assert H == H2 and D == D2 and tuple(v.shape) == (H, Sk, D)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((H, Sq, D), dtype=q.dtype, device=q.device)
    assert out.is_contiguous() and tuple(out.shape) == (H, Sq, D) and out.dtype == q.dtype
    dev = q.device.index or 0
    u64 = ctypes.c_uint64
    _lib.check(_lib.get_lib().kcg_attention_fwd(dev, u64(DeviceInfo.get_cuda_stream(dev)), u64(q.data_ptr()),
                                                u64(k.data_ptr()), u64(v.data_ptr()), u64(out.data_ptr()),
                                                int(FromTorchType(q.dtype)), H, Sq, Sk, D, float(scale)))
    return out


def attention_status(device: int = 0) -> None:
    """Synchronises the device and raises if a bounded wait of the fused attention kernel ran out."""
    import ctypes
    from codegendemo_b200 import _lib
    out = (ctypes.c_uint32 * 4)()
    _lib.check(_lib.get_lib().kcg_attention_status(int(device), out))


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
