"""Launch boundary: ``launchKernel(device, a, b, c)`` on torch's current stream.

Mirror of ``HIPLauncher`` (Runtime/python/kcg/HIPLauncher.py:264-314). The reference generates,
compiles (gcc) and imports one C launcher per kernel signature; here every kernel takes the same
parameter block, so one C entry (``kcg_launch_gemm``) serves all of them and builds the TMA tensor
maps itself. Pointer arguments may be ints or anything with ``data_ptr()`` (HIPLauncher.py:148-187).
"""
import ctypes

from codegendemo_b200 import _lib
from codegendemo_b200.kcg.Loader import CudaLoaderST, KernelLibFile
from codegendemo_b200.kcg.Utils import DeviceInfo


def _pointer_of(obj) -> int:
    if obj is None:
        raise TypeError("KCG launcher: pointer argument is None")
    if isinstance(obj, int):
        return obj
    ptr = getattr(obj, "data_ptr", None)
    if ptr is None:
        raise TypeError("Pointer argument must be either uint64 or have data_ptr method")
    return int(ptr())


class CudaLauncher:
    def __init__(self, kernelBinaryPath, kernelFuncName, shmSize, signature: dict, gridDims: list,
                 blockDims: list, device=0, kernelInfo: dict = None):
        self.m_libFile = KernelLibFile(kernelBinaryPath, kernelFuncName, shmSize, device)
        self.m_signature = signature
        self.m_gridDims = list(gridDims)
        self.m_blockDims = list(blockDims)
        self.m_shmSize = shmSize
        self.m_device = device
        self.m_kernelInfoDict = kernelInfo
        # loaded lazily in the process that owns the GPU (launchers are pickled across processes)
        self.m_runtime = None
        self.m_cInfo = None

    def __getstate__(self):
        st = dict(self.__dict__)
        st["m_runtime"] = None
        st["m_cInfo"] = None
        return st

    def _getWrapper(self):
        if self.m_runtime is None:
            if self.m_kernelInfoDict is None:
                raise RuntimeError("KCG launcher: kernelInfo missing (compile with KCGCompiler first)")
            info = dict(self.m_kernelInfoDict)
            info["grid"], info["block"], info["smem_bytes"] = self.m_gridDims, self.m_blockDims, self.m_shmSize
            self.m_cInfo = _lib.KernelInfo.from_dict(info)
            self.m_runtime = CudaLoaderST().loadBinary(self.m_libFile)
        return self.m_runtime

    def launchKernel(self, device, *args, stream=None, alpha=1.0, beta=0.0, bias=None, relu=False, peers=None,
                     batch=1, lda=0, ldb=0, ldc=0):
        """(a, b, c) -> c = a.b on `stream` (torch's current stream by default). The keyword
        arguments fuse c = act(alpha * a.b + beta * c + bias) into the kernel's store; `peers` (up to 7
        device addresses or tensors shaped like c) also receive every finished tile: the fused
        all-gather of an M-sharded product. The reference's launcher has no such arguments and the plain
        call behaves as the reference's."""
        rt = self._getWrapper()
        if len(args) != 3:
            raise TypeError("matmul kernel takes (a, b, c)")
        if stream is None:
            stream = DeviceInfo.get_cuda_stream(device)
        a, b, c = (_pointer_of(x) for x in args)
        lib = _lib.get_lib()
        if lda or ldb or ldc:
            # operands that are sub-matrices of wider row-major arrays: elements between rows (0 = contiguous)
            if peers:
                raise ValueError("a strided launch has no fused all-gather")
            fused = not (alpha == 1.0 and beta == 0.0 and bias is None and not relu)
            epi = _lib.Epilogue(float(alpha), float(beta), _pointer_of(bias) if bias is not None else 0,
                                int(bool(relu))) if fused else None
            _lib.check(lib.kcg_launch_gemm_strided(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                                   int(device), ctypes.c_uint64(int(stream)), ctypes.c_uint64(a),
                                                   ctypes.c_uint64(b), ctypes.c_uint64(c), int(lda), int(ldb),
                                                   int(ldc), int(batch), ctypes.byref(epi) if fused else None))
            return
        if batch != 1:
            # (a, b, c) hold `batch` contiguous problems of the kernel's M, N, K (torch.bmm layout)
            if peers:
                raise ValueError("a batched launch has no fused all-gather")
            fused = not (alpha == 1.0 and beta == 0.0 and bias is None and not relu)
            epi = _lib.Epilogue(float(alpha), float(beta), _pointer_of(bias) if bias is not None else 0,
                                int(bool(relu))) if fused else None
            _lib.check(lib.kcg_launch_gemm_batched(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                                   int(device), ctypes.c_uint64(int(stream)), ctypes.c_uint64(a),
                                                   ctypes.c_uint64(b), ctypes.c_uint64(c), int(batch),
                                                   ctypes.byref(epi) if fused else None))
            return
        if alpha == 1.0 and beta == 0.0 and bias is None and not relu and not peers:
            _lib.check(lib.kcg_launch_gemm(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                           int(device), ctypes.c_uint64(int(stream)),
                                           ctypes.c_uint64(a), ctypes.c_uint64(b), ctypes.c_uint64(c)))
            return
        epi = _lib.Epilogue(float(alpha), float(beta), _pointer_of(bias) if bias is not None else 0, int(bool(relu)))
        if peers:
            arr = (ctypes.c_uint64 * len(peers))(*[_pointer_of(x) for x in peers])
            _lib.check(lib.kcg_launch_gemm_allgather(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                                     int(device), ctypes.c_uint64(int(stream)), ctypes.c_uint64(a),
                                                     ctypes.c_uint64(b), ctypes.c_uint64(c), ctypes.byref(epi),
                                                     arr, len(peers)))
            return
        _lib.check(lib.kcg_launch_gemm_ex(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                          int(device), ctypes.c_uint64(int(stream)), ctypes.c_uint64(a),
                                          ctypes.c_uint64(b), ctypes.c_uint64(c), ctypes.byref(epi)))

    def runHost(self, device, hostA, hostB, hostC, stream=None):
        """Whole operator on host buffers (H2D, kernel, D2H, synchronise)."""
        rt = self._getWrapper()
        if stream is None:
            stream = DeviceInfo.get_cuda_stream(device)
        _lib.check(_lib.get_lib().kcg_matmul_host(ctypes.c_uint64(rt.m_function), ctypes.byref(self.m_cInfo),
                                                  int(device), ctypes.c_uint64(int(stream)),
                                                  ctypes.c_void_p(_pointer_of(hostA)),
                                                  ctypes.c_void_p(_pointer_of(hostB)),
                                                  ctypes.c_void_p(_pointer_of(hostC))))

    def checkStatus(self, device, stream=None):
        if stream is None:
            stream = DeviceInfo.get_cuda_stream(device)
        _lib.check(_lib.get_lib().kcg_check_status(int(device), ctypes.c_uint64(int(stream))))
