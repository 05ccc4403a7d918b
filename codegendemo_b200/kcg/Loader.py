"""Load boundary: cubin file -> (module, function, n_regs, n_spills).

Mirror of ``HIPLoaderST`` (Runtime/python/kcg/Loader.py:64-105), whose C extension
(loaderCCode/hip.c:60-133) is replaced by ``kcg_load_binary`` / ``kcg_device_properties`` of
libkcg_b200.so (CUDA driver API). Singleton, like the reference's.
"""
import ctypes

from codegendemo_b200 import _lib


class KernelLibFile:
    """What the loader needs to know about one compiled kernel (cf. Kernel.py:52-84)."""

    def __init__(self, filePath: str, kernelFuncName: str, shmSize: int, device: int):
        self.m_filePath = filePath
        self.m_kernelFuncName = kernelFuncName
        self.m_shmSize = shmSize
        self.m_device = device


class KernelRuntimeInfo:
    """Process-lifetime handles, stored as integers (cf. Kernel.py:44-49)."""

    def __init__(self, module: int, func: int, regs: int, spills: int):
        self.m_module = module
        self.m_function = func
        self.m_regs = regs
        self.m_spills = spills


class CudaLoaderST(object):
    def __new__(cls):
        if not hasattr(cls, 'instance'):
            cls.instance = super(CudaLoaderST, cls).__new__(cls)
        return cls.instance

    def __init__(self):
        self._lib = _lib.get_lib()

    def loadBinary(self, info: KernelLibFile) -> KernelRuntimeInfo:
        mod, fn = ctypes.c_uint64(0), ctypes.c_uint64(0)
        regs, spills = ctypes.c_int32(0), ctypes.c_int32(0)
        _lib.check(self._lib.kcg_load_binary(info.m_kernelFuncName.encode(), info.m_filePath.encode(),
                                             int(info.m_shmSize), int(info.m_device), ctypes.byref(mod),
                                             ctypes.byref(fn), ctypes.byref(regs), ctypes.byref(spills)))
        return KernelRuntimeInfo(mod.value, fn.value, regs.value, spills.value)

    def unload(self, rt: KernelRuntimeInfo) -> None:
        _lib.check(self._lib.kcg_unload(ctypes.c_uint64(rt.m_module)))

    def get_device_properties(self, device: int) -> dict:
        p = _lib.DeviceProps()
        _lib.check(self._lib.kcg_device_properties(int(device), ctypes.byref(p)))
        return {name: int(getattr(p, name)) for name, _ in p._fields_}


def is_hip() -> bool:
    return False
