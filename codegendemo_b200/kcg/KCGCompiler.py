"""Compile boundary: tuning config -> cubin on disk + kernel name + launch dims.

Mirror of Runtime/python/kcg/KCGCompiler.py:6-44. The reference imports a CPython module
(``compile_kernel_matmul`` in bin/libkcg_compiler.so, src/main.cc:315-357) that runs MLIR -> AMDGCN;
here the same call goes to ``kcg_compile_matmul_ex`` of libkcg_b200.so, which runs nvcc for sm_100a.
Needs no GPU, so it is safe in compile worker processes.
"""
import ctypes

from codegendemo_b200 import _lib
from codegendemo_b200.kcg.Operators.matmul import KernelArgMatmul


def compile_kernel_matmul(*args, num_stages: int = 0, kernel: int = 0, num_sms: int = 0, force: bool = False,
                          b_trans: int = 0, serpentine: int = 0):
    """Same positional signature and return shape as the reference's module function:
    31 ints in, tuple of ``(binaryPath, kernelName, gx, gy, gz, bx, by, bz)`` out."""
    info = compile_info(args, num_stages=num_stages, kernel=kernel, num_sms=num_sms, force=force, b_trans=b_trans,
                        serpentine=serpentine)
    return ((info.path.decode(), info.name.decode(), info.grid[0], info.grid[1], info.grid[2],
             info.block[0], info.block[1], info.block[2]),)


def compile_info(cfg31, num_stages: int = 0, kernel: int = 0, num_sms: int = 0, force: bool = False,
                 b_trans: int = 0, serpentine: int = 0) -> _lib.KernelInfo:
    lib = _lib.get_lib()
    opts = _lib.CompileOpts(kernel=int(kernel), num_stages=int(num_stages), num_sms=int(num_sms), force=int(bool(force)),
                            b_trans=int(bool(b_trans)), serpentine=int(bool(serpentine)))
    info = _lib.KernelInfo()
    _lib.check(lib.kcg_compile_matmul_ex(_lib.cfg_array(cfg31), ctypes.byref(opts), ctypes.byref(info)))
    return info


class KCGCompiler:
    def __init__(self):
        self.__compile_kernel_matmul = compile_kernel_matmul
        self.lastInfo = None  # kcg_kernel_info of the most recent compile, as a dict

    def compileKernel(self, param: KernelArgMatmul) -> list:
        info = compile_info(param.compileArgs(), num_stages=param.NUM_STAGES, kernel=param.KERNEL_VARIANT,
                            b_trans=param.IS_BTRANS, serpentine=param.RASTER_SERPENTINE)
        self.lastInfo = info.to_dict()
        return [(info.path.decode(), info.name.decode(), info.grid[0], info.grid[1], info.grid[2],
                 info.block[0], info.block[1], info.block[2])]
