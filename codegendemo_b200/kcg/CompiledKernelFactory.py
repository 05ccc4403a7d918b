"""``UserInputs`` / ``CompiledKernelFactory``: mirror of Runtime/python/kcg/CompiledKernelFactory.py."""
from enum import Enum

from codegendemo_b200.kcg.CompiledKernel import CompiledKernel
from codegendemo_b200.kcg.Operators.matmul import KernelArgMatmul, getMatmulSignature
from codegendemo_b200.kcg.Utils import sizeof


class EnumOperator(Enum):
    Invalid = 0
    Matmul = 1
    Convolution = 2
    Poll = 3

    def __str__(self):
        return f'{self.name}'


class UserInputs:
    def __init__(self, hsaco_path: str, kernel_func_name: str, kernelParam: KernelArgMatmul, kernelInfo: dict = None):
        self.operatorKind = EnumOperator.Matmul
        self.hsacoPath = hsaco_path  # name kept from the reference; holds the cubin path
        self.kernelFuncName = kernel_func_name
        self.kernelParam = kernelParam
        self.kernelInfo = kernelInfo  # kcg_kernel_info as a dict (from KCGCompiler.lastInfo)
        self.m_gridDims = [1, 1, 1]
        self.m_blockDims = [1, 1, 1]

    def gridDims(self):
        return self.m_gridDims

    def blockDims(self):
        return self.m_blockDims

    def sharedMem(self) -> int:
        """Dynamic shared memory of the launch. The compile entry reports the exact figure for the
        kernel it built; without it the reference's SIMT formula applies (CompiledKernelFactory.py:30-44)."""
        if self.kernelInfo is not None:
            return int(self.kernelInfo["smem_bytes"])
        kp = self.kernelParam
        sizeAB = (kp.BLOCK_SIZE_M + kp.BLOCK_SIZE_N) * kp.BLOCK_SIZE_K * 4
        if kp.SHARED_PREFETCH > 0:
            sizeAB *= 2
        sizeC = -1
        if kp.LOCAL_SPLIT_U > 1:
            sizeC = kp.BLOCK_SIZE_M * kp.BLOCK_SIZE_N * kp.LOCAL_SPLIT_U * 4
        return max(sizeAB, sizeC)

    def numCTA(self) -> int:
        ret = 1
        for dim in self.gridDims():
            ret *= dim
        return ret


class CompiledKernelFactory:
    @staticmethod
    def getKernel(info: UserInputs, deviceId: int) -> CompiledKernel:
        if info.operatorKind == EnumOperator.Matmul:
            kp = info.kernelParam
            signature = getMatmulSignature(kp.dtypeTorch('A'), kp.dtypeTorch('B'), kp.dtypeTorch('C'))
            return CompiledKernel(info.hsacoPath, info.kernelFuncName, info.sharedMem(), signature,
                                  info.gridDims(), info.blockDims(), deviceId, info.kernelInfo)
        return None
