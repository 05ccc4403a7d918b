"""A compiled kernel ready to run: mirror of Runtime/python/kcg/CompiledKernel.py:6-23."""
from codegendemo_b200.kcg.CudaLauncher import CudaLauncher


class CompiledKernel:
    def __init__(self, kernelBinaryPath: str, kernelName: str, shmSize: int, kernel_signature,
                 gridDims: list, blockDims: list, device=0, kernelInfo: dict = None):
        self.signature = kernel_signature
        self.device = device
        self.m_launcher = CudaLauncher(kernelBinaryPath, kernelName, shmSize, self.signature, gridDims,
                                       blockDims, device, kernelInfo)

    def run(self, *args, **kwargs):
        """Asynchronous launch on torch's current stream: ``run(a, b, c)``."""
        if self.m_launcher is not None:
            self.m_launcher.launchKernel(int(self.device), *args, **kwargs)

    def runHost(self, hostA, hostB, hostC):
        self.m_launcher.runHost(int(self.device), hostA, hostB, hostC)

    def checkStatus(self):
        """Raises if a bounded wait inside the kernel ran out since the last check (synchronises)."""
        self.m_launcher.checkStatus(int(self.device))
