"""Matmul operator config: ``KernelArgMatmul`` and the tuning-space pruners.

Mirror of Runtime/python/kcg/Operators/matmul.py: the 31 tuning keys (:75-107), JSON round trip
(``jsonfy`` :110, ``assignWithJson`` :146), ``check()`` (:180-194) and
``TuningSpaceChecker_Matmul`` (:249-313). Two optional keys are new (``NUM_STAGES``,
``KERNEL_VARIANT``); a config without them behaves exactly like a reference config.
"""
from typing import Dict

from codegendemo_b200.kcg.Utils import (ConfigKeywords, EnumKernelDType, ToTorchType,
                                        get_dtype_from_int, sizeof)

# attribute name on KernelArgMatmul -> JSON key
_ATTR_TO_KEY = {
    "BLOCK_SIZE_M": ConfigKeywords.KEY_BLOCK_SIZE_M, "BLOCK_SIZE_N": ConfigKeywords.KEY_BLOCK_SIZE_N,
    "BLOCK_SIZE_K": ConfigKeywords.KEY_BLOCK_SIZE_K, "THREAD_SIZE_M": ConfigKeywords.KEY_THREAD_SIZE_M,
    "THREAD_SIZE_N": ConfigKeywords.KEY_THREAD_SIZE_N, "WARP_SIZE": ConfigKeywords.KEY_WARP_SIZE,
    "BLOCK_LAYOUT_M": ConfigKeywords.KEY_BLOCK_LAYOUT_M, "BLOCK_LAYOUT_N": ConfigKeywords.KEY_BLOCK_LAYOUT_N,
    "WARP_LAYOUT_M": ConfigKeywords.KEY_WARP_LAYOUT_M, "WARP_LAYOUT_N": ConfigKeywords.KEY_WARP_LAYOUT_N,
    "M": ConfigKeywords.KEY_M, "N": ConfigKeywords.KEY_N, "K": ConfigKeywords.KEY_K,
    "isATranspose": ConfigKeywords.KEY_IS_A_TRANSPOSE,
    "GLOB_LOAD_WIDTH_A": ConfigKeywords.KEY_GLOB_LOAD_WIDTH_A,
    "GLOB_LOAD_WIDTH_B": ConfigKeywords.KEY_GLOB_LOAD_WIDTH_B,
    "WARP_SCATTER_WIDTH_A": ConfigKeywords.KEY_WARP_SCATTER_WIDTH_A,
    "WARP_SCATTER_WIDTH_B": ConfigKeywords.KEY_WARP_SCATTER_WIDTH_B,
    "THREAD_SCATTER_WIDTH_A": ConfigKeywords.KEY_THREAD_SCATTER_WIDTH_A,
    "THREAD_SCATTER_WIDTH_B": ConfigKeywords.KEY_THREAD_SCATTER_WIDTH_B,
    "LOCAL_SPLIT_U": ConfigKeywords.KEY_LOCAL_SPLIT_U, "BLOCK_MAPPING": ConfigKeywords.KEY_BLOCK_MAPPING,
    "GLOB_STORE_WIDTH": ConfigKeywords.KEY_GLOB_STORE_WIDTH, "UNROLL_NUM": ConfigKeywords.KEY_UNROLL_NUM,
    "REG_PREFETCH": ConfigKeywords.KEY_REG_PREFETCH, "SHARED_PREFETCH": ConfigKeywords.KEY_SHARED_PREFETCH,
    "LOAD_CONTINUOUS": ConfigKeywords.KEY_LOAD_CONTINUOUS,
    "REDUCE_C_CONTINUOUS": ConfigKeywords.KEY_REDUCE_C_CONTINUOUS,
}
_OPTIONAL = {"NUM_STAGES": ConfigKeywords.KEY_NUM_STAGES, "KERNEL_VARIANT": ConfigKeywords.KEY_KERNEL_VARIANT,
             "IS_BTRANS": ConfigKeywords.KEY_IS_B_TRANSPOSE, "RASTER_SERPENTINE": ConfigKeywords.KEY_RASTER_SERPENTINE}

# Shared memory one CTA may use on sm_100a (the reference asserts 64 KiB for gfx906).
MAX_SHARED_BYTES = 227 * 1024


def getMatmulSignature(dtypeA, dtypeB, dtypeC) -> dict:
    """Kernel signature {arg index: pointer type}; depends on dtypes only.

    The reference computes it by tracing a stub kernel on three freshly allocated GPU tensors
    (matmul.py:61-72); the result is a constant, so it is returned directly and compile workers
    stay GPU-free.
    """
    import torch
    names = {torch.float32: "*fp32", torch.float16: "*fp16", torch.bfloat16: "*bf16", torch.float64: "*fp64"}
    return {0: names[dtypeA], 1: names[dtypeB], 2: names[dtypeC]}


class KernelArgMatmul:
    def __init__(self, m, n, k, typeA: EnumKernelDType, typeB: EnumKernelDType, typeC: EnumKernelDType):
        self.BLOCK_SIZE_M = 64
        self.BLOCK_SIZE_N = 64
        self.BLOCK_SIZE_K = 16
        self.THREAD_SIZE_M = 4
        self.THREAD_SIZE_N = 4
        self.WARP_SIZE = 32
        self.BLOCK_LAYOUT_M = 4
        self.BLOCK_LAYOUT_N = 2
        self.WARP_LAYOUT_M = 4
        self.WARP_LAYOUT_N = 8
        self.__dataType_A = typeA
        self.__dataType_B = typeB
        self.__dataType_C = typeC
        self.M = m
        self.N = n
        self.K = k
        self.isATranspose = 1
        self.GLOB_LOAD_WIDTH_A = 0
        self.GLOB_LOAD_WIDTH_B = 0
        self.WARP_SCATTER_WIDTH_A = 0
        self.WARP_SCATTER_WIDTH_B = 0
        self.THREAD_SCATTER_WIDTH_A = 0
        self.THREAD_SCATTER_WIDTH_B = 0
        self.LOCAL_SPLIT_U = 0
        self.BLOCK_MAPPING = 0
        self.GLOB_STORE_WIDTH = 0
        self.UNROLL_NUM = 1
        self.REG_PREFETCH = 0
        self.SHARED_PREFETCH = 0
        self.LOAD_CONTINUOUS = 0
        self.REDUCE_C_CONTINUOUS = 0
        # optional, B200-specific
        self.NUM_STAGES = 0       # 0 = derive from SHARED_PREFETCH
        self.KERNEL_VARIANT = 0   # 0 = auto
        self.IS_BTRANS = 0        # 1 = B is stored N x K (tcgen05 16-bit kernels)
        self.RASTER_SERPENTINE = 0  # 1 = odd tile columns of a BLOCK_MAPPING group walk its rows upwards

    def jsonfy(self) -> Dict:
        obj = {key: int(getattr(self, attr)) for attr, key in _ATTR_TO_KEY.items()}
        obj[ConfigKeywords.KEY_DTYPE_A] = int(self.__dataType_A)
        obj[ConfigKeywords.KEY_DTYPE_B] = int(self.__dataType_B)
        obj[ConfigKeywords.KEY_DTYPE_C] = int(self.__dataType_C)
        for attr, key in _OPTIONAL.items():
            if getattr(self, attr):
                obj[key] = int(getattr(self, attr))
        return obj

    def assignWithJson(self, jsonObj) -> None:
        for attr, key in _ATTR_TO_KEY.items():
            setattr(self, attr, int(jsonObj[key]))
        self.__dataType_A = int(jsonObj[ConfigKeywords.KEY_DTYPE_A])
        self.__dataType_B = int(jsonObj[ConfigKeywords.KEY_DTYPE_B])
        self.__dataType_C = int(jsonObj[ConfigKeywords.KEY_DTYPE_C])
        for attr, key in _OPTIONAL.items():
            setattr(self, attr, int(jsonObj.get(key, 0)))

    @classmethod
    def fromJson(cls, jsonObj) -> "KernelArgMatmul":
        o = cls(0, 0, 0, 1, 1, 1)
        o.assignWithJson(jsonObj)
        return o

    def usesTensorCores(self) -> bool:
        """True when the config's tile is one the tcgen05 kernel can build (what AUTO resolves to)."""
        if self.KERNEL_VARIANT in (2, 3, 4, 5):
            return True
        if self.KERNEL_VARIANT == 1:
            return False
        return TuningSpaceChecker_Matmul.tcgen05_tile_ok(self.jsonfy())

    def check(self, verbose: bool = False) -> None:
        # problem size check
        assert self.M % self.BLOCK_SIZE_M == 0
        assert self.N % self.BLOCK_SIZE_N == 0
        assert self.K % self.BLOCK_SIZE_K == 0
        if not self.usesTensorCores():
            # warp-block validation check (the thread-level keys drive the SIMT kernel only)
            assert self.BLOCK_SIZE_M % self.THREAD_SIZE_M == 0
            assert self.BLOCK_SIZE_N % self.THREAD_SIZE_N == 0
            assert (self.BLOCK_LAYOUT_M * self.WARP_LAYOUT_M) == (self.BLOCK_SIZE_M // self.THREAD_SIZE_M)
            assert (self.BLOCK_LAYOUT_N * self.WARP_LAYOUT_N) == (self.BLOCK_SIZE_N // self.THREAD_SIZE_N)
            assert self.WARP_LAYOUT_N * self.WARP_LAYOUT_M == self.WARP_SIZE
        # shm size check
        per_cta = 2 if self.KERNEL_VARIANT == 4 else 1  # a CTA pair splits the tile's operands
        assert 2 * (self.BLOCK_SIZE_M + self.BLOCK_SIZE_N) * self.BLOCK_SIZE_K * sizeof(self.__dataType_A) // per_cta \
            <= MAX_SHARED_BYTES
        if verbose:
            print("===== config check ok!")

    def compileArgs(self) -> list:
        """The 31 integers in the compile entry's positional order."""
        j = self.jsonfy()
        return [int(j[k]) for k in ConfigKeywords.COMPILE_ORDER]

    def setOutputDtype(self, typeC) -> None:
        """DATATYPE_C on its own: float32 C over fp16 / bf16 operands keeps the fp32 accumulators unrounded
        (single-pass tcgen05 kernels); everywhere else C has the operands' type."""
        self.__dataType_C = int(typeC)

    def dtype(self, index: str) -> EnumKernelDType:
        return {'A': self.__dataType_A, 'B': self.__dataType_B, 'C': self.__dataType_C}.get(index)

    def dtypeTorch(self, index: str):
        return ToTorchType(self.dtype(index))

    def __str__(self):
        body = " ,\n".join(f' "{k}"  :  {v}' for k, v in self.jsonfy().items())
        return "{\n" + body + "\n}"


class TuningSpaceChecker_Matmul:
    """Pruners applied while the tuning space is enumerated."""

    @staticmethod
    def check_shm_size(config: Dict) -> bool:
        """Shared-memory bound; also expands a lone DATATYPE_C into DATATYPE_A/B/C like the reference.

        The reference keeps configs below 16 KiB (its LDS budget per wave group); on sm_100a the
        bound is the 227 KiB a CTA can opt in to.
        """
        kw = ConfigKeywords
        dtypeC = config[kw.KEY_DTYPE_C]
        nbytes = sizeof(get_dtype_from_int(dtypeC))
        lsu = max(1, config.get(kw.KEY_LOCAL_SPLIT_U, 1))
        bufs = 2 if config.get(kw.KEY_SHARED_PREFETCH, 0) else 1
        ab = (config[kw.KEY_BLOCK_SIZE_M] + config[kw.KEY_BLOCK_SIZE_N]) * config[kw.KEY_BLOCK_SIZE_K] * nbytes * bufs
        cc = config[kw.KEY_BLOCK_SIZE_M] * config[kw.KEY_BLOCK_SIZE_N] * 4 * lsu if lsu > 1 else 0
        if TuningSpaceChecker_Matmul.tcgen05_tile_ok(config):
            cc = 0  # split-K partials of the tensor-core kernel live in global memory
        if max(ab, cc) <= MAX_SHARED_BYTES:
            config.setdefault(kw.KEY_DTYPE_A, dtypeC)
            config.setdefault(kw.KEY_DTYPE_B, dtypeC)
            return True
        return False

    @staticmethod
    def check_warp(config: Dict) -> bool:
        kw = ConfigKeywords
        return config[kw.KEY_WARP_LAYOUT_M] * config[kw.KEY_WARP_LAYOUT_N] == config[kw.KEY_WARP_SIZE]

    @staticmethod
    def check_size(config: Dict) -> bool:
        kw = ConfigKeywords
        bm, bn, bk = config[kw.KEY_BLOCK_SIZE_M], config[kw.KEY_BLOCK_SIZE_N], config[kw.KEY_BLOCK_SIZE_K]
        if config[kw.KEY_M] % bm or config[kw.KEY_N] % bn or config[kw.KEY_K] % bk:
            return False
        if (config[kw.KEY_BLOCK_LAYOUT_M] * config[kw.KEY_WARP_LAYOUT_M] * config[kw.KEY_THREAD_SIZE_M] != bm or
                config[kw.KEY_BLOCK_LAYOUT_N] * config[kw.KEY_WARP_LAYOUT_N] * config[kw.KEY_THREAD_SIZE_N] != bn):
            return False
        wswa, wswb = config[kw.KEY_WARP_SCATTER_WIDTH_A], config[kw.KEY_WARP_SCATTER_WIDTH_B]
        tswa, tswb = config[kw.KEY_THREAD_SCATTER_WIDTH_A], config[kw.KEY_THREAD_SCATTER_WIDTH_B]
        if wswa < tswa or wswb < tswb:
            return False
        if tswa <= 0 or tswb <= 0 or wswa % tswa != 0 or wswb % tswb != 0:
            return False
        return True

    @staticmethod
    def tcgen05_tile_ok(config: Dict, stages: int = 2) -> bool:
        """Tile rules of the tcgen05 kernels (same rules the compile entry enforces)."""
        kw = ConfigKeywords
        dt = int(config.get(kw.KEY_DTYPE_A, config[kw.KEY_DTYPE_C]))
        if dt not in (int(EnumKernelDType.float16), int(EnumKernelDType.float32), int(EnumKernelDType.bfloat16)):
            return False
        eb = dt % 30
        bm, bn, bk = config[kw.KEY_BLOCK_SIZE_M], config[kw.KEY_BLOCK_SIZE_N], config[kw.KEY_BLOCK_SIZE_K]
        if bm not in (128, 256):
            return False
        atom = 128 // eb
        if bn < atom or bn > 256 or bn % atom or bn % 16:
            return False
        if (bm // 128) * bn > 512:
            return False
        if eb == 4 and ((bm // 128) * bn > 256 or bn % 64):  # 3xTF32: two TMEM buffers + register accumulators
            return False
        rowb = bk * eb
        if not (rowb in (32, 64) or rowb % 128 == 0) or rowb > 512:
            return False
        if bk % (32 // eb) or bk % 8 or (eb == 2 and bk % 16):
            return False
        stage = (bm + bn) * bk * eb
        lo = stages if eb == 4 else 0  # 3xTF32: a ring of lo twins as deep as the ring of hi stages
        staging = 0 if eb == 4 else 32768  # TMA-store staging of the 16-bit kernel's epilogue
        return stage * (stages + lo) + 2048 + staging <= MAX_SHARED_BYTES

    @staticmethod
    def check_simt_loads(config: Dict) -> bool:
        """Divisibility the SIMT kernel needs for its vectorised tile loads and stores."""
        kw = ConfigKeywords
        bm, bn, bk = config[kw.KEY_BLOCK_SIZE_M], config[kw.KEY_BLOCK_SIZE_N], config[kw.KEY_BLOCK_SIZE_K]
        tm, tn = config[kw.KEY_THREAD_SIZE_M], config[kw.KEY_THREAD_SIZE_N]
        lsu = max(1, config.get(kw.KEY_LOCAL_SPLIT_U, 1))
        threads = (bm // tm) * (bn // tn) * lsu
        glwa = max(1, config.get(kw.KEY_GLOB_LOAD_WIDTH_A, 1))
        glwb = max(1, config.get(kw.KEY_GLOB_LOAD_WIDTH_B, 1))
        gsw = max(1, config.get(kw.KEY_GLOB_STORE_WIDTH, 1))
        tswb = max(1, config.get(kw.KEY_THREAD_SCATTER_WIDTH_B, 1))
        wswa = max(1, config.get(kw.KEY_WARP_SCATTER_WIDTH_A, 1))
        wswb = max(1, config.get(kw.KEY_WARP_SCATTER_WIDTH_B, 1))
        if threads > 1024 or bk % lsu or tm % wswa or tn % wswb:
            return False
        if (bm * bk) % (threads * glwa) or (bn * bk) % (threads * glwb):
            return False
        if (bm if config.get(kw.KEY_IS_A_TRANSPOSE, 1) else bk) % glwa or bn % glwb:
            return False
        if lsu > 1:
            return bn % gsw == 0
        return tswb % min(gsw, tswb) == 0
