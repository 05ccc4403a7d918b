"""Shared definitions of the ``kcg`` operator API (mirror of Runtime/python/kcg/Utils.py).

Same names and meanings as the reference: ``EnumKernelDType`` (:198-209, plus ``bfloat16``),
``ToTorchType`` (:211-217), ``sizeof`` (:219-221), ``ConfigKeywords`` (:359-390), ``PathManager``
(:300-356), ``DeviceInfo`` (:264-297) and the pickle helpers. Nothing here touches a GPU at import
time (the reference calls ``torch.cuda.current_device()`` while importing), so compile workers and
CPU-only tests can import the package freely.
"""
import json
import os
import pickle
from datetime import datetime
from enum import Enum, IntEnum
from pathlib import Path
from typing import Dict, List  # noqa: F401  (re-exported for star-importers, as the reference does)


class EnumBackendType(Enum):
    CUDA = 1
    HIP = 2
    INVALID = 3

    def __str__(self):
        return f'{self.name}'


class EnumKernelDType(IntEnum):
    """Value % 30 is the element size in bytes. 62 (bfloat16) is new; the rest are the reference's."""
    float8 = 1
    float16 = 2
    float32 = 4
    float64 = 8
    float128 = 16
    int8 = 31
    int16 = 32
    int32 = 34
    int64 = 38
    bfloat16 = 62

    def __str__(self):
        return f'{self.name}'


def ToTorchType(t: EnumKernelDType):
    import torch
    table = {
        EnumKernelDType.float32: torch.float32,
        EnumKernelDType.float64: torch.float64,
        EnumKernelDType.float16: torch.float16,
        EnumKernelDType.bfloat16: torch.bfloat16,
    }
    return table.get(EnumKernelDType(int(t)))


def FromTorchType(t) -> EnumKernelDType:
    import torch
    return {torch.float32: EnumKernelDType.float32, torch.float64: EnumKernelDType.float64,
            torch.float16: EnumKernelDType.float16, torch.bfloat16: EnumKernelDType.bfloat16}[t]


def sizeof(t: EnumKernelDType) -> int:
    """Element size in bytes."""
    assert t is not None
    return int(t) % 30


def get_dtype_from_int(dtype: int):
    try:
        return EnumKernelDType(int(dtype))
    except ValueError:
        return None


def printTime():
    print(f"--------[ {datetime.now().strftime('%Y-%m-%d %H:%M:%S')} ]------------")


def serialize_to_file(path: str, obj) -> None:
    tmp = f"{path}.{os.getpid()}.part"
    with open(tmp, 'wb') as f:
        pickle.dump(obj, f)
    os.replace(tmp, path)  # readers never see a half-written pickle


def deserialize_from_file(path: str):
    with open(path, 'rb') as f:
        return pickle.load(f)


def delete_files_in_directory(directory: str) -> None:
    if not os.path.isdir(directory):
        return
    for name in os.listdir(directory):
        p = os.path.join(directory, name)
        if os.path.isfile(p):
            try:
                os.remove(p)
            except OSError:
                pass


def is_hip() -> bool:
    return False


class DeviceInfo:
    @staticmethod
    def get_cuda_stream(idx=None) -> int:
        """Raw CUstream of torch's current stream on device ``idx`` (what the launcher launches on)."""
        import torch
        if idx is None:
            idx = DeviceInfo.get_current_device()
        try:
            from torch._C import _cuda_getCurrentRawStream
            return _cuda_getCurrentRawStream(idx)
        except ImportError:
            return torch.cuda.current_stream(idx).cuda_stream

    @staticmethod
    def get_current_device() -> int:
        import torch
        return torch.cuda.current_device()

    @staticmethod
    def set_current_device(idx) -> None:
        import torch
        torch.cuda.set_device(idx)

    @staticmethod
    def get_device_capability(idx):
        import torch
        return torch.cuda.get_device_capability(idx)

    @staticmethod
    def get_warp_size() -> int:
        return 32


class PathManager:
    """Working directories of the autotune flow (same set as the reference's PathManager).

    The root defaults to ``$KCG_WORK_DIR`` or ``./_kcg_work``; cubins are cached by the C library
    in its own cache directory (``kcg_cache_dir()``), not here.
    """
    _root = None

    @staticmethod
    def set_project_dir(path: str) -> None:
        PathManager._root = str(path)
        os.environ["KCG_WORK_DIR"] = str(path)  # spawned compile / perf processes resolve the same root

    @staticmethod
    def project_dir() -> str:
        if PathManager._root is None:
            PathManager._root = os.environ.get("KCG_WORK_DIR", os.path.join(os.getcwd(), "_kcg_work"))
        return PathManager._root

    @staticmethod
    def pikle_dir() -> str:
        return os.path.join(PathManager.project_dir(), '_pkls')

    @staticmethod
    def tmp_dir() -> str:
        return os.path.join(PathManager.project_dir(), '_tmp')

    @staticmethod
    def default_cache_dir() -> str:
        return os.path.join(PathManager.project_dir(), '_cache')

    @staticmethod
    def default_override_dir() -> str:
        return os.path.join(PathManager.project_dir(), '_override')

    @staticmethod
    def default_dump_dir() -> str:
        return os.path.join(PathManager.project_dir(), '_dump')

    @staticmethod
    def tuning_configs_dir() -> str:
        return str(Path(os.path.dirname(os.path.realpath(__file__))).parent / "TuningConfigs")

    @staticmethod
    def kcg_compiler_path() -> str:
        from codegendemo_b200 import _lib
        return _lib.lib_path()

    @staticmethod
    def init(clearPkl=False, clearDump=False, clearOverride=False, clearCache=False, clearTmp=False):
        dirs = [(PathManager.pikle_dir(), clearPkl), (PathManager.default_cache_dir(), clearCache),
                (PathManager.default_override_dir(), clearOverride),
                (PathManager.default_dump_dir(), clearDump), (PathManager.tmp_dir(), clearTmp)]
        for d, clear in dirs:
            os.makedirs(d, exist_ok=True)
            if clear:
                delete_files_in_directory(d)


class ConfigKeywords:
    KEY_BLOCK_SIZE_M = "BLOCK_SIZE_M"
    KEY_BLOCK_SIZE_N = "BLOCK_SIZE_N"
    KEY_BLOCK_SIZE_K = "BLOCK_SIZE_K"
    KEY_THREAD_SIZE_M = "THREAD_SIZE_M"
    KEY_THREAD_SIZE_N = "THREAD_SIZE_N"
    KEY_WARP_SIZE = "WARP_SIZE"
    KEY_BLOCK_LAYOUT_M = "BLOCK_LAYOUT_M"
    KEY_BLOCK_LAYOUT_N = "BLOCK_LAYOUT_N"
    KEY_WARP_LAYOUT_M = "WARP_LAYOUT_M"
    KEY_WARP_LAYOUT_N = "WARP_LAYOUT_N"
    KEY_DTYPE_A = "DATATYPE_A"
    KEY_DTYPE_B = "DATATYPE_B"
    KEY_DTYPE_C = "DATATYPE_C"
    KEY_M = "M_SIZE"
    KEY_N = "N_SIZE"
    KEY_K = "K_SIZE"
    KEY_IS_A_TRANSPOSE = "IS_ATRANS"
    KEY_GLOB_LOAD_WIDTH_A = "GLOB_LOAD_WIDTH_A"
    KEY_GLOB_LOAD_WIDTH_B = "GLOB_LOAD_WIDTH_B"
    KEY_WARP_SCATTER_WIDTH_A = "WARP_SCATTER_WIDTH_A"
    KEY_WARP_SCATTER_WIDTH_B = "WARP_SCATTER_WIDTH_B"
    KEY_THREAD_SCATTER_WIDTH_A = "THREAD_SCATTER_WIDTH_A"
    KEY_THREAD_SCATTER_WIDTH_B = "THREAD_SCATTER_WIDTH_B"
    KEY_LOCAL_SPLIT_U = "LOCAL_SPLIT_U"
    KEY_BLOCK_MAPPING = "BLOCK_MAPPING"
    KEY_GLOB_STORE_WIDTH = "GLOB_STORE_WIDTH"
    KEY_UNROLL_NUM = "UNROLL_NUM"
    KEY_REG_PREFETCH = "REG_PREFETCH"
    KEY_SHARED_PREFETCH = "SHARED_PREFETCH"
    KEY_LOAD_CONTINUOUS = "LOAD_CONTINUOUS"
    KEY_REDUCE_C_CONTINUOUS = "REDUCE_C_CONTINUOUS"
    # Optional keys of this library (absent from the reference's JSONs; defaults apply).
    KEY_NUM_STAGES = "NUM_STAGES"          # shared-memory pipeline depth of the tcgen05 kernels
    KEY_KERNEL_VARIANT = "KERNEL_VARIANT"  # 0 auto, 1 SIMT FFMA, 2 tcgen05 (fp32: 3xTF32), 3 TF32 x1, 4 CTA pairs,
    #                                        5 cluster split-K (LOCAL_SPLIT_U CTAs per tile, shared-memory reduction)
    KEY_IS_B_TRANSPOSE = "IS_BTRANS"       # 1 = B stored N x K row-major (16-bit tcgen05 kernels)
    KEY_RASTER_SERPENTINE = "RASTER_SERPENTINE"  # 1 = serpentine walk inside a BLOCK_MAPPING group (tcgen05 kernels)

    # Positional order of the compile entry (src/main.cc:64-102 == KCGCompiler.py:14-44).
    COMPILE_ORDER = (
        "BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_SIZE_K", "THREAD_SIZE_M", "THREAD_SIZE_N", "WARP_SIZE",
        "BLOCK_LAYOUT_M", "BLOCK_LAYOUT_N", "WARP_LAYOUT_M", "WARP_LAYOUT_N",
        "GLOB_LOAD_WIDTH_A", "GLOB_LOAD_WIDTH_B", "WARP_SCATTER_WIDTH_A", "WARP_SCATTER_WIDTH_B",
        "THREAD_SCATTER_WIDTH_A", "THREAD_SCATTER_WIDTH_B", "LOCAL_SPLIT_U", "BLOCK_MAPPING",
        "GLOB_STORE_WIDTH", "UNROLL_NUM", "REG_PREFETCH", "SHARED_PREFETCH", "LOAD_CONTINUOUS",
        "REDUCE_C_CONTINUOUS", "DATATYPE_A", "DATATYPE_B", "DATATYPE_C", "M_SIZE", "N_SIZE", "K_SIZE",
        "IS_ATRANS")


def save_to_json(obj, output_file="config_combinations.json"):
    with open(output_file, "w") as f:
        json.dump(obj, f, indent=4)
