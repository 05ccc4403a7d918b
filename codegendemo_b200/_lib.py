"""ctypes binding of ``libkcg_b200.so`` (the C ABI declared in ``include/kcg_b200.h``).

The shared library is built in-tree by :mod:`codegendemo_b200.build` and must be present:
there is no Python or CPU fallback for any entry point. Errors come back as the C
function's status code; :func:`check` turns a non-zero status into ``RuntimeError`` carrying
``kcg_last_error()`` (prefix ``"KCG Error[CUDA]: Code: ..."``, the reference loader's
convention, Runtime/python/kcg/loaderCCode/hip.c:8-21).
"""
import ctypes
import os

NUM_CFG_KEYS = 31
LIB_NAME = "libkcg_b200.so"

KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05, KERNEL_TF32X1, KERNEL_TCGEN05_PAIR, KERNEL_TCGEN05_CLUSTERK = 0, 1, 2, 3, 4, 5
KERNEL_NAIVE, KERNEL_WAIT_PROBE = 100, 101

E_BAD_CONFIG, E_COMPILE, E_NO_DRIVER, E_IO, E_DEVICE_TIMEOUT, E_BAD_ARG, E_TOO_LARGE = (
    -1, -2, -3, -4, -5, -6, -7)

# Every symbol include/kcg_b200.h declares; tests check the library exports all of them.
EXPORTED_SYMBOLS = (
    "kcg_compile_matmul", "kcg_compile_matmul_ex", "kcg_kernel_name", "kcg_cache_dir",
    "kcg_load_binary", "kcg_unload", "kcg_device_properties", "kcg_launch_gemm",
    "kcg_launch_gemm_ex", "kcg_launch_gemm_batched", "kcg_launch_gemm_strided", "kcg_softmax_rows", "kcg_softmax_rows_ex",
    "kcg_attention_fwd", "kcg_attention_status",
    "kcg_launch_gemm_allgather", "kcg_peer_alloc", "kcg_peer_open", "kcg_peer_close",
    "kcg_peer_free", "kcg_check_status", "kcg_matmul_host", "kcg_launch_count", "kcg_shutdown",
    "kcg_last_error", "kcg_version", "kcg_gemm_bf16_splitk_noalloc",
)


class KernelInfo(ctypes.Structure):
    """``kcg_kernel_info``."""
    _fields_ = [
        ("path", ctypes.c_char * 1024),
        ("name", ctypes.c_char * 512),
        ("grid", ctypes.c_int32 * 3),
        ("block", ctypes.c_int32 * 3),
        ("cluster", ctypes.c_int32 * 3),
        ("smem_bytes", ctypes.c_int32),
        ("kernel", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("bm", ctypes.c_int32), ("bn", ctypes.c_int32), ("bk", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("splitk", ctypes.c_int32),
        ("group", ctypes.c_int32),
        ("atrans", ctypes.c_int32),
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 8),
    ]

    _SCALARS = ("smem_bytes", "kernel", "dtype", "bm", "bn", "bk", "stages", "splitk", "group",
                "atrans", "m", "n", "k")
    _RESERVED = {"num_sms": 0, "b_trans": 1, "serpentine": 2, "dtype_c": 3, "acc_buffers": 4}  # named slots of `reserved`

    def to_dict(self) -> dict:
        """Plain, picklable form (compile workers hand it to the process that owns the GPU)."""
        d = {k: int(getattr(self, k)) for k in self._SCALARS}
        d["path"] = self.path.decode()
        d["name"] = self.name.decode()
        d["grid"] = list(self.grid)
        d["block"] = list(self.block)
        d["cluster"] = list(self.cluster)
        for name, i in self._RESERVED.items():
            d[name] = int(self.reserved[i])
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "KernelInfo":
        o = cls()
        o.path = d["path"].encode()
        o.name = d["name"].encode()
        for i in range(3):
            o.grid[i] = d["grid"][i]
            o.block[i] = d["block"][i]
            o.cluster[i] = d["cluster"][i]
        for k in cls._SCALARS:
            setattr(o, k, d[k])
        for name, i in cls._RESERVED.items():
            o.reserved[i] = int(d.get(name, 0))
        return o


class CompileOpts(ctypes.Structure):
    """``kcg_compile_opts``."""
    _fields_ = [("kernel", ctypes.c_int32), ("num_stages", ctypes.c_int32),
                ("num_sms", ctypes.c_int32), ("force", ctypes.c_int32), ("b_trans", ctypes.c_int32),
                ("serpentine", ctypes.c_int32), ("reserved", ctypes.c_int32 * 2)]


class Epilogue(ctypes.Structure):
    """``kcg_epilogue``: C = act(alpha * A.B + beta * C + bias[col])."""
    _fields_ = [("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("bias", ctypes.c_uint64),
                ("relu", ctypes.c_int32), ("reserved", ctypes.c_int32 * 3)]


class DeviceProps(ctypes.Structure):
    """``kcg_device_props``."""
    _fields_ = [("max_shared_mem", ctypes.c_int32), ("multiprocessor_count", ctypes.c_int32),
                ("sm_clock_rate", ctypes.c_int32), ("mem_clock_rate", ctypes.c_int32),
                ("mem_bus_width", ctypes.c_int32), ("l2_cache_bytes", ctypes.c_int32),
                ("cc_major", ctypes.c_int32), ("cc_minor", ctypes.c_int32)]


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


_lib = None


def get_lib() -> ctypes.CDLL:
    """Loads the library once. Raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m codegendemo_b200.build` "
            "(the GEMM path has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(path)
    u64, i32p = ctypes.c_uint64, ctypes.POINTER(ctypes.c_int32)
    cfg_t = ctypes.POINTER(ctypes.c_int32)
    lib.kcg_compile_matmul.argtypes = [cfg_t, ctypes.POINTER(KernelInfo)]
    lib.kcg_compile_matmul_ex.argtypes = [cfg_t, ctypes.POINTER(CompileOpts), ctypes.POINTER(KernelInfo)]
    lib.kcg_kernel_name.argtypes = [cfg_t, ctypes.POINTER(CompileOpts), ctypes.c_char_p, ctypes.c_int]
    lib.kcg_cache_dir.restype = ctypes.c_char_p
    lib.kcg_load_binary.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                    ctypes.POINTER(u64), ctypes.POINTER(u64), i32p, i32p]
    lib.kcg_unload.argtypes = [u64]
    lib.kcg_device_properties.argtypes = [ctypes.c_int, ctypes.POINTER(DeviceProps)]
    lib.kcg_launch_gemm.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64, u64, u64, u64]
    lib.kcg_launch_gemm_ex.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64, u64, u64, u64,
                                       ctypes.POINTER(Epilogue)]
    lib.kcg_launch_gemm_allgather.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64, u64, u64, u64,
                                              ctypes.POINTER(Epilogue), ctypes.POINTER(u64), ctypes.c_int]
    lib.kcg_launch_gemm_batched.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64, u64, u64, u64,
                                            ctypes.c_int, ctypes.POINTER(Epilogue)]
    lib.kcg_launch_gemm_batched.restype = ctypes.c_int
    lib.kcg_launch_gemm_strided.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64, u64, u64, u64,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                            ctypes.POINTER(Epilogue)]
    lib.kcg_launch_gemm_strided.restype = ctypes.c_int
    lib.kcg_softmax_rows.argtypes = [ctypes.c_int, u64, u64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
                                     ctypes.c_float, ctypes.c_int]
    lib.kcg_softmax_rows.restype = ctypes.c_int
    lib.kcg_softmax_rows_ex.argtypes = [ctypes.c_int, u64, u64, ctypes.c_int, ctypes.c_int64, u64, ctypes.c_int,
                                        ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_float]
    lib.kcg_softmax_rows_ex.restype = ctypes.c_int
    lib.kcg_attention_fwd.argtypes = [ctypes.c_int, u64, u64, u64, u64, u64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_float]
    lib.kcg_attention_fwd.restype = ctypes.c_int
    lib.kcg_attention_status.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_uint32)]
    lib.kcg_attention_status.restype = ctypes.c_int
    lib.kcg_peer_alloc.argtypes = [ctypes.c_int, u64, ctypes.POINTER(u64), ctypes.c_char_p]
    lib.kcg_peer_open.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(u64)]
    lib.kcg_peer_close.argtypes = [ctypes.c_int, u64]
    lib.kcg_peer_free.argtypes = [ctypes.c_int, u64]
    for name in ("kcg_launch_gemm_allgather", "kcg_peer_alloc", "kcg_peer_open", "kcg_peer_close", "kcg_peer_free"):
        getattr(lib, name).restype = ctypes.c_int
    lib.kcg_check_status.argtypes = [ctypes.c_int, u64]
    lib.kcg_matmul_host.argtypes = [u64, ctypes.POINTER(KernelInfo), ctypes.c_int, u64,
                                    ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.kcg_gemm_bf16_splitk_noalloc.argtypes = [ctypes.c_int, u64, u64, u64, u64, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_int]
    lib.kcg_gemm_bf16_splitk_noalloc.restype = ctypes.c_int
    lib.kcg_launch_count.restype = u64
    lib.kcg_last_error.restype = ctypes.c_char_p
    lib.kcg_version.restype = ctypes.c_char_p
    for name in ("kcg_compile_matmul", "kcg_compile_matmul_ex", "kcg_kernel_name", "kcg_load_binary",
                 "kcg_unload", "kcg_device_properties", "kcg_launch_gemm", "kcg_launch_gemm_ex",
                 "kcg_check_status", "kcg_matmul_host", "kcg_shutdown"):
        getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


class KCGError(RuntimeError):
    """A C-ABI call failed; ``code`` is its return value (CUresult > 0, KCG_E_* < 0)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def check(status: int) -> None:
    if status != 0:
        msg = get_lib().kcg_last_error()
        raise KCGError(status, msg.decode(errors="replace") if msg else f"KCG Error: code {status}")


def cfg_array(values) -> ctypes.Array:
    vals = [int(v) for v in values]
    if len(vals) != NUM_CFG_KEYS:
        raise ValueError(f"expected {NUM_CFG_KEYS} config integers, got {len(vals)}")
    return (ctypes.c_int32 * NUM_CFG_KEYS)(*vals)
