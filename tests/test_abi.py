"""The C-ABI library: loads without a GPU, exports every declared symbol, validates configs, names and
compiles kernels (nvcc cross-compiles sm_100a without a GPU), and refuses to compute without a driver."""
import ctypes
import os
import re

import pytest
import torch

from codegendemo_b200 import _lib
from codegendemo_b200.kcg.KCGCompiler import KCGCompiler, compile_info, compile_kernel_matmul
from codegendemo_b200.kcg.matmul_op import default_config
from codegendemo_b200.kcg.Utils import EnumKernelDType as E

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.get_lib()
    header = open(os.path.join(ROOT, "include", "kcg_b200.h")).read()
    declared = set(re.findall(r"\b(kcg_[a-z_0-9]+)\s*\(", header))
    declared -= {"kcg_cfg_index"}
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/kcg_b200.h but not exported"
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    assert b"sm_100a" in lib.kcg_version()


def test_struct_layout_matches_header():
    assert ctypes.sizeof(_lib.KernelInfo) == 1024 + 512 + 4 * (9 + 13 + 8)
    assert ctypes.sizeof(_lib.CompileOpts) == 32  # kernel, num_stages, num_sms, force, b_trans, reserved[3]
    assert ctypes.sizeof(_lib.DeviceProps) == 32


def test_compile_entry_returns_reference_shaped_tuple():
    kpm = default_config(256, 256, 256, E.bfloat16, BLOCK_SIZE_N=128)
    res = compile_kernel_matmul(*kpm.compileArgs())
    assert isinstance(res, tuple) and len(res) == 1 and len(res[0]) == 8
    path, name, gx, gy, gz, bx, by, bz = res[0]
    assert os.path.exists(path) and path.endswith(name + ".cubin")
    assert name.startswith("GEMM_MNK256x256x256_DTabcbfloat16xbfloat16xbfloat16_AT0_")
    assert (gx, gy, gz) == (4, 1, 1) and (bx, by, bz) == (256, 1, 1)
    # launch shared memory = what the kernel lays out: stages, barriers + slack, epilogue staging
    info = compile_info(kpm.compileArgs())
    assert info.smem_bytes == info.stages * (128 + 128) * 64 * 2 + 2048 + 32768 <= 227 * 1024
    # cached: second call does not recompile
    mtime = os.path.getmtime(path)
    compile_kernel_matmul(*kpm.compileArgs())
    assert os.path.getmtime(path) == mtime


def test_kernel_name_scheme_covers_every_key():
    kpm = default_config(1024, 1024, 1024, E.float32, BLOCK_SIZE_N=128, LOCAL_SPLIT_U=2, BLOCK_MAPPING=4)
    info = compile_info(kpm.compileArgs())
    name = info.name.decode()
    for part in ("MNK1024x1024x1024", "DTabcfloat32xfloat32xfloat32", "AT0", "BTmnk128x128x32", "LSU2", "BM4",
                 "UNROLL4", "REGP1", "SHMP1", "LC0", "RC0", "ST", "_V2"):
        assert part in name, part
    assert info.kernel == _lib.KERNEL_TCGEN05 and info.block[0] == 512  # 3xTF32: 4 warpgroups
    assert info.splitk == 2 and info.grid[0] == min(148, 8 * 8 * 2)


def test_auto_variant_falls_back_to_simt_for_reference_sized_tiles():
    kpm = default_config(1024, 1024, 1024, E.float32, BLOCK_SIZE_M=64, BLOCK_SIZE_N=64, BLOCK_SIZE_K=16,
                         THREAD_SIZE_M=4, THREAD_SIZE_N=4, BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=2, WARP_LAYOUT_M=4,
                         WARP_LAYOUT_N=8, WARP_SCATTER_WIDTH_A=4, WARP_SCATTER_WIDTH_B=4,
                         THREAD_SCATTER_WIDTH_A=4, THREAD_SCATTER_WIDTH_B=4)
    info = compile_info(kpm.compileArgs())
    assert info.kernel == _lib.KERNEL_SIMT
    assert info.grid[0] == 16 * 16 and info.block[0] == 16 * 16
    assert info.smem_bytes == 2 * (64 + 64) * 16 * 4


@pytest.mark.parametrize("mutate, fragment", [
    (dict(M=1000), "not divisible"),
    (dict(BLOCK_SIZE_M=64, KERNEL_VARIANT=2), "not buildable"),
    (dict(LOCAL_SPLIT_U=64), "exceeds"),
    (dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=128), "CTA-pair"),
])
def test_bad_configs_are_rejected_with_kcg_error(mutate, fragment):
    kpm = default_config(1024, 1024, 1024, E.bfloat16)
    for k, v in mutate.items():
        setattr(kpm, k, v)
    with pytest.raises(_lib.KCGError) as ei:
        compile_info(kpm.compileArgs(), kernel=kpm.KERNEL_VARIANT)
    assert ei.value.code == _lib.E_BAD_CONFIG
    assert str(ei.value).startswith("KCG Error[CUDA]: Code: -1, Messsage: ")
    assert fragment in str(ei.value)


def test_mixed_dtypes_rejected():
    args = default_config(256, 256, 256, E.bfloat16).compileArgs()
    args[24] = int(E.float32)  # DATATYPE_A differs from B/C
    with pytest.raises(_lib.KCGError):
        compile_info(args)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback_without_a_driver():
    lib = _lib.get_lib()
    props = _lib.DeviceProps()
    rc = lib.kcg_device_properties(0, ctypes.byref(props))
    assert rc == _lib.E_NO_DRIVER
    mod, fn = ctypes.c_uint64(), ctypes.c_uint64()
    rc = lib.kcg_load_binary(b"k", b"/nonexistent.cubin", 0, 0, ctypes.byref(mod), ctypes.byref(fn), None, None)
    assert rc == _lib.E_NO_DRIVER
    info = _lib.KernelInfo()
    rc = lib.kcg_launch_gemm(1, ctypes.byref(info), 0, 0, 16, 16, 16)
    assert rc == _lib.E_NO_DRIVER
    assert b"driver unavailable" in lib.kcg_last_error()


def test_kcgcompiler_class_mirrors_reference_usage():
    kpm = default_config(256, 512, 512, E.bfloat16)
    path, name, gx, gy, gz, bx, by, bz = KCGCompiler().compileKernel(kpm)[0]
    assert os.path.exists(path) and gx * gy * gz >= 1 and bx == 256


def test_every_gpu_test_config_cross_compiles():
    """All kernels the GPU tests launch are compiled here (no GPU needed), so the cubins travel with the tree."""
    from codegendemo_b200.build import compile_many
    from tests import gpu_cases
    seen = set()
    for path, name in compile_many(gpu_cases.all_configs()):
        assert os.path.getsize(path) > 1000
        seen.add(name)
    assert len(seen) >= 30


def test_pair_variant_launch_geometry():
    kpm = default_config(8192, 8192, 8192, E.bfloat16, KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, NUM_STAGES=4)
    info = compile_info(kpm.compileArgs(), num_stages=4, kernel=4)
    assert info.kernel == _lib.KERNEL_TCGEN05_PAIR and list(info.cluster) == [2, 1, 1]
    assert info.grid[0] == 148 and info.block[0] == 256
    # per CTA: 256 rows of A, 128 columns of B, + 32 KiB of TMA-store staging for the epilogue
    assert info.smem_bytes == 4 * (256 + 128) * 64 * 2 + 2048 + 32768
    f32 = default_config(4096, 4096, 4096, E.float32, KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256,
                         BLOCK_SIZE_K=32, NUM_STAGES=3)
    i2 = compile_info(f32.compileArgs(), num_stages=3, kernel=4)
    assert i2.block[0] == 512 and list(i2.cluster) == [2, 1, 1]
    # three TMA-fed hi stages of the per-CTA slices + a ring of three lo twins
    assert i2.smem_bytes == (3 + 3) * (128 + 128) * 32 * 4 + 2048


def test_cubin_cache_is_keyed_by_the_kernel_sources(tmp_path):
    """Cubins live under <cache>/src-<hash of the kernel sources>: editing any kernel header must
    never be served by a cubin built from the old text."""
    import shutil
    import subprocess
    import sys
    here = _lib.get_lib().kcg_cache_dir().decode()
    assert re.fullmatch(r"src-[0-9a-f]{12}", os.path.basename(here)), here
    src = os.path.join(os.path.dirname(_lib.__file__), "csrc", "kernels")
    copy = tmp_path / "kernels"
    shutil.copytree(src, copy)
    with open(copy / "ptx_sm100.cuh", "a") as f:
        f.write("// edited\n")
    code = ("from codegendemo_b200 import _lib; import os;"
            "print(os.path.basename(_lib.get_lib().kcg_cache_dir().decode()))")
    root = os.path.dirname(os.path.dirname(_lib.__file__))
    tags = []
    for srcdir in (src, str(copy)):
        env = dict(os.environ, KCG_KERNEL_SRC_DIR=srcdir, KCG_CACHE_DIR=str(tmp_path / "cache"))
        tags.append(subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True,
                                   check=True).stdout.strip())
    assert tags[0] == os.path.basename(here) and tags[1] != tags[0] and tags[1].startswith("src-")
