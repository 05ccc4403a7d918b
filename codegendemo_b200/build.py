"""Builds ``libkcg_b200.so`` in-tree and (optionally) a family of cubins ahead of time.

    python -m codegendemo_b200.build            # library + default cubins
    python -m codegendemo_b200.build --lib-only

The library is built with nvcc for sm_100a: its host code binds the CUDA driver lazily (so it loads without a GPU),
and two pieces of device code are linked into it (the allocation-free split-K entry and the row softmax). The GEMM
kernels themselves are compiled per config by the library's own compile entry with
``nvcc -cubin -gencode arch=compute_100a,code=sm_100a``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_library(force: bool = False) -> str:
    out = os.path.join(HERE, "libkcg_b200.so")
    srcs = [os.path.join(HERE, "csrc", "kcg_shim.cpp")]
    kdir = os.path.join(HERE, "csrc", "kernels")  # the allocation-free entry instantiates a kernel from these
    deps = srcs + [os.path.join(kdir, f) for f in sorted(os.listdir(kdir))] + [
        os.path.join(os.path.dirname(HERE), "include", "kcg_b200.h")]
    # device code linked into the library itself: the allocation-free split-K entry and the row softmax
    extra = [os.path.join(HERE, "csrc", f) for f in ("kcg_noalloc.cu", "kcg_softmax.cu", "kcg_attention.cu")]
    deps += extra
    if not force and _newer(out, deps):
        return out
    nvcc = os.path.join(CUDA_HOME, "bin", "nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-cudart", "static", "-I" + os.path.join(HERE, "csrc", "kernels"),
           "-o", out, *srcs, *extra, "-ldl", "-lpthread"]
    subprocess.check_call(cmd)
    return out


def prebuilt_configs():
    """Configs compiled ahead of time, so that a GPU box needs no nvcc for the smoke run and the bench."""
    from codegendemo_b200.kcg.matmul_op import default_config, tuned_config
    from codegendemo_b200.kcg.Utils import EnumKernelDType as E
    simt = dict(KERNEL_VARIANT=1, BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=16, THREAD_SIZE_M=8,
                THREAD_SIZE_N=8, BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=2, WARP_LAYOUT_M=4, WARP_LAYOUT_N=8,
                WARP_SCATTER_WIDTH_A=4, WARP_SCATTER_WIDTH_B=4, THREAD_SCATTER_WIDTH_A=4, THREAD_SCATTER_WIDTH_B=4)
    cfgs = [tuned_config(1024, 1024, 1024, E.float32), tuned_config(4096, 4096, 4096, E.float32),
            default_config(4096, 4096, 4096, E.float32, **simt), tuned_config(8192, 8192, 8192, E.bfloat16)]
    # the rectangular sweep the benchmark line carries
    cfgs += [tuned_config(m, nk, nk, dt) for nk in (4096, 11008) for m in (128, 512, 2048)
             for dt in (E.float32, E.bfloat16)]
    for g in (1, 2, 4, 8):
        cfgs.append(tuned_config(32768 // g, 8192, 8192, E.bfloat16))
        if g > 1:  # tile of the bench's fused GEMM + all-gather leg (two TMEM accumulator buffers)
            cfgs.append(default_config(32768 // g, 8192, 8192, E.bfloat16))
    return cfgs


def prune_stale_cubins() -> None:
    """Cubins are cached under _cache/src-<hash of the kernel sources>; drop the directories of older sources."""
    import shutil
    from codegendemo_b200 import _lib
    cur = _lib.get_lib().kcg_cache_dir().decode()
    base = os.path.dirname(cur)
    if os.path.basename(base) != "_cache":
        return
    for d in os.listdir(base):
        full = os.path.join(base, d)
        if full != cur and (d.startswith("src-") or d.endswith(".cubin")):
            shutil.rmtree(full) if os.path.isdir(full) else os.remove(full)


def compile_many(kpms, workers: int = 0, verbose: bool = False):
    """Compiles a list of configs on a thread pool (the compile entry is reentrant and runs nvcc in a child
    process, so threads suffice); returns [(path, name)] in input order. Cached cubins cost nothing."""
    from concurrent.futures import ThreadPoolExecutor
    from codegendemo_b200.kcg.KCGCompiler import KCGCompiler

    def one(kpm):
        kpm.check()
        path, name = KCGCompiler().compileKernel(kpm)[0][:2]
        if verbose:
            print("cubin:", os.path.basename(path))
        return path, name

    workers = workers or min(16, os.cpu_count() or 1)
    with ThreadPoolExecutor(max_workers=workers) as pool:
        return list(pool.map(one, kpms))


def prebuild_kernels(verbose: bool = True) -> int:
    prune_stale_cubins()
    return len(compile_many(prebuilt_configs(), verbose=verbose))


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    print(build_library(force="--force" in sys.argv))
    if "--lib-only" not in sys.argv:
        prebuild_kernels()
