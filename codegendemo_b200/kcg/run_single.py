"""Compile, run and check ONE tuning config from the command line.

The single-case counterpart of the autotune driver (role of the reference's ad-hoc
Runtime/python/kcg/test.py): handy for a quick check of a config and as a small, self-ending
workload for profilers.

    python -m codegendemo_b200.kcg.run_single --m 2048 --n 8192 --k 8192 --dtype bf16 \
        --set BLOCK_SIZE_M=256 --set BLOCK_SIZE_N=256 --set NUM_STAGES=3 --launches 3 --warmup 2
"""
import argparse
import math
import sys

from codegendemo_b200.kcg.matmul_op import build_kernel, default_config, tuned_config
from codegendemo_b200.kcg.Utils import EnumKernelDType


_PHASES = ["entry", "set-up barrier passed", "first TMA issued", "first stage landed", "MMAs of unit 0 issued",
           "accumulator of unit 0 seen full", "last C store of unit 0 issued", "C stores read out",
           "exit barrier passed", "TMEM released"]
_PHASES_CLUSTERK = ["entry", "set-up barrier passed", "first TMA issued", "MMAs issued", "accumulator seen full",
                    "warp 0's copies issued", "peers' partials received", "C stored", "TMEM released"]


def print_timeline(C, variant: int) -> None:
    """Decodes the %globaltimer stamps a KCG_TIMELINE build of the tcgen05 kernels leaves in C[0, :]."""
    import torch
    t = C.view(torch.uint8).flatten()[:128].view(torch.int64).cpu().tolist()
    names = _PHASES_CLUSTERK if variant == 5 else _PHASES
    print(f"in-kernel time of CTA 0: {(t[len(names) - 1] - t[0]) / 1e3:.2f} us")
    print("  " + "  ".join(f"{names[i]} +{(t[i] - t[0]) / 1e3:.2f}" for i in range(1, len(names))))
    if variant == 5:
        extra = {9: "ring-idle signals sent", 10: "blocks staged", 12: "warp 1's copies issued", 15: "own block read",
                 11: "first block summed", 13: "first block stored"}
        print("  " + "  ".join(f"{name} +{(t[i] - t[0]) / 1e3:.2f}" for i, name in extra.items() if t[i] > t[0]))
    if variant != 5 and t[14] > t[0]:
        print(f"  K-split unit 0: partial published +{(t[14] - t[0]) / 1e3:.2f}"
              + (f"  tile reduced and stored +{(t[15] - t[0]) / 1e3:.2f}" if t[15] > t[0] else "  (not the reducer)"))
    if variant != 5:
        print(f"  cycles over the K loop: producer waiting {t[10]}, producer issuing {t[11]}, "
              f"MMA thread waiting {t[12]}, MMA thread issuing {t[13]}")


def main(argv=None) -> int:
    import torch
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="override a tuning key (attribute of KernelArgMatmul), e.g. BLOCK_SIZE_N=128")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--tuned", action="store_true",
                    help="start from the kernel database / rule of thumb for this shape instead of the default config")
    ap.add_argument("--cublas", action="store_true",
                    help="also launch torch.matmul (cuBLAS) on the same operands the same number of times: "
                         "a comparison line, and a second kernel in a profiler's launch list")
    ap.add_argument("--timeline", action="store_true",
                    help="print the in-kernel phase stamps of CTA 0. Needs kernels compiled with "
                         "KCG_NVCC_FLAGS=-DKCG_TIMELINE=1 (add -DKCG_PROBE_NO_MMA=1 to time the operand loads "
                         "alone) into a private KCG_CACHE_DIR; such kernels overwrite the first words of C, "
                         "so the result check is skipped")
    a = ap.parse_args(argv)
    edt = {"bf16": EnumKernelDType.bfloat16, "fp16": EnumKernelDType.float16, "fp32": EnumKernelDType.float32}[a.dtype]
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    keys = {}
    for kv in a.set:
        k, v = kv.split("=", 1)
        keys[k] = int(v)
    if a.tuned:
        kpm = tuned_config(a.m, a.n, a.k, edt)
        for k, v in keys.items():
            setattr(kpm, k, v)
    else:
        kpm = default_config(a.m, a.n, a.k, edt, **keys)
    torch.cuda.set_device(a.device)
    dev = f"cuda:{a.device}"
    inConfig, kern = build_kernel(kpm, a.device)
    g = torch.Generator(device=dev).manual_seed(0)
    A = (torch.randn(a.m, a.k, generator=g, device=dev) / math.sqrt(a.k)).to(tdt)
    B = (torch.randn(a.k, a.n, generator=g, device=dev) / math.sqrt(a.k)).to(tdt)
    C = torch.empty(a.m, a.n, dtype=tdt, device=dev)
    a_in = A.t().contiguous() if kpm.isATranspose else A
    for _ in range(a.warmup):
        kern.run(a_in, B, C)
    torch.cuda.synchronize()
    times = []
    for _ in range(a.launches):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        kern.run(a_in, B, C)
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    kern.checkStatus()
    times.sort()
    med = times[len(times) // 2]
    print(f"kernel {inConfig.kernelFuncName}")
    print(f"grid {inConfig.gridDims()} block {inConfig.blockDims()} smem {inConfig.sharedMem()} B")
    print(f"median {med:.4f} ms  {2.0 * a.m * a.n * a.k / (med * 1e9):.1f} TFLOP/s over {a.launches} launches")
    if a.timeline:
        print_timeline(C, kpm.KERNEL_VARIANT)
        return 0
    if a.cublas:
        ref_out = torch.empty_like(C)
        lib_times = []
        for i in range(a.warmup + a.launches):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            torch.matmul(A, B, out=ref_out)
            e.record()
            torch.cuda.synchronize()
            if i >= a.warmup:
                lib_times.append(s.elapsed_time(e))
        lib_times.sort()
        lib = lib_times[len(lib_times) // 2]
        print(f"torch.matmul (cuBLAS) median {lib:.4f} ms  {2.0 * a.m * a.n * a.k / (lib * 1e9):.1f} TFLOP/s")
    if not a.no_check:
        rows = min(a.m, 512)
        ref = (A[:rows].double() @ B.double()) if tdt == torch.float32 else (A[:rows].float() @ B.float())
        diff = (C[:rows].to(ref.dtype) - ref).abs()
        rms = ref.pow(2).mean().sqrt()
        max_rel = (diff / torch.maximum(ref.abs(), rms)).max().item()
        tol = 1e-4 if tdt == torch.float32 else 2e-2
        print(f"max_rel (first {rows} rows, device reference) {max_rel:.3e}  tolerance {tol}  "
              f"{'OK' if max_rel <= tol else 'FAIL'}")
        return 0 if max_rel <= tol else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
