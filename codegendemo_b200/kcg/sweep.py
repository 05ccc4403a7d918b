"""Measures the GEMM kernels on a list of shapes and prints one markdown table row per case.

    python -m codegendemo_b200.kcg.sweep                  # 1024^3, 4096^3, 8192^3 and the rectangular sweep
    python -m codegendemo_b200.kcg.sweep --only rect --json out.json

Per case: median and best of single-launch CUDA-event timings (the reference's protocol,
Runtime/python/kcg/KCGTask.py:171-181), TFLOP/s, fraction of the per-shape roofline
min(tensor peak, arithmetic intensity x HBM bandwidth), achieved GB/s, the same shape through
``torch.matmul`` on the device (cuBLAS, a comparison only), max relative error against a
higher-precision device GEMM, and ``torch.matmul`` on host tensors (the reference's CPU oracle call)
timed on all host threads. Inputs are seeded: uniform[-1, 1) for fp32 and the rectangular shapes,
normal(0,1)/sqrt(K) for the square 16-bit cases. The JSON record also holds the mean over a back-to-back
batch of launches (clock droop under the power cap) and says whether the case ran on a warm L2;
``--cold`` rotates operand copies for the cases that fit L2 (the strategy the reference's authors
float for their unstable timings, doc/结果汇总.md:12).
"""
import argparse
import json
import math
import os
import sys
import time

from codegendemo_b200.kcg.matmul_op import build_kernel, default_config, tuned_config
from codegendemo_b200.kcg.Utils import EnumKernelDType as E

from codegendemo_b200.kcg import roofline as rl

SIMT_128 = dict(KERNEL_VARIANT=1, BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=16, THREAD_SIZE_M=8,
                THREAD_SIZE_N=8, BLOCK_LAYOUT_M=4, BLOCK_LAYOUT_N=2, WARP_LAYOUT_M=4, WARP_LAYOUT_N=8,
                WARP_SCATTER_WIDTH_A=4, WARP_SCATTER_WIDTH_B=4, THREAD_SCATTER_WIDTH_A=4, THREAD_SCATTER_WIDTH_B=4)


def cases(which: str):
    out = []
    if which in ("all", "square"):
        out += [("c1 1024^3 fp32 3xTF32", 1024, 1024, 1024, E.float32, "uniform", None),
                ("c1 1024^3 fp32 SIMT", 1024, 1024, 1024, E.float32, "uniform", SIMT_128),
                ("c2 4096^3 fp32 3xTF32", 4096, 4096, 4096, E.float32, "uniform", None),
                ("c2 4096^3 fp32 SIMT", 4096, 4096, 4096, E.float32, "uniform", SIMT_128),
                ("c3 8192^3 bf16", 8192, 8192, 8192, E.bfloat16, "normal", None),
                ("c3 8192^3 fp16", 8192, 8192, 8192, E.float16, "normal", None)]
    if which in ("all", "rect"):
        for nk in (4096, 11008):
            for m in (128, 512, 2048):
                out.append((f"c4 {m}x{nk}x{nk} fp32", m, nk, nk, E.float32, "uniform", None))
                out.append((f"c4 {m}x{nk}x{nk} bf16", m, nk, nk, E.bfloat16, "uniform", None))
    return out


def run_case(tag, M, N, K, edt, dist, keys, device, iters, cpu, cold=False, peaks=None):
    import torch
    tdt = {E.float32: torch.float32, E.bfloat16: torch.bfloat16, E.float16: torch.float16}[edt]
    g = torch.Generator().manual_seed(0)
    if dist == "uniform":
        A = (torch.rand(M, K, generator=g) * 2 - 1).to(tdt)
        B = (torch.rand(K, N, generator=g) * 2 - 1).to(tdt)
    else:
        A = (torch.randn(M, K, generator=g) / math.sqrt(K)).to(tdt)
        B = (torch.randn(K, N, generator=g) / math.sqrt(K)).to(tdt)
    dev = f"cuda:{device}"
    a, b = A.to(dev), B.to(dev)
    c = torch.empty(M, N, dtype=tdt, device=dev)
    kpm = tuned_config(M, N, K, edt) if keys is None else default_config(M, N, K, edt, **keys)
    inc, kern = build_kernel(kpm, device)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2], ts[0]

    warm_l2 = (a.numel() + b.numel() + c.numel()) * a.element_size() < 126e6
    if cold and warm_l2:
        # The whole problem fits L2, so repeats run on warm lines. Rotate over enough copies of the
        # operands to push each launch's working set out of the 126 MB L2 before it comes round again.
        copies = int(2 * 126e6 // ((a.numel() + b.numel() + c.numel()) * a.element_size())) + 2
        sets = [(a.clone(), b.clone(), torch.empty_like(c)) for _ in range(copies)]
        turn = [0]

        def launch():
            x, y, z = sets[turn[0] % copies]
            turn[0] += 1
            kern.run(x, y, z)
    else:
        def launch():
            kern.run(a, b, c)
    med, best = timed(launch)
    kern.checkStatus()
    # mean over a back-to-back batch (>= 50 launches and >= 0.2 s): shows the clock droop under the
    # power cap that single-launch medians hide
    n_batch = max(50, int(0.2e3 / max(med, 1e-3)))
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(n_batch):
        launch()
    e0.record()
    torch.cuda.synchronize()
    batch_ms = s0.elapsed_time(e0) / n_batch
    kern.run(a, b, c)  # the accuracy check below reads c
    lib_med, _ = timed(lambda: torch.matmul(a, b))
    rows = min(M, 512)
    ref = (a[:rows].double() @ b.double()) if tdt == torch.float32 else (a[:rows].float() @ b.float())
    diff = (c[:rows].to(ref.dtype) - ref).abs()
    rms = ref.pow(2).mean().sqrt()
    max_rel = float((diff / torch.maximum(ref.abs(), rms)).max().item())
    flops = rl.gemm_flops(M, N, K)
    eb = 4 if tdt == torch.float32 else 2
    nbytes = rl.gemm_bytes(M, N, K, eb)
    variant = int(inc.kernelInfo["kernel"])
    peaks = peaks or rl.load_peaks(None)
    # "of dense peak" is quoted against the nominal figures, "of roofline" against min(that, AI x HBM bandwidth)
    peak = rl.tensor_peak_tflops(str(tdt).replace("torch.", ""), variant == 1, peaks, nominal=True)
    roof = rl.shape_roofline(M, N, K, eb, peak, peaks["hbm_gbs"])["peak"]  # TFLOP/s
    rec = {"case": tag, "m": M, "n": N, "k": K, "dtype": str(tdt).replace("torch.", ""),
           "kernel": {1: "simt", 2: "tcgen05", 3: "tf32x1", 4: "tcgen05 pair", 5: "tcgen05 cluster split-K"}.get(
               variant, str(variant)),
           "tile": f"{kpm.BLOCK_SIZE_M}x{kpm.BLOCK_SIZE_N}x{kpm.BLOCK_SIZE_K}", "ms_median": med, "ms_best": best,
           "tflops": flops / med / 1e9, "gbs": nbytes / med / 1e6, "roofline_tflops": roof,
           "frac_roofline": flops / med / 1e9 / roof, "frac_peak": flops / med / 1e9 / peak,
           "cublas_tflops": flops / lib_med / 1e9, "max_rel": max_rel,
           "batch_launches": n_batch, "ms_batch_mean": batch_ms, "tflops_batch": flops / batch_ms / 1e9,
           "l2": "cold (rotating operand copies)" if (cold and warm_l2) else ("warm (problem fits L2)" if warm_l2 else "larger than L2")}
    if cpu:
        threads = os.cpu_count() or 1
        torch.set_num_threads(threads)
        Af, Bf = A.float(), B.float()
        mrows = M if flops < 3e11 else max(128, int(M * 3e11 / flops) // 128 * 128)
        torch.matmul(Af[:8], Bf)
        t0 = time.perf_counter()
        torch.matmul(Af[:mrows], Bf)
        dt = (time.perf_counter() - t0) * M / mrows  # scaled linearly in M when a row slab was timed
        rec.update({"cpu_ms": dt * 1e3, "cpu_threads": threads,
                    "cpu_kind": "torch_fp32" + ("" if mrows == M else f" (extrapolated from {mrows} rows)")})
    return rec


def to_row(r):
    cpu = f"{r['cpu_ms']:.1f} ({r['cpu_threads']}){'*' if 'extrapolated' in r.get('cpu_kind', '') else ''}" if "cpu_ms" in r else ""
    return (f"| {r['case']} | {r['kernel']} {r['tile']} | {r['ms_median']:.4f} / {r['ms_best']:.4f} | "
            f"{r['tflops']:.1f} | {100 * r['frac_peak']:.1f} % | {100 * r['frac_roofline']:.1f} % | {r['gbs']:.0f} | "
            f"{r['cublas_tflops']:.1f} | {r['max_rel']:.1e} | {cpu} |")


def main(argv=None) -> int:
    import torch
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", default="all", choices=["all", "square", "rect"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cold", action="store_true",
                    help="problems that fit L2 rotate over copies of their operands, so every launch starts cold")
    ap.add_argument("--json", default="")
    ap.add_argument("--peaks", default="", help="JSON file with measured hbm_gbs / bf16_tflops of this machine "
                    "(default: the stated fallback figures)")
    a = ap.parse_args(argv)
    peaks = rl.load_peaks(a.peaks or None)
    torch.cuda.set_device(a.device)
    print("| case | kernel, tile | ms median / best | TFLOP/s | of dense peak | of roofline | GB/s | cuBLAS TFLOP/s | "
          "max rel err | CPU ms (threads) |")
    print("|---|---|---|---|---|---|---|---|---|---|")
    recs = []
    for (tag, M, N, K, edt, dist, keys) in cases(a.only):
        r = run_case(tag, M, N, K, edt, dist, keys, a.device, a.iters, not a.no_cpu, cold=a.cold, peaks=peaks)
        recs.append(r)
        print(to_row(r), flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(recs, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
