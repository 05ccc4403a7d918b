"""Run, time and check ONE fused attention problem from the command line (the counterpart of run_single for
``kcg_attention_fwd``): a small, self-ending workload for profilers and a quick check of the kernel.

    python -m codegendemo_b200.kcg.run_attention --heads 16 --sq 2048 --sk 2048 --d 128 --launches 3 --warmup 2
"""
import argparse
import math
import sys


def main(argv=None) -> int:
    import torch
    from codegendemo_b200.kcg.matmul_op import attention_fused, attention_status
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--sq", type=int, default=2048)
    ap.add_argument("--sk", type=int, default=0, help="keys per head (default: --sq)")
    ap.add_argument("--d", type=int, default=128, choices=[64, 128])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--library", action="store_true",
                    help="also launch torch's scaled_dot_product_attention the same number of times (a comparison "
                         "line, and a second kernel in a profiler's launch list)")
    ap.add_argument("--no-check", action="store_true")
    a = ap.parse_args(argv)
    sk = a.sk or a.sq
    tdt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    torch.cuda.set_device(a.device)
    dev = f"cuda:{a.device}"
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(a.heads, a.sq, a.d, generator=g, device=dev).to(tdt)
    k = torch.randn(a.heads, sk, a.d, generator=g, device=dev).to(tdt)
    v = torch.randn(a.heads, sk, a.d, generator=g, device=dev).to(tdt)
    o = torch.empty_like(q)
    flops = 4.0 * a.heads * a.sq * sk * a.d

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(a.launches):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    med = timed(lambda: attention_fused(q, k, v, out=o))
    attention_status(a.device)
    print(f"fused attention {a.heads} heads x {a.sq} x {sk} x {a.d} {a.dtype}: median {med:.4f} ms  "
          f"{flops / (med * 1e9):.1f} TFLOP/s over {a.launches} launches")
    if a.library:
        lib = timed(lambda: torch.nn.functional.scaled_dot_product_attention(q[None], k[None], v[None]))
        print(f"torch scaled_dot_product_attention median {lib:.4f} ms  {flops / (lib * 1e9):.1f} TFLOP/s")
    if not a.no_check:
        h = a.heads // 2
        rows = min(a.sq, 256)
        s = (q[h, :rows].float() @ k[h].float().t()) / math.sqrt(a.d)
        ref = torch.softmax(s, dim=-1) @ v[h].float()
        err = ((o[h, :rows].float() - ref).abs().max() / ref.abs().max()).item()
        print(f"max_rel (head {h}, first {rows} rows, device fp32 composition) {err:.3e}  tolerance 0.02  "
              f"{'OK' if err <= 2e-2 else 'FAIL'}")
        return 0 if err <= 2e-2 else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
