"""Roofline arithmetic shared by ``bench.py`` and ``kcg.sweep``.

A GEMM of M x N x K does 2*M*N*K flop on elt*(M*K + K*N + M*N) algorithmic bytes. Its ceiling is the lower of
the tensor (or FFMA) peak of its data type and arithmetic intensity x HBM bandwidth; the skinny shapes of the
rectangular sweep (M = 128) sit on the HBM side. Denominators come from a peaks file measured on the machine
(a STREAM-style copy and a cuBLAS bf16 GEMM) when one is given, else from the stated fallback figures.
"""
import json
import os
from typing import Optional

NOMINAL_BF16_TFLOPS = 2250.0   # dense fp16 / bf16, datasheet
NOMINAL_TF32_TFLOPS = 1100.0   # dense TF32, datasheet; fp32 run as 3xTF32 has a third of it
FFMA_TFLOPS = 74.0             # 148 SMs x 128 lanes x 2 flop x 1.965 GHz
FALLBACK = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def load_peaks(path: Optional[str] = None) -> dict:
    """Peaks from a JSON file with keys hbm_gbs, bf16_tflops, bf16_tflops_sustained (source: "measured"),
    else the fallback figures (source: "fallback")."""
    if path and os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return dict(FALLBACK)


def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


def gemm_bytes(m: int, n: int, k: int, elt: int) -> int:
    return elt * (m * k + k * n + m * n)


def tensor_peak_tflops(dtype: str, simt: bool, peaks: dict, nominal: bool = False) -> float:
    """Compute-side ceiling: FFMA pipe for the SIMT kernel, TF32 / 3 for fp32 as 3xTF32, the bf16 figure
    (measured cuBLAS burst, or nominal when asked) for 16-bit data."""
    if simt:
        return FFMA_TFLOPS
    if dtype in ("float32", "fp32", "f32"):
        return NOMINAL_TF32_TFLOPS / 3.0
    return NOMINAL_BF16_TFLOPS if nominal else peaks["bf16_tflops"]


def shape_roofline(m: int, n: int, k: int, elt: int, tensor_peak: float, hbm_gbs: float) -> dict:
    """{"bound": "hbm" | "tensor", "peak": TFLOP/s ceiling, "hbm_tflops": AI x bandwidth, "ai": flop per byte}."""
    ai = gemm_flops(m, n, k) / gemm_bytes(m, n, k, elt)
    hbm_tflops = ai * hbm_gbs / 1e3
    bound = "hbm" if hbm_tflops < tensor_peak else "tensor"
    return {"bound": bound, "peak": min(tensor_peak, hbm_tflops), "hbm_tflops": hbm_tflops, "ai": ai}
