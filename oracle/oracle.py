"""TEST INFRASTRUCTURE — CPU oracle for C = A @ B as the reference defines and checks it.

Not part of the product: only tests/, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may
import this module; ``codegendemo_b200`` never does.

What it restates (file:line in the reference):
  * ``host_matmul`` / ``naive_matmul``  — Runtime/python/kcg/KCGTask.py:94 (``torch.matmul(a, b)`` is
    the reference's correctness oracle; it runs it on the GPU through rocBLAS, here the same call
    runs on host tensors), at the precision the north-star names: fp64 for fp32 inputs, fp32
    accumulation for bf16/fp16 inputs.
  * ``c_host_matmul``                   — matmul.cpp:2351-2360 (``hostMatmul``: i, j, k loops,
    ``C[i*N+j] += A[k*M+i] * B[k*N+j]``) and src/lib/Operators/Matmul.cc:41-66, via oracle/host_matmul.c.
  * ``reference_allclose``              — KCGTask.py:177 (``torch.allclose(c, D, atol=1e-1, rtol=1e-1)``).
  * ``compare_with_error``              — KCGTask.py:67-74 (count of elements failing both an absolute
    and a relative bound, and the max absolute error).

Pinning. The reference stores no input/output vectors for this path (inputs are unseeded
``torch.randn``). The C restatement is pinned against the reference's own ``hostMatmul`` compiled from
the reference tree (oracle/_ref, see build_oracle.py): tests/golden/*.npz hold its outputs and the
restatement reproduces them bit for bit. The arithmetic of ``torch.matmul`` itself lives in PyTorch's
CPU BLAS (torch 2.11.0+cu128 here; the reference pins no version): for that library call parity is
unpinned by the reference, and the tests cross-check it against the pinned C restatement instead.
"""
import ctypes
import math
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_port = None
_ref = None


def _load(path):
    lib = ctypes.CDLL(path)
    return lib


def port_lib():
    """libkcg_oracle.so (built on demand from host_matmul.c; gcc is the only requirement)."""
    global _port
    if _port is None:
        path = os.path.join(HERE, "_build", "libkcg_oracle.so")
        if not os.path.exists(path):
            from oracle.build_oracle import build_port
            path = build_port()
        _port = _load(path)
        _port.kcg_oracle_verify_f32.restype = ctypes.c_long
    return _port


def ref_lib():
    """The reference's own hostMatmul (oracle/_ref/libkcg_ref.so) or None if it was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libkcg_ref.so")
        if not os.path.exists(path):
            return None
        _ref = _load(path)
    return _ref


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def c_host_matmul(A: np.ndarray, B: np.ndarray, a_transposed: bool, accumulate_into: np.ndarray = None) -> np.ndarray:
    """Sequential-k GEMM in the element type of A (float32 or float64). ``A`` is K x M when
    ``a_transposed`` (the layout the reference's kernels and hostMatmul take), else M x K."""
    assert A.dtype == B.dtype and A.dtype in (np.float32, np.float64)
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    K, N = B.shape
    M = A.shape[1] if a_transposed else A.shape[0]
    assert (A.shape[0] if a_transposed else A.shape[1]) == K
    C = np.zeros((M, N), dtype=A.dtype) if accumulate_into is None else np.ascontiguousarray(accumulate_into)
    fn = port_lib().kcg_oracle_matmul_f32 if A.dtype == np.float32 else port_lib().kcg_oracle_matmul_f64
    fn(_ptr(A), _ptr(B), _ptr(C), M, N, K, int(bool(a_transposed)), int(accumulate_into is not None))
    return C


def c_host_matmul_acc64(A: np.ndarray, B: np.ndarray, a_transposed: bool) -> np.ndarray:
    """float32 inputs, float64 accumulation (the 'fp64 host GEMM' bar for fp32 kernels)."""
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    K, N = B.shape
    M = A.shape[1] if a_transposed else A.shape[0]
    C = np.zeros((M, N), dtype=np.float64)
    port_lib().kcg_oracle_matmul_f32_acc64(_ptr(A), _ptr(B), _ptr(C), M, N, K, int(bool(a_transposed)))
    return C


def ref_host_matmul(At: np.ndarray, B: np.ndarray) -> np.ndarray:
    """The reference's compiled hostMatmul on A stored K x M. Raises if oracle/_ref was not built."""
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libkcg_ref.so not built (needs the reference tree)")
    At = np.ascontiguousarray(At)
    B = np.ascontiguousarray(B)
    K, M = At.shape
    N = B.shape[1]
    C = np.zeros((M, N), dtype=At.dtype)
    fn = lib.ref_host_matmul_f32 if At.dtype == np.float32 else lib.ref_host_matmul_f64
    fn(_ptr(At), _ptr(B), _ptr(C), M, N, K)
    return C


def host_matmul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """The reference's check, ``torch.matmul(a, b)``, on host tensors at oracle precision:
    fp32 inputs -> float64 result; bf16/fp16 inputs -> float32 accumulation and result."""
    A = A.detach().cpu()
    B = B.detach().cpu()
    if A.dtype == torch.float32:
        return torch.matmul(A.double(), B.double())
    return torch.matmul(A.float(), B.float())


def host_matmul_fused(A, B, alpha=1.0, beta=0.0, C=None, bias=None, relu=False) -> torch.Tensor:
    """Checker for the fused epilogue, ``act(alpha * A @ B + beta * C + bias)``, on the host at
    oracle precision. The reference has no fused epilogue (it only sketches matmul -> bias/ReLU
    chains), so this composes its check, ``torch.matmul``, with the elementwise steps: parity of the
    extension is pinned to that composition, not to reference output."""
    out = host_matmul(A, B)
    out = out * alpha
    if beta != 0.0:
        out = out + beta * C.detach().cpu().to(out.dtype)
    if bias is not None:
        out = out + bias.detach().cpu().to(out.dtype)[None, :]
    if relu:
        out = torch.clamp_min(out, 0.0)
    return out


# ------------------------------------------------------------------ seeded inputs
def make_inputs(M: int, N: int, K: int, dtype: torch.dtype, dist: str = "uniform", seed: int = 0):
    """Seeded synthetic A (M x K) and B (K x N) on the host, identical bytes on every machine.

    ``uniform``: i.i.d. uniform[-1, 1) (the fp32 configs); ``normal``: normal(0,1)/sqrt(K) (the bf16
    configs). A is drawn first, then B, from one CPU generator; low-precision dtypes are cast
    after generation.
    """
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        A = torch.rand(M, K, generator=g) * 2 - 1
        B = torch.rand(K, N, generator=g) * 2 - 1
    elif dist == "normal":
        A = torch.randn(M, K, generator=g) / math.sqrt(K)
        B = torch.randn(K, N, generator=g) / math.sqrt(K)
    else:
        raise ValueError(dist)
    return A.to(dtype), B.to(dtype)


# ------------------------------------------------------------------ error metrics
def rel_errors(c: torch.Tensor, ref: torch.Tensor) -> dict:
    """Error figures of ``c`` against the oracle result ``ref`` (both on host).

    max_rel        max_ij |c - ref| / max(|ref_ij|, rms(ref))      — the tolerance gate
    max_rel_eps2   same with the floor lowered to 1e-2 * rms(ref)  — reported, stricter near zeros
    normwise       ||c - ref||_F / ||ref||_F
    allclose_ref   the reference's own flag: allclose(c, ref, atol=1e-1, rtol=1e-1) (KCGTask.py:177)
    """
    c = c.detach().cpu().double()
    ref = ref.detach().cpu().double()
    diff = (c - ref).abs()
    rms = ref.pow(2).mean().sqrt().clamp_min(1e-300)
    out = {
        "max_rel": (diff / torch.maximum(ref.abs(), rms)).max().item(),
        "max_rel_eps2": (diff / torch.maximum(ref.abs(), 1e-2 * rms)).max().item(),
        "normwise": (diff.norm() / ref.norm().clamp_min(1e-300)).item(),
        "max_abs": diff.max().item(),
        "allclose_ref": bool(torch.allclose(c, ref, atol=1e-1, rtol=1e-1)),
        "nan": bool(torch.isnan(c).any().item()),
    }
    if out["nan"]:
        out["max_rel"] = out["max_rel_eps2"] = out["normwise"] = float("inf")
    return out


def reference_allclose(c: torch.Tensor, ref: torch.Tensor) -> bool:
    return bool(torch.allclose(c.detach().cpu().double(), ref.detach().cpu().double(), atol=1e-1, rtol=1e-1))


def compare_with_error(t1: torch.Tensor, t2: torch.Tensor, abs_error=1e-2, rel_error=1e-2):
    """(number of elements whose absolute AND relative difference exceed the bounds, max abs diff)."""
    t1 = t1.detach().cpu().double()
    t2 = t2.detach().cpu().double()
    abs_diff = (t1 - t2).abs()
    rel_diff = abs_diff / (t1.abs() + 1e-5)
    mask = (abs_diff > abs_error) & (rel_diff > rel_error)
    return int(mask.sum().item()), float(abs_diff.max().item())


# Tolerances the north-star states, on ``max_rel``.
TOL_FP32 = 1e-4   # fp32 (3xTF32 or FFMA) against the fp64 host GEMM
TOL_16BIT = 2e-2  # bf16 / fp16 against fp32 accumulation


def tolerance_for(dtype: torch.dtype) -> float:
    return TOL_FP32 if dtype == torch.float32 else TOL_16BIT
