"""Generates tests/golden/*.npz: small seeded GEMM cases with the outputs of the REFERENCE'S OWN
``hostMatmul`` (matmul.cpp:2351-2360), compiled from the reference tree by oracle/build_oracle.py.

Run in a container that has the reference tree:   python tests/golden/make_golden.py
Each fixture holds A (M x K), B (K x N), C32 = hostMatmul<float>(A^T, B), C64 = hostMatmul<double>.
Inputs are uniform[-1,1) rounded to multiples of 2^-8 (exact in bf16-free fp32 products is not
required; the rounding just keeps the files compressible).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import build_oracle, oracle  # noqa: E402

CASES = {
    # name: (M, N, K, seed)
    "tile_128x64x64": (128, 64, 64, 1),          # one tensor-core tile, one or two K blocks
    "multi_256x128x96": (256, 128, 96, 2),       # several tiles, K = 3 blocks of 32
    "ref_tile_64x48x32": (64, 48, 32, 3),        # the reference's own test tile (test.py:20-57)
    "ragged_33x17x5": (33, 17, 5, 4),            # oracle-only: not a multiple of any tile
    "empty_k_8x8x0": (8, 8, 0, 5),               # K = 0 -> C stays zero
}


def main():
    build_oracle.build_port()
    if build_oracle.build_ref() is None:
        raise SystemExit("reference tree not found: cannot generate golden vectors")
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name, (M, N, K, seed) in CASES.items():
        rng = np.random.default_rng(seed)
        A = (np.floor(rng.uniform(-1, 1, size=(M, K)) * 256) / 256).astype(np.float32)
        B = (np.floor(rng.uniform(-1, 1, size=(K, N)) * 256) / 256).astype(np.float32)
        At = np.ascontiguousarray(A.T)
        if K > 0:
            C32 = oracle.ref_host_matmul(At, B)
            C64 = oracle.ref_host_matmul(At.astype(np.float64), B.astype(np.float64))
        else:
            C32 = np.zeros((M, N), np.float32)
            C64 = np.zeros((M, N), np.float64)
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), A=A, B=B, C32=C32, C64=C64)
        print(name, A.shape, B.shape, float(np.abs(C64).max()))


if __name__ == "__main__":
    main()
