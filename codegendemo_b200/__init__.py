"""B200-native (sm_100a) implementation of the GEMM hot path of Xiebaokang/CodeGenDemo ("KCG").

``codegendemo_b200.kcg`` mirrors the reference's Python operator API (Runtime/python/kcg);
``libkcg_b200.so`` (C ABI in ``include/kcg_b200.h``) compiles, loads and launches the CUDA kernels
under ``csrc/kernels``. There is no CPU or PyTorch fallback for the GEMM itself.
"""
__version__ = "0.1.0"
