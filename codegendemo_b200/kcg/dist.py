"""M-sharded multi-GPU GEMM: rank r of G computes ``C[r*M/G:(r+1)*M/G, :] = A[rows] @ B``.

The reference runs on one device only (Runtime/python/kcg/KCGTask.py:77-87, Benchmark.sh:4); this is
the one multi-GPU capability added around its kernel. Rows of C are independent given all of B, so the
GEMM needs no exchange: every rank runs the single-GPU kernel on its slab against a replicated B. The
optional all-gather of the C slabs is a plain NCCL collective on its own events so it can be timed apart
from the GEMM. One process per GPU (``torch.distributed``; ``nccl`` on GPUs, ``gloo`` in CPU tests).
"""
from typing import Tuple


def shard_rows(M: int, world_size: int, rank: int, block_m: int = 1) -> Tuple[int, int]:
    """[start, end) rows of rank ``rank``. M must split evenly into slabs that are multiples of
    ``block_m`` (the kernel's BLOCK_SIZE_M), as the kernels require M % BLOCK_SIZE_M == 0."""
    if M % world_size != 0:
        raise ValueError(f"M={M} does not split evenly over {world_size} ranks")
    slab = M // world_size
    if slab % block_m != 0:
        raise ValueError(f"slab of {slab} rows is not a multiple of BLOCK_SIZE_M={block_m}")
    return rank * slab, (rank + 1) * slab


def shard_config(kpm_json: dict, world_size: int) -> dict:
    """The per-rank tuning config: same keys, M_SIZE divided by the number of ranks."""
    out = dict(kpm_json)
    start, end = shard_rows(int(kpm_json["M_SIZE"]), world_size, 0, int(kpm_json["BLOCK_SIZE_M"]))
    out["M_SIZE"] = end - start
    return out


def replicate_b(b_local, src: int = 0, group=None):
    """Broadcast B from ``src`` so every rank holds the full K x N operand (outside any timed region)."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(b_local, src=src, group=group)
    return b_local


def all_gather_c(c_slab, c_full=None, group=None):
    """Gathers the row slabs into the full M x N matrix on every rank (in rank order)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if c_full is None:
        c_full = torch.empty((c_slab.shape[0] * world, c_slab.shape[1]), dtype=c_slab.dtype, device=c_slab.device)
    if world == 1:
        c_full.copy_(c_slab)
    else:
        dist.all_gather_into_tensor(c_full, c_slab.contiguous(), group=group)
    return c_full


def max_over_ranks(value_ms: float, device=None, group=None) -> float:
    """Device time of a multi-GPU step = the slowest rank's."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value_ms)
    t = torch.tensor([value_ms], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
