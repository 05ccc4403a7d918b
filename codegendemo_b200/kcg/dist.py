"""M-sharded multi-GPU GEMM: rank r of G computes ``C[r*M/G:(r+1)*M/G, :] = A[rows] @ B``.

The reference runs on one device only (Runtime/python/kcg/KCGTask.py:77-87, Benchmark.sh:4); this is
the one multi-GPU capability added around its kernel. Rows of C are independent given all of B, so the
GEMM needs no exchange: every rank runs the single-GPU kernel on its slab against a replicated B. The
optional all-gather of the C slabs is either a plain NCCL collective on its own events, so it can be
timed apart from the GEMM, or fused into the kernel: ``SymmetricC`` maps every GPU's full C into every
rank and the epilogue stores each finished tile into all of them over NVLink (``matmul_allgather``).
One process per GPU (``torch.distributed``; ``nccl`` on GPUs, ``gloo`` in CPU tests).
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


# ------------------------------------------------------------- fused all-gather of C
def slab_targets(rank: int, bases, slab_bytes: int):
    """Where rank ``rank`` writes its slab: (address inside its own full C, addresses inside every
    other rank's full C). ``bases[i]`` is the device address of rank i's full C as mapped into this
    process; slab r lives at byte offset r * slab_bytes in each of them."""
    if not 0 <= rank < len(bases):
        raise ValueError(f"rank {rank} outside 0..{len(bases) - 1}")
    if len(bases) - 1 > 7:
        raise ValueError("at most 8 ranks (7 peers) share one fused all-gather")
    off = rank * slab_bytes
    return bases[rank] + off, [b + off for i, b in enumerate(bases) if i != rank]


class _DevicePointer:
    """Lets torch view raw device memory (``torch.as_tensor(obj, device='cuda')``)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


class SymmetricC:
    """The full M x N result of an M-sharded product, one copy per GPU, every copy mapped into
    every rank's process (CUDA IPC through ``kcg_peer_alloc`` / ``kcg_peer_open``), so that a
    kernel can store its tiles straight into all of them. One process per GPU on one node.

    ``exchange`` swaps the 64-byte handles; it defaults to ``torch.distributed.all_gather_object``."""

    def __init__(self, M: int, N: int, elem_bytes: int, rank: int, world: int, device: int, exchange=None,
                 group=None):
        import ctypes
        from codegendemo_b200 import _lib
        if M % world:
            raise ValueError(f"M={M} does not split evenly over {world} ranks")
        self.M, self.N, self.elem_bytes = M, N, elem_bytes
        self.rank, self.world, self.device = rank, world, device
        self.slab_bytes = (M // world) * N * elem_bytes
        lib = _lib.get_lib()
        ptr, handle = ctypes.c_uint64(0), ctypes.create_string_buffer(64)
        _lib.check(lib.kcg_peer_alloc(int(device), ctypes.c_uint64(M * N * elem_bytes), ctypes.byref(ptr), handle))
        self._own = ptr.value
        if exchange is None:
            import torch.distributed as dist

            def exchange(mine):
                out = [None] * world
                dist.all_gather_object(out, mine, group=group)
                return out
        handles = exchange(handle.raw) if world > 1 else [handle.raw]
        self.bases, self._opened = [], []
        for r, h in enumerate(handles):
            if r == rank:
                self.bases.append(self._own)
                continue
            p = ctypes.c_uint64(0)
            _lib.check(lib.kcg_peer_open(int(device), ctypes.c_char_p(h), ctypes.byref(p)))
            self.bases.append(p.value)
            self._opened.append(p.value)
        self.local_slab, self.peer_slabs = slab_targets(rank, self.bases, self.slab_bytes)

    def full(self, dtype):
        """This GPU's full C as a torch tensor (no copy)."""
        import torch
        typestr = {torch.bfloat16: "<i2", torch.float16: "<f2", torch.float32: "<f4"}[dtype]
        t = torch.as_tensor(_DevicePointer(self._own, (self.M, self.N), typestr), device=f"cuda:{self.device}")
        return t.view(dtype) if dtype == torch.bfloat16 else t

    def close(self):
        """Unmap the peers' copies; free the own copy (call after a barrier: peers unmap first)."""
        from codegendemo_b200 import _lib
        lib = _lib.get_lib()
        for p in self._opened:
            _lib.check(lib.kcg_peer_close(int(self.device), p))
        self._opened = []

    def free(self):
        from codegendemo_b200 import _lib
        if self._own:
            _lib.check(_lib.get_lib().kcg_peer_free(int(self.device), self._own))
            self._own = 0


def matmul_allgather(kern, a_slab, b, sym: "SymmetricC", **epilogue):
    """One fused launch: this rank's slab of C = a_slab @ b lands in every GPU's full C.
    Complete everywhere after every rank synchronised its stream and a barrier."""
    kern.run(a_slab, b, sym.local_slab, peers=sym.peer_slabs, **epilogue)
