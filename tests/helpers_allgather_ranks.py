"""Rank body of the two-GPU fused all-gather test (launched with torch.distributed.run).

Each rank computes its row slab of C = A @ B with one fused launch that stores every finished tile
into its own full C and into the peer's (mapped through CUDA IPC), then checks the FULL matrix it
holds against the host oracle. No kernel waits on another: completion is stream synchronise + barrier.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from codegendemo_b200.kcg.dist import SymmetricC, matmul_allgather, shard_rows  # noqa: E402
from codegendemo_b200.kcg.matmul_op import build_kernel, default_config  # noqa: E402
from codegendemo_b200.kcg.Utils import EnumKernelDType as E  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    M, N, K = 2048, 1024, 1024
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=9)
    ref = oracle.host_matmul(A, B)
    for keys in (dict(), dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=512, BLOCK_SIZE_N=256, NUM_STAGES=4),
                 dict(LOCAL_SPLIT_U=2),
                 dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)):
        r0, r1 = shard_rows(M, world, rank, keys.get("BLOCK_SIZE_M", 128))
        _, kern = build_kernel(default_config(r1 - r0, N, K, E.bfloat16, **keys), local)
        sym = SymmetricC(M, N, 2, rank, world, local)
        full = sym.full(torch.bfloat16)
        full.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()  # every copy is poisoned before anyone stores into it
        a, b = A[r0:r1].contiguous().cuda(), B.cuda()
        matmul_allgather(kern, a, b, sym)
        kern.checkStatus()  # synchronises the stream
        dist.barrier()
        err = oracle.rel_errors(full, ref)
        assert not err["nan"], f"rank {rank}: part of the full C was never written ({keys})"
        assert err["max_rel"] <= oracle.TOL_16BIT, (rank, keys, err)
        dist.barrier()
        sym.close()
        dist.barrier()
        sym.free()
    print(f"ALLGATHER_OK rank {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
