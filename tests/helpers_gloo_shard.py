"""Two gloo ranks on CPU: M-sharded GEMM plumbing (shard_rows, replicate_b, all_gather_c, max_over_ranks)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from codegendemo_b200.kcg import dist as kdist  # noqa: E402

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
M, N, K = 512, 96, 64
g = torch.Generator().manual_seed(0)
A = torch.rand(M, K, generator=g) * 2 - 1
B_full = torch.rand(K, N, generator=g) * 2 - 1
B = B_full.clone() if rank == 0 else torch.zeros(K, N)
kdist.replicate_b(B, src=0)
assert torch.equal(B, B_full)
r0, r1 = kdist.shard_rows(M, world, rank, 128)
c_slab = A[r0:r1] @ B
c_full = kdist.all_gather_c(c_slab)
assert torch.allclose(c_full, A @ B_full, atol=1e-5)
t = kdist.max_over_ranks(1.0 + rank)
assert t == float(world)
print(f"SHARD_OK rank{rank}", flush=True)
dist.barrier()
dist.destroy_process_group()
