"""GPU parity tests: every kernel family through the C ABI (compile -> load -> launch) against the CPU oracle.

Tolerances (on oracle.rel_errors()['max_rel'] = max |c-ref| / max(|ref|, rms(ref))):
  fp32 kernels (3xTF32 tcgen05, FFMA SIMT) vs the fp64 host GEMM ........ 1e-4
  bf16 / fp16 kernels vs fp32 accumulation on the host ................... 2e-2
plus the reference's own flag, allclose(atol=1e-1, rtol=1e-1) (KCGTask.py:177).
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from codegendemo_b200 import _lib
from codegendemo_b200.kcg.matmul_op import build_kernel, default_config
from codegendemo_b200.kcg.Utils import EnumKernelDType as E, ToTorchType
from oracle import oracle
from tests import gpu_cases

pytestmark = pytest.mark.gpu
GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


def run_config(kpm, A, B):
    """A is M x K on the host; the kernel gets A^T (K x M, contiguous) when IS_ATRANS=1."""
    inc, kern = build_kernel(kpm, 0)
    tdt = kpm.dtypeTorch('A')
    a = (A.t().contiguous() if kpm.isATranspose else A).to(tdt).cuda()
    b = (B.t().contiguous() if kpm.IS_BTRANS else B).to(tdt).cuda()  # N x K storage when IS_BTRANS=1
    c = torch.full((kpm.M, kpm.N), float("nan"), dtype=tdt, device="cuda:0")  # poisoned output
    before = _lib.get_lib().kcg_launch_count()
    kern.run(a, b, c)
    kern.checkStatus()
    assert _lib.get_lib().kcg_launch_count() == before + 1
    return c, kern, (a, b)


@pytest.mark.parametrize("case", gpu_cases.SEEDED, ids=[c[0] for c in gpu_cases.SEEDED])
def test_seeded_case_matches_oracle(case):
    _, M, N, K, dt, dist, keys = case
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, N, K, tdt, dist, seed=0)
    c, _, _ = run_config(default_config(M, N, K, dt, **keys), A, B)
    err = oracle.rel_errors(c, oracle.host_matmul(A, B))
    assert not err["nan"], "kernel left part of C unwritten"
    assert err["max_rel"] <= oracle.tolerance_for(tdt), err
    assert err["allclose_ref"], err


@pytest.mark.parametrize("case", gpu_cases.GOLDEN, ids=[f"{c[0]}-{c[1]}-{i}" for i, c in enumerate(gpu_cases.GOLDEN)])
def test_golden_vectors(case):
    """Inputs and outputs of the reference's own hostMatmul. Golden inputs are multiples of 2^-8 in
    [-1, 1), exactly representable in bf16 and fp16, so every dtype sees the same operands."""
    name, dt, keys = case
    g = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    A, B = torch.from_numpy(g["A"]), torch.from_numpy(g["B"])
    M, N, K = gpu_cases.GOLDEN_SHAPES[name]
    tdt = ToTorchType(dt)
    assert torch.equal(A.to(tdt).float(), A) and torch.equal(B.to(tdt).float(), B)
    c, _, _ = run_config(default_config(M, N, K, dt, **keys), A, B)
    err = oracle.rel_errors(c, torch.from_numpy(g["C64"]))
    assert err["max_rel"] <= oracle.tolerance_for(tdt), err
    if dt == E.float32:
        # fp32 kernels also sit within fp32 rounding noise of the reference's fp32 result
        assert oracle.rel_errors(c, torch.from_numpy(g["C32"]).double())["max_rel"] <= 1e-4
        assert oracle.port_lib().kcg_oracle_verify_f32(
            g["C32"].ctypes.data_as(ctypes.c_void_p), c.cpu().numpy().ctypes.data_as(ctypes.c_void_p), M, N,
            ctypes.c_double(0.01)) == 0  # the reference's verify(): |host - device| < 0.01 everywhere


def test_results_are_bitwise_reproducible_including_split_k():
    for keys in (dict(), dict(LOCAL_SPLIT_U=4)):
        A, B = oracle.make_inputs(256, 512, 2048, torch.bfloat16, "normal", seed=3)
        kpm = default_config(256, 512, 2048, E.bfloat16, **keys)
        c1, kern, (a, b) = run_config(kpm, A, B)
        c2 = torch.empty_like(c1)
        for _ in range(3):
            kern.run(a, b, c2)
        kern.checkStatus()
        assert torch.equal(c1, c2)


EPILOGUES = [dict(alpha=0.5, beta=-0.75, bias=True, relu=True), dict(bias=True), dict(relu=True),
             dict(alpha=-1.25, beta=0.5), dict(alpha=2.0)]


@pytest.mark.parametrize("case", gpu_cases.FUSED, ids=[c[0] for c in gpu_cases.FUSED])
def test_fused_epilogue_matches_oracle(case):
    """c = act(alpha * a.b + beta * c + bias) through kcg_launch_gemm_ex, every kernel family and
    both store paths (whole-K tiles and the K-split reduction), against the host composition."""
    _, M, N, K, dt, dist, keys = case
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, N, K, tdt, dist, seed=4)
    g = torch.Generator().manual_seed(11)
    Cin = (torch.rand(M, N, generator=g) * 2 - 1).to(tdt)
    bias = (torch.rand(N, generator=g) * 2 - 1).to(tdt)
    kpm = default_config(M, N, K, dt, **keys)
    _, kern = build_kernel(kpm, 0)
    a = (A.t().contiguous() if kpm.isATranspose else A).cuda()
    b, bias_d = B.cuda(), bias.cuda()
    for epi in EPILOGUES:
        kw = dict(epi)
        use_bias = kw.pop("bias", False)
        beta = kw.get("beta", 0.0)
        # beta == 0 must not read C: poison it
        c = Cin.cuda() if beta != 0.0 else torch.full((M, N), float("nan"), dtype=tdt, device="cuda:0")
        kern.run(a, b, c, bias=bias_d if use_bias else None, **kw)
        kern.checkStatus()
        ref = oracle.host_matmul_fused(A, B, alpha=kw.get("alpha", 1.0), beta=beta, C=Cin,
                                       bias=bias if use_bias else None, relu=kw.get("relu", False))
        err = oracle.rel_errors(c, ref)
        assert not err["nan"], (epi, "kernel left part of C unwritten or read a poisoned C")
        assert err["max_rel"] <= oracle.tolerance_for(tdt), (epi, err)
    # the plain call on the same kernel is unchanged
    c = torch.full((M, N), float("nan"), dtype=tdt, device="cuda:0")
    kern.run(a, b, c)
    kern.checkStatus()
    assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.tolerance_for(tdt)


@pytest.mark.parametrize("case", gpu_cases.BATCHED, ids=[c[0] for c in gpu_cases.BATCHED])
def test_batched_product_matches_oracle_per_batch(case):
    """kcg_launch_gemm_batched: one launch over all batches (torch.bmm layout), checked batch by batch
    against the host oracle; then once more with a fused bias + ReLU."""
    _, batch, M, N, K, dt, dist, keys = case
    tdt = ToTorchType(dt)
    pairs = [oracle.make_inputs(M, N, K, tdt, dist, seed=20 + i) for i in range(batch)]
    A = torch.stack([p[0] for p in pairs])
    B = torch.stack([p[1] for p in pairs])
    kpm = default_config(M, N, K, dt, **keys)
    _, kern = build_kernel(kpm, 0)
    a = (A.transpose(1, 2).contiguous() if kpm.isATranspose else A).cuda()
    b = B.cuda()
    c = torch.full((batch, M, N), float("nan"), dtype=tdt, device="cuda:0")
    kern.run(a, b, c, batch=batch)
    kern.checkStatus()
    for i in range(batch):
        err = oracle.rel_errors(c[i], oracle.host_matmul(A[i], B[i]))
        assert not err["nan"] and err["max_rel"] <= oracle.tolerance_for(tdt), (i, err)
    bias = torch.linspace(-0.5, 0.5, N).to(tdt)
    c.fill_(float("nan"))
    kern.run(a, b, c, batch=batch, bias=bias.cuda(), relu=True)
    kern.checkStatus()
    for i in (0, batch - 1):
        ref = oracle.host_matmul_fused(A[i], B[i], bias=bias, relu=True)
        assert oracle.rel_errors(c[i], ref)["max_rel"] <= oracle.tolerance_for(tdt), i


def test_bmm_op_and_batched_launch_rejects_simt():
    from codegendemo_b200.kcg.matmul_op import bmm
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(8, 128, 256, generator=g) / 16).bfloat16()
    y = (torch.randn(8, 256, 256, generator=g) / 16).bfloat16()
    z = bmm(x.cuda(), y.cuda())
    torch.cuda.synchronize()
    assert oracle.rel_errors(z.reshape(-1, 256), torch.bmm(x.float(), y.float()).reshape(-1, 256))["max_rel"] <= 2e-2
    _, simt = build_kernel(default_config(256, 256, 256, E.float32, **gpu_cases.SIMT_128), 0)
    t = torch.zeros(2, 256, 256, device="cuda:0")
    with pytest.raises(_lib.KCGError) as ei:
        simt.run(t, t, t.clone(), batch=2)
    assert ei.value.code == _lib.E_BAD_CONFIG


def test_matmul_op_fuses_bias_relu_chain():
    """matmul -> bias + ReLU -> matmul, the chain the reference sketches, as two fused launches."""
    from codegendemo_b200.kcg.matmul_op import matmul
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(512, 1024, generator=g) / 32).bfloat16()
    w1 = (torch.randn(1024, 512, generator=g) / 32).bfloat16()
    w2 = (torch.randn(512, 256, generator=g) / 22).bfloat16()
    b1 = (torch.randn(512, generator=g) / 8).bfloat16()
    h = matmul(x.cuda(), w1.cuda(), bias=b1.cuda(), relu=True)
    y = matmul(h, w2.cuda())
    torch.cuda.synchronize()
    h_ref = torch.relu(x.float() @ w1.float() + b1.float()).bfloat16()
    assert oracle.rel_errors(h, h_ref.float())["max_rel"] <= 2e-2
    assert oracle.rel_errors(y, h_ref.float() @ w2.float())["max_rel"] <= 2e-2


@pytest.mark.parametrize("case", [c for c in gpu_cases.FUSED if c[0] in (
    "bf16_tma_store", "fp16_tma_store", "bf16_pair", "bf16_splitk_reduce")] + gpu_cases.ALLGATHER_EXTRA,
    ids=lambda c: c[0])
def test_fused_allgather_stores_reach_every_target(case):
    """The all-gather epilogue on one GPU: the 'peers' are three more buffers of this GPU, so the
    kernel's extra stores (staged path and K-split reduction) are checked without a second device."""
    _, M, N, K, dt, dist, keys = case
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, N, K, tdt, dist, seed=6)
    _, kern = build_kernel(default_config(M, N, K, dt, **keys), 0)
    a, b = A.cuda(), B.cuda()
    c = torch.full((M, N), float("nan"), dtype=tdt, device="cuda:0")
    peers = [torch.full((M, N), float("nan"), dtype=tdt, device="cuda:0") for _ in range(3)]
    kern.run(a, b, c, peers=peers)
    kern.checkStatus()
    assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.tolerance_for(tdt)
    for pc in peers:
        assert torch.equal(pc, c)
    # with a fused epilogue the peers receive the finished values too
    bias = torch.linspace(-1, 1, N).to(tdt).cuda()
    kern.run(a, b, c, peers=peers[:1], bias=bias, relu=True)
    kern.checkStatus()
    assert torch.equal(peers[0], c) and not torch.equal(peers[1], c)


def test_fused_allgather_rejects_kernels_without_a_staged_epilogue():
    _, kern = build_kernel(default_config(256, 256, 256, E.float32, BLOCK_SIZE_N=128), 0)
    x = torch.zeros(256, 256, device="cuda:0")
    with pytest.raises(_lib.KCGError) as ei:
        kern.run(x, x, x.clone(), peers=[x.clone()])
    assert ei.value.code == _lib.E_BAD_CONFIG


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allgather_two_gpus():
    """Two ranks, one GPU each: every rank's full C holds both slabs after one fused launch per rank."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29631",
                        os.path.join(root, "tests", "helpers_allgather_ranks.py")],
                       cwd=root, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ALLGATHER_OK") == 2, r.stdout[-3000:]


def test_host_buffer_entry_matches_device_entry():
    A, B = oracle.make_inputs(512, 512, 512, torch.bfloat16, "normal", seed=1)
    kpm = default_config(512, 512, 512, E.bfloat16)
    c, kern, _ = run_config(kpm, A, B)
    hA, hB = A.pin_memory(), B.pin_memory()
    hC = torch.empty(512, 512, dtype=torch.bfloat16).pin_memory()
    kern.runHost(hA, hB, hC)
    assert torch.equal(hC, c.cpu())
    hC2 = torch.zeros(512, 512, dtype=torch.bfloat16)  # pageable memory works too
    kern.runHost(A, B, hC2)
    assert torch.equal(hC2, c.cpu())


def test_host_buffer_entry_pipelined_slabs_match_device_entry():
    """Above 64 MiB of A + C the host entry moves row slabs through three streams. A slab launch may
    K-split its last wave differently from the whole-matrix launch, so the two results agree to fp32
    summation-order noise (a rare last-bit difference after rounding to bf16), not bit for bit."""
    M, N, K = 4096, 4096, 4096
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=8)
    kpm = default_config(M, N, K, E.bfloat16, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, NUM_STAGES=3)
    c, kern, _ = run_config(kpm, A, B)
    hA, hB = A.pin_memory(), B.pin_memory()
    hC = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    before = _lib.get_lib().kcg_launch_count()
    kern.runHost(hA, hB, hC)
    assert _lib.get_lib().kcg_launch_count() - before == 4  # 64 MiB of A + C: four slabs of four tile rows
    ref = oracle.host_matmul(A, B)
    first = hC.clone()
    assert oracle.rel_errors(first, ref)["max_rel"] <= oracle.TOL_16BIT
    dev = c.cpu()
    differing = (first != dev).float().mean().item()
    assert differing < 1e-2 and oracle.rel_errors(first, dev.float())["max_rel"] <= 1e-2
    hC.fill_(float("nan"))
    kern.runHost(hA, hB, hC)  # buffers, streams and events are reused; same slabs -> same bits
    assert torch.equal(hC, first)


def _column_checksum_ok(c, a, b, tol):
    """1^T (A B) == (1^T A) B — a full-size property that needs no O(MNK) reference."""
    lhs = c.double().sum(0)
    rhs = a.double().sum(0) @ b.double()
    scale = (a.double().abs().sum(0) @ b.double().abs()).clamp_min(1e-30)
    return ((lhs - rhs).abs() / scale).max().item() <= tol


def _check_row_blocks(c, A, B, rows, tol):
    ref = oracle.host_matmul(A[rows], B)
    err = oracle.rel_errors(c[rows.cuda()].cpu(), ref)
    assert err["max_rel"] <= tol and err["allclose_ref"], err


def test_c2_fp32_4096_full_size_properties():
    _, M, N, K, dt, keys = gpu_cases.BIG_FP32
    A, B = oracle.make_inputs(M, N, K, torch.float32, "uniform", seed=0)
    c, kern, (a, b) = run_config(default_config(M, N, K, dt, **keys), A, B)
    assert _column_checksum_ok(c, a, b, 1e-6)
    g = torch.Generator().manual_seed(5)
    rows = torch.randperm(M, generator=g)[:256].sort().values
    _check_row_blocks(c, A, B, rows, oracle.TOL_FP32)
    # linearity in A: (2A) B == 2 (A B) exactly (power-of-two scaling commutes with every rounding)
    c2 = torch.empty_like(c)
    kern.run(a * 2, b, c2)
    kern.checkStatus()
    assert torch.equal(c2, c * 2)


def test_c3_bf16_8192_full_size_properties():
    _, M, N, K, dt, keys = gpu_cases.BIG_BF16
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=0)
    c, kern, (a, b) = run_config(default_config(M, N, K, dt, **keys), A, B)
    assert _column_checksum_ok(c, a, b, 5e-3)
    g = torch.Generator().manual_seed(6)
    rows = torch.randperm(M, generator=g)[:128].sort().values
    _check_row_blocks(c, A, B, rows, oracle.TOL_16BIT)
    # row-slab independence (what M-sharding relies on): a slab computed alone equals the slab of the full product
    kslab = default_config(M // 8, N, K, dt, **gpu_cases.BIG_BF16_SLAB)
    _, kern2 = build_kernel(kslab, 0)
    cs = torch.empty(M // 8, N, dtype=torch.bfloat16, device="cuda:0")
    kern2.run(a[3 * (M // 8):4 * (M // 8)], b, cs)
    kern2.checkStatus()
    # another kernel family and tile shape, same products summed in the same K order per element
    assert torch.equal(cs, c[3 * (M // 8):4 * (M // 8)])


@pytest.mark.parametrize("case", gpu_cases.RECT, ids=[c[0] for c in gpu_cases.RECT])
def test_rectangular_sweep_points(case):
    _, M, N, K, dt, keys = case
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, N, K, tdt, "uniform", seed=0)
    c, _, (a, b) = run_config(default_config(M, N, K, dt, **keys), A, B)
    g = torch.Generator().manual_seed(7)
    rows = torch.randperm(M, generator=g)[:min(M, 64)].sort().values
    _check_row_blocks(c, A, B, rows, oracle.tolerance_for(tdt))
    assert _column_checksum_ok(c, a, b, 1e-6 if dt == E.float32 else 5e-3)


def _random_row_blocks(M, blocks, seed, block=128):
    """Row indices of `blocks` distinct, randomly chosen `block`-row blocks of an M-row matrix (all of them if M is small)."""
    nb = M // block
    g = torch.Generator().manual_seed(seed)
    pick = torch.randperm(nb, generator=g)[:min(blocks, nb)].sort().values
    return torch.cat([torch.arange(int(b) * block, (int(b) + 1) * block) for b in pick])


@pytest.mark.parametrize("case", gpu_cases.TUNED_SHAPES, ids=[c[0] for c in gpu_cases.TUNED_SHAPES])
def test_tuned_config_of_every_benchmarked_shape_matches_oracle(case):
    """Every point of the rectangular sweep and every row-slab shape of the M-sharded headline product, run with
    the config `tuned_config` hands the operator and the benchmark for that shape (kernel database entry or rule
    of thumb) - the reference checks every config it times (Runtime/python/kcg/KCGTask.py:177-191). C starts as
    NaN; eight random 128-row blocks are compared with the host oracle, all of C through the column checksum."""
    from codegendemo_b200.kcg.matmul_op import tuned_config
    _, M, N, K, dt, dist = case
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, N, K, tdt, dist, seed=0)
    c, _, (a, b) = run_config(tuned_config(M, N, K, dt), A, B)
    assert not torch.isnan(c).any().item(), "kernel left part of C unwritten"
    rows = _random_row_blocks(M, 8, seed=M + N)
    _check_row_blocks(c, A, B, rows, oracle.tolerance_for(tdt))
    assert _column_checksum_ok(c, a, b, 1e-6 if dt == E.float32 else 5e-3)


def test_two_streams_run_split_k_launches_side_by_side():
    """Launches on different streams of one GPU own separate split-K workspaces, counters and status words: two
    K-split products queued side by side (no ordering between the streams) give the bits of their serial runs."""
    shapes = [(256, 512, 4096, dict(LOCAL_SPLIT_U=4)), (128, 1024, 8192, dict(LOCAL_SPLIT_U=8, BLOCK_SIZE_N=128))]
    kerns, ops, serial = [], [], []
    for i, (M, N, K, keys) in enumerate(shapes):
        A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=30 + i)
        c, kern, (a, b) = run_config(default_config(M, N, K, E.bfloat16, **keys), A, B)
        assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT
        kerns.append(kern), ops.append((a, b)), serial.append(c)
    streams = [torch.cuda.Stream(device=0) for _ in shapes]
    outs = [torch.full_like(c, float("nan")) for c in serial]
    torch.cuda.synchronize()
    for _ in range(20):  # interleaved: the launches of the two streams overlap on the GPU
        for st, kern, (a, b), out in zip(streams, kerns, ops, outs):
            with torch.cuda.stream(st):
                kern.run(a, b, out)
    for st, kern in zip(streams, kerns):
        with torch.cuda.stream(st):
            kern.checkStatus()  # synchronises this stream and reads ITS status block
    torch.cuda.synchronize()
    for out, c in zip(outs, serial):
        assert torch.equal(out, c)


# (M, N, K, keys): remainders of a persistent grid's waves, small enough for the host product.
#  - 80 / 160 tiles on 74 pairs / 148 CTAs: the few left-over tiles are cut eight ways and run first,
#    their partial tiles summed (a share per contributor, straight from L2) under the whole tiles' main loops;
#  - 22 tiles on 74 pairs: no whole tiles follow, the contributors sum their shares out of the idle operand ring.
REMAINDER_CASES = [
    (1280, 4096, 1024, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64)),
    (1280, 4096, 1024, dict(KERNEL_VARIANT=2, BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64)),
    (512, 2816, 2048, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)),
    (640, 2816, 1536, dict(KERNEL_VARIANT=2, BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=64)),
    # 128 pair tiles on 74 pairs: the even split cuts the 54 left-over tiles into quarters, three rounds of units
    (2048, 4096, 2048, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)),
]


@pytest.mark.parametrize("plan", ["3", "4", "5"], ids=["stream-k", "even-split", "stream-k-first"])
@pytest.mark.parametrize("case", REMAINDER_CASES, ids=lambda c: f"{c[0]}x{c[1]}x{c[2]}-V{c[3]['KERNEL_VARIANT']}")
def test_remainder_split_plans_match_oracle_and_repeat_bitwise(case, plan, monkeypatch):
    """The ways of splitting the tiles that do not fill a wave (KCG_TAIL_SPLIT: 3 = stream-K after the whole tiles,
    4 = even split before them, 5 = stream-K before them; each without its cost gate so that these small problems
    take it): the product matches the host oracle, every element of C is written, and a second launch gives the
    same bits (partials are summed in K order whoever sums them)."""
    M, N, K, keys = case
    monkeypatch.setenv("KCG_TAIL_SPLIT", plan)
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=M + int(plan))
    c, kern, (a, b) = run_config(default_config(M, N, K, E.bfloat16, **keys), A, B)
    assert not torch.isnan(c).any().item(), "kernel left part of C unwritten"
    assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT
    again = torch.full_like(c, float("nan"))
    for _ in range(3):
        kern.run(a, b, again)
    kern.checkStatus()
    assert torch.equal(again, c)
    monkeypatch.setenv("KCG_TAIL_SPLIT", "0")  # whole tiles only: same values up to the order of the fp32 sums
    whole = torch.full_like(c, float("nan"))
    kern.run(a, b, whole)
    kern.checkStatus()
    assert (whole.float() - c.float()).abs().max().item() <= 2e-2 * c.float().abs().max().item()


def test_two_full_grids_with_shared_reductions_side_by_side():
    """Two persistent launches that each want every SM, queued on two streams without ordering, both with a split
    remainder whose contributors wait for each other's partial tiles: whichever way the hardware deals the SMs - a
    contributor may not be running while its partners wait - the waits are bounded and abandoned shares are taken
    over, so both products complete and equal their serial runs bit for bit."""
    shapes = [(512, 11008, 2048, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=128)),
              (1280, 4096, 2048, dict(KERNEL_VARIANT=2, BLOCK_SIZE_M=128, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64))]
    os.environ["KCG_TAIL_SPLIT"] = "4"
    try:
        kerns, ops, serial = [], [], []
        for i, (M, N, K, keys) in enumerate(shapes):
            A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=50 + i)
            c, kern, (a, b) = run_config(default_config(M, N, K, E.bfloat16, **keys), A, B)
            assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT
            kerns.append(kern), ops.append((a, b)), serial.append(c)
        streams = [torch.cuda.Stream(device=0) for _ in shapes]
        outs = [torch.full_like(c, float("nan")) for c in serial]
        torch.cuda.synchronize()
        for _ in range(30):
            for st, kern, (a, b), out in zip(streams, kerns, ops, outs):
                with torch.cuda.stream(st):
                    kern.run(a, b, out)
        for st, kern in zip(streams, kerns):
            with torch.cuda.stream(st):
                kern.checkStatus()
        torch.cuda.synchronize()
        for out, c in zip(outs, serial):
            assert torch.equal(out, c)
    finally:
        os.environ.pop("KCG_TAIL_SPLIT", None)


@pytest.mark.parametrize("shape", [(512, 2816, 2048, 128), (1280, 4096, 1024, 64)],
                         ids=["shares-of-rows-through-the-ring", "shares-of-blocks-from-l2"])
def test_abandoned_shares_of_a_split_reduction_are_summed_by_the_last_arriver(shape, monkeypatch, tmp_path):
    """A contributor that gives up waiting for the other partial tiles hands its share of the sum to the last
    arriver. Built with a waiting time of zero (KCG_SHARE_WAIT_NS=0, private cubin cache) every contributor that
    is not last gives up at once, so the hand-over runs on every split tile; the sum order does not change, so
    the result must equal the normal build's bit for bit. Two plans: no whole tiles follow (22 tiles on 74 pairs:
    shares are rows, summed out of the idle operand ring) and whole tiles follow (80 tiles: shares are blocks,
    summed straight from L2 under the next unit's main loop)."""
    M, N, K, bk = shape
    keys = dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=bk)
    monkeypatch.setenv("KCG_TAIL_SPLIT", "4")
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=77)
    c, _, (a, b) = run_config(default_config(M, N, K, E.bfloat16, **keys), A, B)
    monkeypatch.setenv("KCG_NVCC_FLAGS", "-DKCG_SHARE_WAIT_NS=0")
    monkeypatch.setenv("KCG_CACHE_DIR", str(tmp_path))
    c2, kern2, _ = run_config(default_config(M, N, K, E.bfloat16, **keys), A, B)
    assert torch.equal(c2, c)
    for _ in range(5):  # the counters are left at zero every time
        out = torch.full_like(c, float("nan"))
        kern2.run(a, b, out)
        kern2.checkStatus()
        assert torch.equal(out, c)


@pytest.mark.parametrize("shape", [
    (256, 2048, dict(KERNEL_VARIANT=5, BLOCK_SIZE_N=128, BLOCK_SIZE_K=128, LOCAL_SPLIT_U=4)),
    (2048, 2048, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=64)),
    (1024, 1024, dict(KERNEL_VARIANT=2, BLOCK_SIZE_M=128, BLOCK_SIZE_N=128, BLOCK_SIZE_K=64, LOCAL_SPLIT_U=2)),
    (512, 1024, dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256, BLOCK_SIZE_N=256, BLOCK_SIZE_K=32, dtype=E.float32)),
], ids=["cluster-split-k", "cta-pairs", "single-cta-split-k", "fp32-3xtf32-pairs"])
def test_back_to_back_dependent_launches_see_each_others_results(shape):
    """Launches of the tcgen05 kernels carry the programmatic-dependent-launch attribute:
    the next kernel of a stream is brought onto the GPU while the one before it drains, and waits
    (griddepcontrol.wait) before it touches global memory. A chain X1 = A.B, X2 = X1.B, X3 = X2.B queued without any
    synchronisation, repeated over the same buffers (each round overwrites what the round before still reads last),
    must give the bits of the same chain run with a device synchronisation after every launch."""
    M, K, keys = shape
    keys = dict(keys)
    dt = keys.pop("dtype", E.bfloat16)
    tdt = ToTorchType(dt)
    A, B = oracle.make_inputs(M, K, K, tdt, "normal", seed=5)
    _, kern = build_kernel(default_config(M, K, K, dt, **keys), 0)
    a, b = A.cuda(), (B * (K ** 0.5) * 0.9).to(tdt).cuda()   # keeps the chain's magnitude level
    xs = [torch.zeros(M, K, dtype=tdt, device="cuda:0") for _ in range(3)]

    def chain(sync):
        src = a
        for x in xs:
            kern.run(src, b, x)
            if sync:
                torch.cuda.synchronize()
            src = x

    chain(True)
    kern.checkStatus()
    want = [x.clone() for x in xs]
    assert torch.isfinite(want[2].float()).all().item() and want[2].float().abs().max().item() > 0
    for x in xs:
        x.zero_()
    for _ in range(20):
        chain(False)
    kern.checkStatus()
    for x, w_ in zip(xs, want):
        assert torch.equal(x, w_)


def test_strided_operands_are_read_and_written_in_place():
    """kcg_launch_gemm_strided: A, B and C as column blocks of wider row-major arrays (leading dimension > row
    length); what lies outside the C block is left untouched."""
    from codegendemo_b200.kcg.matmul_op import matmul
    M, N, K = 256, 512, 384
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=12)
    wide_a = torch.zeros(M, K + 128, dtype=torch.bfloat16, device="cuda:0")
    wide_b = torch.zeros(K, N + 256, dtype=torch.bfloat16, device="cuda:0")
    wide_c = torch.full((M, N + 64), 7.0, dtype=torch.bfloat16, device="cuda:0")
    wide_a[:, 64:64 + K] = A.cuda()
    wide_b[:, 128:128 + N] = B.cuda()
    before = _lib.get_lib().kcg_launch_count()
    matmul(wide_a[:, 64:64 + K], wide_b[:, 128:128 + N], c=wide_c[:, 32:32 + N])
    torch.cuda.synchronize()
    assert _lib.get_lib().kcg_launch_count() == before + 1  # no hidden copy kernels of ours, one GEMM launch
    ref = oracle.host_matmul(A, B)
    assert oracle.rel_errors(wide_c[:, 32:32 + N], ref)["max_rel"] <= oracle.TOL_16BIT
    assert (wide_c[:, :32] == 7.0).all().item() and (wide_c[:, 32 + N:] == 7.0).all().item()
    # fp32 (3xTF32 kernel stores from registers with the pitch) and a K-split launch (reducer stores with the pitch)
    Af, Bf = oracle.make_inputs(128, 256, 2048, torch.float32, "uniform", seed=13)
    wc = torch.full((128, 256 + 32), -3.0, dtype=torch.float32, device="cuda:0")
    wa = torch.zeros(128, 2048 + 8, dtype=torch.float32, device="cuda:0")
    wa[:, 4:4 + 2048] = Af.cuda()
    matmul(wa[:, 4:4 + 2048], Bf.cuda(), c=wc[:, 16:16 + 256], BLOCK_SIZE_N=128, LOCAL_SPLIT_U=2)
    torch.cuda.synchronize()
    assert oracle.rel_errors(wc[:, 16:16 + 256], oracle.host_matmul(Af, Bf))["max_rel"] <= oracle.TOL_FP32
    assert (wc[:, :16] == -3.0).all().item() and (wc[:, 16 + 256:] == -3.0).all().item()
    # rows that are not 16-byte aligned are refused, not mis-read
    with pytest.raises(_lib.KCGError) as ei:
        matmul(wide_a[:, 1:1 + K], wide_b[:, 128:128 + N])
    assert ei.value.code == _lib.E_BAD_ARG


def test_float32_c_over_bf16_operands_keeps_the_accumulators():
    """DATATYPE_C = float32 with bf16 A and B: C holds the fp32 accumulators, so it agrees with the fp32-accumulate
    oracle to fp32 summation-order noise (1e-5 here), far inside the 16-bit bound. Whole-K store path, K-split
    reducer and the CTA-pair kernel."""
    M, N, K = 512, 512, 1024
    A, B = oracle.make_inputs(M, N, K, torch.bfloat16, "normal", seed=15)
    ref = oracle.host_matmul(A, B)
    for keys in (dict(), dict(LOCAL_SPLIT_U=2), dict(KERNEL_VARIANT=4, BLOCK_SIZE_M=256)):
        kpm = default_config(M, N, K, E.bfloat16, out_dtype=E.float32, **keys)
        _, kern = build_kernel(kpm, 0)
        c = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda:0")
        kern.run(A.cuda(), B.cuda(), c)
        kern.checkStatus()
        err = oracle.rel_errors(c, ref)
        assert not err["nan"] and err["max_rel"] <= 1e-5, (keys, err)


def test_nt_product_takes_b_as_stored():
    from codegendemo_b200.kcg.matmul_op import matmul
    M, N, K = 512, 768, 256
    A, B = oracle.make_inputs(M, N, K, torch.float16, "normal", seed=14)
    bt = B.t().contiguous().cuda()  # N x K, as a key matrix is stored
    c = matmul(A.cuda(), bt, b_transposed=True)
    torch.cuda.synchronize()
    assert oracle.rel_errors(c, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT


@pytest.mark.parametrize("shape", [(4, 256, 256, 64), (16, 2048, 2048, 128), (3, 128, 384, 128)],
                         ids=["4x256x256x64", "16x2048x2048x128", "3x128x384x128"])
def test_attention_chain_matches_host_composition(shape):
    """softmax(scale * q k^T) v as batched NT product -> row softmax -> batched product. The reference has no
    attention operator (it lists the chain among its next ones), so the checker is the composition of its
    ``torch.matmul`` check with ``torch.softmax`` on the host in fp32: parity of this extension is pinned to
    that composition, not to reference output. Tolerance: the 16-bit bound, 2e-2 on max_rel."""
    import math
    from codegendemo_b200.kcg.matmul_op import attention
    H, Sq, Sk, D = shape
    g = torch.Generator().manual_seed(21)
    q = torch.randn(H, Sq, D, generator=g).bfloat16()
    k = torch.randn(H, Sk, D, generator=g).bfloat16()
    v = torch.randn(H, Sk, D, generator=g).bfloat16()
    out = attention(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    heads = range(H) if H <= 4 else (0, H // 2, H - 1)
    for h in heads:
        s = torch.matmul(q[h].float(), k[h].float().t()) / math.sqrt(D)
        ref = torch.matmul(torch.softmax(s, dim=-1), v[h].float())
        err = oracle.rel_errors(out[h], ref)
        assert not err["nan"] and err["max_rel"] <= oracle.TOL_16BIT, (h, err)


@pytest.mark.parametrize("shape", [(4, 256, 256, 64, "bf16"), (16, 2048, 2048, 128, "bf16"), (3, 128, 384, 128, "fp16"),
                                   (2, 200, 328, 64, "fp16"), (5, 77, 1000, 128, "bf16"), (1, 128, 128, 128, "bf16"),
                                   (96, 640, 384, 64, "bf16"), (2, 257, 129, 128, "fp16")],
                         ids=["4x256x256x64", "16x2048x2048x128", "3x128x384x128-fp16", "ragged-2x200x328x64-fp16",
                              "ragged-5x77x1000x128", "one-step", "many-heads-96x640x384x64", "ragged-2x257x129x128-fp16"])
def test_fused_attention_kernel_matches_host_composition(shape):
    """The same chain as one kernel (scores and probabilities stay on the SM): checked against the same host
    composition, every head, with ragged row and key counts (tiles clipped at the end of a head, keys masked), a
    scale that is not the default, NaN-poisoned output, and the kernel's status word afterwards."""
    from codegendemo_b200.kcg.matmul_op import attention_fused, attention_status
    H, Sq, Sk, D, dt = shape
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    g = torch.Generator().manual_seed(23)
    q = torch.randn(H, Sq, D, generator=g).to(tdt)
    k = torch.randn(H, Sk, D, generator=g).to(tdt)
    v = torch.randn(H, Sk, D, generator=g).to(tdt)
    scale = 0.11
    out = torch.full((H, Sq, D), float("nan"), dtype=tdt, device="cuda:0")
    attention_fused(q.cuda(), k.cuda(), v.cuda(), scale=scale, out=out)
    attention_status(0)
    heads = range(H) if H <= 5 else (0, H // 2, H - 1)
    for h in heads:
        s = torch.matmul(q[h].float(), k[h].float().t()) * scale
        ref = torch.matmul(torch.softmax(s, dim=-1), v[h].float())
        err = oracle.rel_errors(out[h], ref)
        assert not err["nan"] and err["max_rel"] <= oracle.TOL_16BIT, (h, err)
    # twice the same launch gives the same bits
    again = torch.empty_like(out)
    attention_fused(q.cuda(), k.cuda(), v.cuda(), scale=scale, out=again)
    attention_status(0)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))


def test_fused_attention_argument_checks():
    lib = _lib.get_lib()
    x = torch.zeros(2, 128, 128, dtype=torch.bfloat16, device="cuda:0")
    p = ctypes.c_uint64(x.data_ptr())
    assert lib.kcg_attention_fwd(0, 0, p, p, p, p, 62, 2, 128, 128, 96, ctypes.c_float(1.0)) == _lib.E_BAD_CONFIG
    assert lib.kcg_attention_fwd(0, 0, p, p, p, p, 4, 2, 128, 128, 128, ctypes.c_float(1.0)) == _lib.E_BAD_ARG
    assert lib.kcg_attention_fwd(0, 0, 0, p, p, p, 62, 2, 128, 128, 128, ctypes.c_float(1.0)) == _lib.E_BAD_ARG


def test_row_softmax_entry():
    lib = _lib.get_lib()
    from codegendemo_b200.kcg.Utils import DeviceInfo
    g = torch.Generator().manual_seed(22)
    for tdt, code, tol in ((torch.float32, 4, 1e-5), (torch.bfloat16, 62, 8e-3), (torch.float16, 2, 2e-3)):
        x = (torch.randn(300, 1000 if tdt == torch.float32 else 1008, generator=g) * 3).to(tdt)
        wide = torch.zeros(300, x.shape[1] + 24, dtype=tdt, device="cuda:0")
        wide[:, :x.shape[1]] = x.cuda()
        rc = lib.kcg_softmax_rows(0, ctypes.c_uint64(DeviceInfo.get_cuda_stream(0)), ctypes.c_uint64(wide.data_ptr()),
                                  300, x.shape[1], wide.shape[1], ctypes.c_float(0.5), code)
        assert rc == 0, lib.kcg_last_error()
        torch.cuda.synchronize()
        ref = torch.softmax(0.5 * x.float(), dim=-1)
        assert (wide[:, :x.shape[1]].float().cpu() - ref).abs().max().item() <= tol
        assert (wide[:, x.shape[1]:] == 0).all().item()
    assert lib.kcg_softmax_rows(0, 0, 16, 4, 7, 0, ctypes.c_float(1.0), 62) == _lib.E_BAD_ARG  # 14-byte rows
    # fp32 scores in, bf16 probabilities out, each matrix with its own pitch
    x = (torch.randn(64, 512, generator=g) * 4)
    src = torch.zeros(64, 520, dtype=torch.float32, device="cuda:0")
    src[:, :512] = x.cuda()
    dst = torch.full((64, 528), -1.0, dtype=torch.bfloat16, device="cuda:0")
    rc = lib.kcg_softmax_rows_ex(0, ctypes.c_uint64(DeviceInfo.get_cuda_stream(0)), ctypes.c_uint64(src.data_ptr()), 4,
                                 520, ctypes.c_uint64(dst.data_ptr()), 62, 528, 64, 512, ctypes.c_float(1.0))
    assert rc == 0, lib.kcg_last_error()
    torch.cuda.synchronize()
    assert (dst[:, :512].float().cpu() - torch.softmax(x, dim=-1)).abs().max().item() <= 4e-3
    assert (dst[:, 512:] == -1.0).all().item() and torch.equal(src[:, :512].cpu(), x)


def test_device_naive_reference_agrees_with_tensor_core_kernel():
    """The on-device one-thread-per-element kernel (role of the reference's gemm_kernel) vs the tcgen05 kernel."""
    A, B = oracle.make_inputs(256, 256, 256, torch.float32, "uniform", seed=2)
    c_tc, _, _ = run_config(default_config(256, 256, 256, E.float32, BLOCK_SIZE_N=128), A, B)
    c_nv, _, _ = run_config(default_config(256, 256, 256, E.float32, KERNEL_VARIANT=100), A, B)
    assert oracle.rel_errors(c_tc, c_nv.double())["max_rel"] <= 1e-4


def test_single_pass_tf32_is_less_accurate_than_3x():
    """Shows the gate discriminates: one TF32 pass misses 1e-4 by a wide margin, three passes meet it."""
    A, B = oracle.make_inputs(512, 512, 1024, torch.float32, "uniform", seed=0)
    ref = oracle.host_matmul(A, B)
    c1, _, _ = run_config(default_config(512, 512, 1024, E.float32, KERNEL_VARIANT=3, BLOCK_SIZE_N=128), A, B)
    c3, _, _ = run_config(default_config(512, 512, 1024, E.float32, KERNEL_VARIANT=2, BLOCK_SIZE_N=128), A, B)
    e1, e3 = oracle.rel_errors(c1, ref), oracle.rel_errors(c3, ref)
    assert e3["max_rel"] <= 1e-4 < e1["max_rel"]
    assert e3["normwise"] * 50 < e1["normwise"]


def test_perf_tester_flow_on_gpu(work_dir):
    """The reference-style timing/correctness step (KCGTask.py:133-193) on a real kernel."""
    from codegendemo_b200.kcg.KCGTask import PerfTester
    PerfTester._a = PerfTester._b = None
    PerfTester.BestPerf = []
    for keys in (dict(BLOCK_SIZE_N=128), dict(BLOCK_SIZE_N=256)):
        kpm = default_config(1024, 1024, 1024, E.bfloat16, **keys)
        inc, kern = build_kernel(kpm, 0)
        r = PerfTester._test_perf(kpm, inc, kern, benchmarkCount=5, warmupCount=1, nTorchEpsInitTest=5)
        assert r.isCorrect and r.kcg_elapseTimeMs > 0 and r.tflops > 1 and r.maxRelErr < 2e-2
        PerfTester._getBestPerf([r], 2)
    assert len(PerfTester.BestPerf) == 2
    PerfTester._a = PerfTester._b = None
    PerfTester.BestPerf = []


def test_device_properties_and_load_errors():
    lib = _lib.get_lib()
    p = _lib.DeviceProps()
    _lib.check(lib.kcg_device_properties(0, ctypes.byref(p)))
    assert p.cc_major == 10 and p.multiprocessor_count >= 100 and p.max_shared_mem >= 227 * 1024
    mod, fn = ctypes.c_uint64(), ctypes.c_uint64()
    rc = lib.kcg_load_binary(b"nope", b"/nonexistent/file.cubin", 0, 0, ctypes.byref(mod), ctypes.byref(fn), None, None)
    assert rc == _lib.E_IO and b"KCG Error[CUDA]" in lib.kcg_last_error()


def test_expired_device_wait_reports_status_and_leaves_the_context_usable():
    """Failure detection on the device, without a fault: a probe kernel waits 20 ms on a barrier nothing
    signals, records its status word and returns; the host reads KCG_E_DEVICE_TIMEOUT and the next launch works."""
    A, B = oracle.make_inputs(256, 256, 256, torch.bfloat16, "normal", seed=4)
    probe = default_config(256, 256, 256, E.bfloat16, KERNEL_VARIANT=101, BLOCK_SIZE_N=64)
    _, kern = build_kernel(probe, 0)
    a, b = A.cuda(), B.cuda()
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda:0")
    kern.run(a, b, c)
    with pytest.raises(_lib.KCGError) as ei:
        kern.checkStatus()
    assert ei.value.code == _lib.E_DEVICE_TIMEOUT and "bounded wait" in str(ei.value)
    assert torch.count_nonzero(c).item() == 0      # the probe wrote nothing
    kern.checkStatus()                              # status was cleared by the failing check
    good, _, _ = run_config(default_config(256, 256, 256, E.bfloat16), A, B)   # context still fine
    assert oracle.rel_errors(good, oracle.host_matmul(A, B))["max_rel"] <= oracle.TOL_16BIT
