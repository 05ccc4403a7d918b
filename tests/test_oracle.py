"""The CPU oracle against the golden vectors (outputs of the reference's own hostMatmul) and against
itself: C restatement bit-exact, torch.matmul fp64 within rounding, error metrics behave."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import oracle

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def test_golden_files_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_c_port_reproduces_reference_host_matmul_bit_exact(path):
    g = np.load(path)
    A, B = g["A"], g["B"]
    At = np.ascontiguousarray(A.T)
    c32 = oracle.c_host_matmul(At, B, a_transposed=True)
    c64 = oracle.c_host_matmul(At.astype(np.float64), B.astype(np.float64), a_transposed=True)
    assert c32.dtype == np.float32 and np.array_equal(c32, g["C32"])
    assert np.array_equal(c64, g["C64"])
    # the NN layout (A as M x K) walks the same products in the same order
    assert np.array_equal(oracle.c_host_matmul(A, B, a_transposed=False), g["C32"])


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_torch_fp64_oracle_agrees_with_golden(path):
    g = np.load(path)
    A, B = torch.from_numpy(g["A"]), torch.from_numpy(g["B"])
    ref = oracle.host_matmul(A, B)
    assert ref.dtype == torch.float64
    assert np.allclose(ref.numpy(), g["C64"], rtol=1e-12, atol=1e-12)
    if A.shape[1] > 0:
        e = oracle.rel_errors(torch.from_numpy(g["C32"]), ref)
        assert e["max_rel"] < 1e-5 and e["allclose_ref"]


@pytest.mark.skipif(oracle.ref_lib() is None, reason="oracle/_ref not built (reference tree absent)")
def test_reference_host_matmul_matches_port_on_fresh_inputs():
    rng = np.random.default_rng(7)
    At = rng.uniform(-1, 1, size=(40, 24)).astype(np.float32)  # K x M
    B = rng.uniform(-1, 1, size=(40, 56)).astype(np.float32)
    assert np.array_equal(oracle.ref_host_matmul(At, B), oracle.c_host_matmul(At, B, a_transposed=True))


def test_accumulate_semantics_of_host_matmul():
    # hostMatmul adds into C (matmul.cpp:2356); the IR definition starts from 0 (Matmul.cc:41-66)
    A = np.ones((4, 3), np.float32)
    B = np.ones((3, 5), np.float32)
    base = np.full((4, 5), 2.0, np.float32)
    out = oracle.c_host_matmul(A, B, a_transposed=False, accumulate_into=base.copy())
    assert np.array_equal(out, base + 3.0)
    assert np.array_equal(oracle.c_host_matmul(A, B, a_transposed=False), np.full((4, 5), 3.0, np.float32))


def test_acc64_oracle():
    A, B = oracle.make_inputs(32, 48, 40, torch.float32, "uniform", seed=0)
    ref = oracle.host_matmul(A, B).numpy()
    got = oracle.c_host_matmul_acc64(A.numpy(), B.numpy(), a_transposed=False)
    assert np.allclose(got, ref, rtol=1e-13, atol=1e-13)


def test_seeded_inputs_are_reproducible_and_typed():
    A1, B1 = oracle.make_inputs(64, 32, 16, torch.float32, "uniform", seed=0)
    A2, B2 = oracle.make_inputs(64, 32, 16, torch.float32, "uniform", seed=0)
    assert torch.equal(A1, A2) and torch.equal(B1, B2)
    assert A1.min() >= -1 and A1.max() < 1
    A3, _ = oracle.make_inputs(64, 32, 16, torch.float32, "uniform", seed=1)
    assert not torch.equal(A1, A3)
    Ab, Bb = oracle.make_inputs(64, 32, 256, torch.bfloat16, "normal", seed=0)
    assert Ab.dtype == torch.bfloat16 and abs(Ab.float().std().item() - 1 / 16) < 0.01


def test_error_metrics():
    ref = torch.tensor([[1.0, -2.0], [0.0, 4.0]], dtype=torch.float64)
    e0 = oracle.rel_errors(ref.clone(), ref)
    assert e0["max_rel"] == 0 and e0["normwise"] == 0 and e0["allclose_ref"]
    c = ref.clone()
    c[1, 0] = 1e-3  # error on an element whose reference is zero: floored by rms, not unbounded
    e = oracle.rel_errors(c, ref)
    rms = ref.pow(2).mean().sqrt().item()
    assert abs(e["max_rel"] - 1e-3 / rms) < 1e-12
    assert e["max_rel_eps2"] > e["max_rel"]
    c[0, 0] = float("nan")
    assert oracle.rel_errors(c, ref)["max_rel"] == float("inf")
    n, mx = oracle.compare_with_error(ref, ref + 0.5)
    assert n == 4 and abs(mx - 0.5) < 1e-12


def test_tolerances_are_the_stated_ones():
    assert oracle.tolerance_for(torch.float32) == 1e-4
    assert oracle.tolerance_for(torch.bfloat16) == 2e-2
    assert oracle.tolerance_for(torch.float16) == 2e-2
