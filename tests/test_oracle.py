"""Pins the CPU oracle (oracle/mops_oracle.c) before anything is checked against it:
(1) against golden vectors made by the reference's NumPy implementations, (2) against the
unmodified reference CPU library where it has been built, in f64 and f32, on the
reference's fixture shapes and on the benchmark shapes."""
import os

import numpy as np
import pytest

import fixtures
from conftest import assert_parity
from mops_b200 import workloads

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def run_all(impl, name, d, dtype=np.float64, second_order=True):
    """Every level of one op on one input dict -> {key: array}."""
    c = lambda x: np.ascontiguousarray(x, dtype=dtype)
    op = name.split("_")[0]
    out = {}
    if op == "hpe":
        out["output"] = impl.hpe(c(d["A"]), c(d["C"]), d["indices_A"])
        out["grad_A"] = impl.hpe_vjp(c(d["grad_output"]), c(d["A"]), c(d["C"]), d["indices_A"])
        if second_order and "grad_grad_A" in d:
            out["grad_grad_output"], out["grad_A_2"] = impl.hpe_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_output"]), c(d["A"]), c(d["C"]), d["indices_A"])
    elif op == "sap":
        idx = (d["indices_A"], d["indices_B"], d["indices_output"])
        out["output"] = impl.sap(c(d["A"]), c(d["B"]), c(d["C"]), *idx, d["output_size"])
        out["grad_A"], out["grad_B"] = impl.sap_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), c(d["C"]), *idx)
        if second_order and "grad_grad_A" in d:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = impl.sap_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_grad_B"]), c(d["grad_output"]), c(d["A"]),
                c(d["B"]), c(d["C"]), *idx)
    elif op == "opsa":
        out["output"] = impl.opsa(c(d["A"]), c(d["B"]), d["indices_output"], d["output_size"])
        out["grad_A"], out["grad_B"] = impl.opsa_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), d["indices_output"])
        if second_order and "grad_grad_A" in d:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = impl.opsa_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_grad_B"]), c(d["grad_output"]), c(d["A"]),
                c(d["B"]), d["indices_output"])
    elif op == "opsaw":
        idx = (d["indices_W"], d["indices_output"])
        out["output"] = impl.opsaw(c(d["A"]), c(d["B"]), c(d["W"]), *idx)
        out["grad_A"], out["grad_B"], out["grad_W"] = impl.opsaw_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), c(d["W"]), *idx)
    elif op == "sasaw":
        idx = (d["indices_A"], d["indices_W_1"], d["indices_W_2"], d["indices_output_1"],
               d["indices_output_2"])
        out["output"] = impl.sasaw(c(d["A"]), c(d["B"]), c(d["C"]), c(d["W"]), *idx,
                                   d["output_size"])
        out["grad_A"], out["grad_B"], out["grad_W"] = impl.sasaw_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), c(d["C"]), c(d["W"]), *idx)
    return out


@pytest.mark.parametrize("name", sorted(fixtures.CASES))
def test_oracle_matches_golden(oracle, name):
    got = run_all(oracle, name, fixtures.CASES[name]())
    keys = [k for k in GOLD.files if k.startswith(name + "/")]
    assert keys and len(keys) == len(got)
    for k in keys:
        assert_parity(got[k.split("/")[1]], GOLD[k], k)


@pytest.mark.parametrize("name", sorted(fixtures.CASES))
def test_reference_library_matches_golden(reference, name):
    got = run_all(reference, name, fixtures.CASES[name]())
    for k, v in got.items():
        assert_parity(v, GOLD[f"{name}/{k}"], f"{name}/{k}")


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("name", sorted(fixtures.CASES))
def test_oracle_matches_reference_library_fixtures(oracle, reference, name, dtype):
    d = fixtures.CASES[name]()
    a, b = run_all(oracle, name, d, dtype), run_all(reference, name, d, dtype)
    for k in a:
        assert_parity(a[k], b[k], f"{name}/{k}/{np.dtype(dtype).name}")


SMALL = {
    "hpe": dict(), "sap": dict(), "opsa": dict(), "opsaw": dict(),
    # SASAW at E=60000 costs the scalar oracle about a second per level; 6000 edges keep
    # the CPU suite short while still giving ~60 edges per node.
    "sasaw": dict(E=6000, n=100),
}


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("op", sorted(SMALL))
def test_oracle_matches_reference_library_benchmark_shapes(oracle, reference, op, dtype):
    d = workloads.GENERATORS[op](dtype=dtype, **SMALL[op])
    a, b = run_all(oracle, op, d, dtype), run_all(reference, op, d, dtype)
    for k in a:
        assert_parity(a[k], b[k], f"{op}/{k}/{np.dtype(dtype).name}")


def test_hpe_orders_0_to_10(oracle, reference):
    r = np.random.default_rng(7)
    A, C = r.uniform(-1, 1, (37, 11)), r.standard_normal(23)
    gO = r.standard_normal(37)
    # K = 0: the reference's host index check reads past an empty index array
    # (mops/src/internal/checks/utils.hpp:58-61), so that order is pinned analytically.
    P0 = np.zeros((23, 0), np.int32)
    assert_parity(oracle.hpe(A, C, P0), np.full(37, C.sum()), "K=0", tol=1e-14)
    assert_parity(oracle.hpe_vjp(gO, A, C, P0), np.zeros_like(A), "vjp K=0")
    for K in range(1, 11):
        P = r.integers(0, 11, (23, K), dtype=np.int32)
        assert_parity(oracle.hpe(A, C, P), reference.hpe(A, C, P), f"K={K}")
        assert_parity(oracle.hpe_vjp(gO, A, C, P), reference.hpe_vjp(gO, A, C, P), f"vjp K={K}")
