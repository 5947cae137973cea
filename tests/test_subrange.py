"""The sub-range checker itself, on the CPU: the oracle's full result must pass its own
sub-range checks at sizes with several blocks, and a corrupted result must not."""
import numpy as np
import pytest

import subrange
from helpers import run_checker
from mops_b200 import workloads

SIZES = {"hpe": dict(I=3 * 4096 + 777, N=12, J=40, K=3), "sap": dict(I=3 * 4096 + 777, K=200),
         "opsa": dict(J=60000, nO=1000), "opsaw": dict(E=60000, n=1000, K=5, L=8),
         "sasaw": dict(E=20000, n=1000, N=60, L=8)}


@pytest.mark.parametrize("op", sorted(SIZES))
def test_oracle_passes_its_own_subrange_checks(oracle, op):
    d = workloads.GENERATORS[op](**SIZES[op])
    full = run_checker(oracle, op, d, np.float64)

    def library_vjp(sub):
        return run_checker(oracle, op, sub, np.float64)["grad_W"]

    report = subrange.check_case(oracle, op, d, full, library_vjp=library_vjp)
    blocks = 3 * (3 if op in ("sap", "opsa", "opsaw", "sasaw") else 2)
    assert len(report) >= blocks
    assert all(r["max_abs_err"] <= 1e-12 * max(r["scale"], 1.0) for r in report)


@pytest.mark.parametrize("op", ["sap", "opsa", "sasaw"])
def test_a_corrupted_result_is_caught(oracle, op):
    d = workloads.GENERATORS[op](**SIZES[op])
    full = run_checker(oracle, op, d, np.float64)
    bad = dict(full)
    bad["grad_A"] = full["grad_A"].copy()
    bad["grad_A"][-1, 0] += 1e-6  # inside the last block of every op
    with pytest.raises(subrange.Mismatch):
        subrange.check_case(oracle, op, d, bad)
    bad = dict(full)
    bad["output"] = full["output"].copy()
    bad["output"][3] *= 1.0 + 1e-9
    with pytest.raises(subrange.Mismatch):
        subrange.check_case(oracle, op, d, bad)


def test_row_blocks_cover_both_ends_and_a_ragged_tail():
    b = subrange.row_blocks(1 << 20, 4096)
    assert b[0] == (0, 4096) and b[-1][1] == 1 << 20 and (b[-1][1] - b[-1][0]) % 32 != 0
    assert subrange.row_blocks(100, 4096) == [(0, 100)]
