"""Parity of the sm_100a kernels, called through the C ABI, against the CPU oracle, the
committed golden vectors and (where built) the unmodified reference CPU library.

Tolerances (conftest.assert_parity): 1e-12 of the tensor's largest magnitude for f64,
1e-5 for f32."""
import os

import numpy as np
import pytest

import fixtures
from conftest import assert_parity
from helpers import run_checker, run_library, to_dev
from mops_b200 import workloads

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
DTYPES = [np.float64, np.float32]


def compare(op, d, dtype, checker, second_order=False, what="", tol=None):
    got = run_library(op, to_dev(d, dtype), second_order)
    want = run_checker(checker, op, d, dtype, second_order)
    assert set(got) == set(want)
    for k in want:
        assert_parity(got[k], want[k], f"{what or op}/{k}/{np.dtype(dtype).name}", tol=tol)


# ---------------------------------------------------------------- the reference's fixtures
@pytest.mark.parametrize("name", sorted(fixtures.CASES))
def test_golden_vectors(name):
    """f64 results equal the vectors produced by the reference's NumPy implementations.
    Scatter indices of these fixtures are unsorted: exercises the unsorted-index path."""
    d = fixtures.CASES[name]()
    op = name.split("_")[0]
    got = run_library(op, to_dev(d, np.float64), second_order=(op in ("hpe", "sap", "opsa")))
    keys = [k for k in GOLD.files if k.startswith(name + "/")]
    assert len(keys) == len(got)
    for k in keys:
        assert_parity(got[k.split("/")[1]], GOLD[k], k)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(fixtures.CASES))
def test_fixtures_against_oracle(oracle, name, dtype):
    op = name.split("_")[0]
    compare(op, fixtures.CASES[name](), dtype, oracle, second_order=(op in ("hpe", "sap", "opsa")),
            what=name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["opsa", "opsa_empty_row", "opsaw", "opsaw_empty_row", "sasaw"])
def test_fixtures_sorted_indices(oracle, name, dtype):
    """The same fixtures with the entries sorted by output row: the segmented fast path
    (this is how the reference's own CUDA tests call OPSA, python/mops/tests/opsa.py:96)."""
    d = fixtures.CASES[name]()
    key = "indices_output_1" if name == "sasaw" else "indices_output"
    order = np.argsort(d[key], kind="stable")
    per_entry = {"A", "B", key, "indices_W", "indices_W_1", "grad_grad_A", "grad_grad_B"}
    d = {k: (v[order] if k in per_entry and isinstance(v, np.ndarray) else v) for k, v in d.items()}
    op = name.split("_")[0]
    compare(op, d, dtype, oracle, second_order=(op == "opsa"), what=name + "/sorted")


# ---------------------------------------------------------------- benchmark shapes
SMALL = {"hpe": {}, "sap": {}, "opsa": {}, "opsaw": {}, "sasaw": dict(E=6000, n=100)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", sorted(SMALL))
def test_benchmark_shapes_against_oracle(oracle, op, dtype):
    compare(op, workloads.GENERATORS[op](dtype=dtype, **SMALL[op]), dtype, oracle)


@pytest.mark.parametrize("op", sorted(SMALL))
def test_benchmark_shapes_against_reference_library(reference, op):
    compare(op, workloads.GENERATORS[op](**SMALL[op]), np.float64, reference)


def test_sasaw_full_small_config(oracle):
    """SASAW at the full E=60000 / 1000-node shape (about two seconds of oracle time)."""
    compare("sasaw", workloads.sasaw(), np.float64, oracle)


def test_sasaw_full_small_config_against_reference_library(reference):
    """The same full shape against the unmodified reference CPU library."""
    compare("sasaw", workloads.sasaw(), np.float64, reference)


# ---------------------------------------------------------------- edge cases
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("K", list(range(0, 11)))
def test_hpe_every_order(oracle, K, dtype):
    r = np.random.default_rng(100 + K)
    d = dict(A=r.uniform(-1, 1, (77, 13)), C=r.standard_normal(41),
             indices_A=r.integers(0, 13, (41, K), dtype=np.int32), grad_output=r.standard_normal(77),
             grad_grad_A=r.standard_normal((77, 13)))
    compare("hpe", d, dtype, oracle, second_order=True, what=f"hpe K={K}")


def test_hpe_order_above_10_is_an_error():
    import torch
    import mops_b200 as M
    A = torch.zeros(4, 3, device="cuda", dtype=torch.float64)
    C = torch.zeros(2, device="cuda", dtype=torch.float64)
    P = torch.zeros(2, 11, device="cuda", dtype=torch.int32)
    with pytest.raises(M.MopsError, match="Only up to polynomial order 10 is supported"):
        M.homogeneous_polynomial_evaluation(A, C, P)


@pytest.mark.parametrize("I", [1, 31, 32, 33, 257])
def test_ragged_batch_sizes(oracle, I):
    compare("hpe", workloads.hpe(I=I, N=17, J=50, K=3), np.float64, oracle, what=f"hpe I={I}")
    compare("sap", workloads.sap(I=I, K=120), np.float64, oracle, second_order=False,
            what=f"sap I={I}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_hpe_large_batch(oracle, dtype):
    """Batches large enough for the two- and four-rows-per-lane HPE kernels (chosen when the
    batch still fills the GPU that way), with ragged last blocks."""
    compare("hpe", workloads.hpe(I=148 * 64 * 8 + 37, N=17, J=60, K=3), dtype, oracle,
            what="hpe large batch")
    compare("hpe", workloads.hpe(I=148 * 128 * 8 + 69, N=11, J=40, K=4), dtype, oracle,
            what="hpe larger batch")
    compare("hpe", workloads.hpe(I=148 * 64 * 8 + 1, N=9, J=25, K=1), dtype, oracle,
            what="hpe large batch, K=1")


@pytest.mark.parametrize("dtype", DTYPES)
def test_wide_operands_take_the_global_memory_kernels(oracle, dtype):
    """Operand widths whose tiles do not fit in shared memory."""
    compare("hpe", workloads.hpe(I=70, N=1500, J=64, K=3), dtype, oracle, what="hpe wide")
    compare("sap", workloads.sap(I=70, nA=900, nB=700, nO=800, K=500), dtype, oracle,
            what="sap wide")
    compare("opsa", workloads.opsa(J=300, K=40, L=900, nO=7), dtype, oracle, what="opsa wide")
    compare("opsaw", workloads.opsaw(E=300, K=40, L=900, n=7), dtype, oracle, what="opsaw wide")
    compare("sasaw", workloads.sasaw(E=200, nA=5, L=700, n=6, N=40, nW2=30, nO2=40), dtype,
            oracle, what="sasaw wide")


@pytest.mark.parametrize("K,L", [(1, 1), (3, 7), (13, 20), (17, 33), (40, 5), (2, 64), (25, 25)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_outer_product_shapes(oracle, K, L, dtype):
    compare("opsa", workloads.opsa(J=700, K=K, L=L, nO=23), dtype, oracle, what=f"opsa {K}x{L}")
    compare("opsaw", workloads.opsaw(E=700, K=K, L=L, n=23), dtype, oracle, what=f"opsaw {K}x{L}")


@pytest.mark.parametrize("K", [9, 13, 16])
@pytest.mark.parametrize("dtype", DTYPES)
def test_weighted_outer_product_fixed_shapes(oracle, K, dtype):
    """The weighted kernels with K and L fixed at compile time (L = 32, K = 9, 13, 16): ragged
    rows, empty rows, one row that spans many chunks, an entry count that is no multiple of
    the chunk."""
    d = workloads.opsaw(E=4999, K=K, L=32, n=211)
    po = d["indices_output"]
    po[po == 5] = 6          # row 5 is empty
    po[1000:1900] = po[1000]  # a long row
    po.sort()
    compare("opsaw", d, dtype, oracle, what=f"opsaw fixed {K}x32")
    compare("opsaw", workloads.opsaw(E=7, K=K, L=32, n=3), dtype, oracle, what=f"opsaw tiny {K}x32")
    # long rows on average (the VJP then keeps one grad_output slot per warp), among them
    # empty rows and rows of a single entry
    d = workloads.opsaw(E=6001, K=K, L=32, n=60)
    po = d["indices_output"]
    po[(po % 7 == 3) & (po < 59)] += 1
    po[:3] = 0
    po.sort()
    compare("opsaw", d, dtype, oracle, what=f"opsaw fixed {K}x32, long rows")


@pytest.mark.parametrize("seed", list(range(16)))
def test_outer_product_random_shapes_and_row_lengths(oracle, seed):
    """Random widths within the streaming kernels' range (K <= 16, L <= 32), entry counts that
    are no multiple of a chunk, and row lengths from empty to several chunks: the whole /
    ragged step logic at every alignment, both dtypes, with and without weights."""
    r = np.random.default_rng(9000 + seed)
    K, L = int(r.integers(1, 17)), int(r.integers(1, 33))
    if seed % 2:
        L = int(r.choice([2, 4, 8, 12, 16, 20, 24, 28, 32]))  # weighted streaming needs 16-byte rows
    nO = int(r.integers(1, 120))
    J = int(r.integers(1, 2500))
    # row lengths: a few long rows, many short ones, some empty
    weights = r.random(nO) ** 4
    weights[r.random(nO) < 0.3] = 0.0
    if weights.sum() == 0:
        weights[0] = 1.0
    rows = np.sort(r.choice(nO, size=J, p=weights / weights.sum())).astype(np.int32)
    for dtype in DTYPES:
        d = workloads.opsa(J=J, K=K, L=L, nO=nO, seed=seed)
        d["indices_output"] = rows
        compare("opsa", d, dtype, oracle, what=f"opsa random {K}x{L} J={J} nO={nO}")
        d = workloads.opsaw(E=J, K=K, L=L, n=nO, seed=seed)
        d["indices_output"] = rows
        compare("opsaw", d, dtype, oracle, what=f"opsaw random {K}x{L} E={J} n={nO}")


@pytest.mark.parametrize("seed", list(range(10)))
def test_sasaw_random_shapes_and_row_lengths(oracle, seed):
    """SASAW with the compiled-in channel counts (4, 9, 16) and with arbitrary ones, several
    widths of B, and rows from empty to many quads of edges: the walk over quads across row
    boundaries at every alignment."""
    r = np.random.default_rng(7000 + seed)
    if seed % 2 == 0:
        nA = nW2 = nO2 = int(r.choice([4, 9, 16]))
    else:
        nA, nW2, nO2 = (int(x) for x in r.integers(1, 17, 3))
    L = int(r.choice([32, 32, 8, 20, 40, 64]))
    n = int(r.integers(1, 60))
    E = int(r.integers(1, 1500))
    N = int(r.integers(1, 400))
    weights = r.random(n) ** 4
    weights[r.random(n) < 0.3] = 0.0
    if weights.sum() == 0:
        weights[0] = 1.0
    d = workloads.sasaw(E=E, nA=nA, L=L, n=n, N=N, nW2=nW2, nO2=nO2, seed=seed)
    d["indices_output_1"] = np.sort(r.choice(n, size=E, p=weights / weights.sum())).astype(np.int32)
    # one row may hold most of the edges here: an f32 sum of that many terms (thousands, in
    # two different orders) is good to a few 1e-5 of the largest element, not to 1e-5
    for dtype, tol in ((np.float64, None), (np.float32, 5e-5)):
        compare("sasaw", d, dtype, oracle, tol=tol,
                what=f"sasaw random {nA},{nW2},{nO2} L={L} E={E} n={n} N={N}")


@pytest.mark.parametrize("op", ["opsa", "opsaw", "sasaw"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_operands_that_are_views_at_odd_addresses(oracle, op, dtype):
    """Per-entry operands that are views starting one scalar into a larger allocation (what a
    slice of a bigger array looks like): not 16-byte aligned, so the streaming kernels do not
    apply and the general kernels must give the same results."""
    import torch
    d = {"opsa": workloads.opsa(J=3001, K=13, L=20, nO=57),
         "opsaw": workloads.opsaw(E=3001, K=13, L=32, n=57),
         "sasaw": workloads.sasaw(E=1501, n=57)}[op]
    t = to_dev(d, dtype)
    for name in ("A", "B", "grad_output"):
        flat = torch.empty(t[name].numel() + 1, dtype=t[name].dtype, device="cuda")
        flat[1:] = t[name].reshape(-1)
        t[name] = flat[1:].view(t[name].shape)
        assert t[name].data_ptr() % 16 != 0 and t[name].is_contiguous()
    got = run_library(op, t)
    want = run_checker(oracle, op, d, dtype)
    for k in want:
        assert_parity(got[k], want[k], f"{op} unaligned views {k}")


@pytest.mark.parametrize("kw", [
    dict(I=100, nA=3, nB=20, nO=7, K=300),      # A is the register-resident operand
    dict(I=257, nA=20, nB=16, nO=50, K=1000),   # widest register-resident row
    dict(I=33, nA=9, nB=9, nO=9, K=400),
    dict(I=64, nA=1, nB=1, nO=1, K=5),
    dict(I=90, nA=17, nB=40, nO=30, K=700),     # neither operand is narrow: general kernels
    dict(I=70, nA=5, nB=8, nO=300, K=40),       # most output columns receive nothing
], ids=lambda kw: "-".join(f"{k}{v}" for k, v in kw.items()))
@pytest.mark.parametrize("dtype", DTYPES)
def test_sap_operand_widths(oracle, kw, dtype):
    """SAP with either operand narrow enough to sit in registers, and with neither; the output
    index in random order (the plan kernels sort the triplets themselves)."""
    d = workloads.sap(**kw)
    r = np.random.default_rng(11)
    d["indices_output"] = r.permutation(d["indices_output"])
    d["grad_grad_A"] = r.standard_normal(d["A"].shape)
    d["grad_grad_B"] = r.standard_normal(d["B"].shape)
    compare("sap", d, dtype, oracle, second_order=True, what=f"sap {kw}")
    t = to_dev(d, dtype)
    import mops_b200 as M
    want = run_checker(oracle, "sap", d, dtype)
    for need_a, need_b in ((True, False), (False, True)):
        gA, gB = M.sparse_accumulation_of_products_vjp(
            t["grad_output"], t["A"], t["B"], t["C"], t["indices_A"], t["indices_B"],
            t["indices_output"], compute_grad_A=need_a, compute_grad_B=need_b)
        assert (gA is not None) == need_a and (gB is not None) == need_b
        if need_a:
            assert_parity(gA.cpu().numpy(), want["grad_A"], f"grad_A only {kw}")
        if need_b:
            assert_parity(gB.cpu().numpy(), want["grad_B"], f"grad_B only {kw}")


def test_single_giant_segment_and_many_empty_rows(oracle):
    d = workloads.opsa(J=5000, K=5, L=6, nO=40)
    d["indices_output"][:] = 17
    compare("opsa", d, np.float64, oracle, what="opsa one segment")
    d = workloads.opsa(J=50, K=5, L=6, nO=4000)
    compare("opsa", d, np.float64, oracle, what="opsa mostly empty")
    d = workloads.sasaw(E=40, n=300, N=60)
    compare("sasaw", d, np.float64, oracle, what="sasaw mostly empty")


def test_sasaw_shapes(oracle):
    for kw in (dict(E=500, nA=1, L=1, n=9, N=1, nW2=1, nO2=1),
               dict(E=500, nA=4, L=33, n=9, N=37, nW2=3, nO2=5),
               dict(E=500, nA=16, L=64, n=9, N=300, nW2=7, nO2=3)):
        d = workloads.sasaw(**kw)
        d["indices_output_2"] = np.random.default_rng(3).permutation(d["indices_output_2"])
        compare("sasaw", d, np.float64, oracle, what=f"sasaw {kw}")


@pytest.mark.parametrize("kw", [
    dict(E=1, nA=9, L=32, n=3, N=100, nW2=9, nO2=9),
    dict(E=7, nA=9, L=32, n=3, N=100, nW2=9, nO2=9),
    dict(E=501, nA=16, L=32, n=11, N=900, nW2=16, nO2=16),
    dict(E=1003, nA=5, L=40, n=17, N=70, nW2=7, nO2=12),
    dict(E=333, nA=3, L=96, n=5, N=50, nW2=5, nO2=8),
    dict(E=260, nA=12, L=17, n=40, N=200, nW2=12, nO2=4),
    dict(E=90, nA=8, L=31, n=4, N=64, nW2=8, nO2=1),
], ids=lambda kw: "-".join(f"{k}{v}" for k, v in kw.items()))
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shuffled", [False, True])
def test_sasaw_small_channel_kernels(oracle, kw, dtype, shuffled):
    """Shapes served by the tensor-core (f64) and register-tile (f32) SASAW kernels: ragged
    edge counts (batches of eight edges), several 32-wide chunks of B, every padded width, and
    edges both sorted by output row and in random order."""
    d = workloads.sasaw(**kw)
    if shuffled:
        order = np.random.default_rng(7).permutation(kw["E"])
        for k in ("A", "B", "indices_W_1", "indices_output_1"):
            d[k] = d[k][order]
    compare("sasaw", d, dtype, oracle, what=f"sasaw {kw} shuffled={shuffled}")


def test_sasaw_skipped_gradients(oracle):
    import mops_b200 as M
    d = workloads.sasaw(E=700, n=20)
    t = to_dev(d, np.float64)
    want = run_checker(oracle, "sasaw", d, np.float64)
    for need in [(True, False, False), (False, True, False), (False, False, True),
                 (True, True, False), (False, True, True)]:
        got = M.sparse_accumulation_scatter_add_with_weights_vjp(
            t["grad_output"], t["A"], t["B"], t["C"], t["W"], t["indices_A"], t["indices_W_1"],
            t["indices_W_2"], t["indices_output_1"], t["indices_output_2"], *need)
        for g, name, n in zip(got, ("grad_A", "grad_B", "grad_W"), need):
            assert (g is not None) == n
            if n:
                assert_parity(g.cpu().numpy(), want[name], f"{name} with {need}")


def test_empty_inputs():
    import torch
    import mops_b200 as M
    f = dict(device="cuda", dtype=torch.float64)
    i = dict(device="cuda", dtype=torch.int32)
    out = M.outer_product_scatter_add(torch.zeros(0, 3, **f), torch.zeros(0, 4, **f),
                                      torch.zeros(0, **i), 5)
    assert out.shape == (5, 3, 4) and float(out.abs().sum()) == 0.0
    out = M.sparse_accumulation_of_products(torch.zeros(6, 3, **f), torch.zeros(6, 2, **f),
                                            torch.zeros(0, **f), torch.zeros(0, **i),
                                            torch.zeros(0, **i), torch.zeros(0, **i), 4)
    assert out.shape == (6, 4) and float(out.abs().sum()) == 0.0
    out = M.homogeneous_polynomial_evaluation(torch.zeros(0, 3, **f), torch.zeros(2, **f),
                                              torch.zeros(2, 2, **i))
    assert out.shape == (0,)
    out = M.homogeneous_polynomial_evaluation(torch.ones(5, 3, **f), torch.zeros(0, **f),
                                              torch.zeros(0, 2, **i))
    assert out.shape == (5,) and float(out.abs().sum()) == 0.0


def test_skipped_gradients(oracle):
    import mops_b200 as M
    d = workloads.opsaw(E=400, n=11)
    t = to_dev(d, np.float64)
    want = run_checker(oracle, "opsaw", d, np.float64)
    for need in [(True, False, False), (False, True, False), (False, False, True)]:
        gA, gB, gW = M.outer_product_scatter_add_with_weights_vjp(
            t["grad_output"], t["A"], t["B"], t["W"], t["indices_W"], t["indices_output"], *need)
        for g, name, n in zip((gA, gB, gW), ("grad_A", "grad_B", "grad_W"), need):
            assert (g is not None) == n
            if n:
                assert_parity(g.cpu().numpy(), want[name], name)
    d = workloads.sap(I=100)
    t = to_dev(d, np.float64)
    want = run_checker(oracle, "sap", d, np.float64)
    gA, gB = M.sparse_accumulation_of_products_vjp(
        t["grad_output"], t["A"], t["B"], t["C"], t["indices_A"], t["indices_B"],
        t["indices_output"], compute_grad_A=False)
    assert gA is None
    assert_parity(gB.cpu().numpy(), want["grad_B"], "grad_B only")


def test_out_of_range_indices_are_reported():
    """The reference trusts device index arrays; here they are checked on the device."""
    import mops_b200 as M
    d = workloads.opsa(J=500, nO=10)
    d["indices_output"][-1] = 10
    t = to_dev(d, np.float64)
    with pytest.raises(M.MopsError, match="Index array indices_output in operation "
                                          "cuda_outer_product_scatter_add contains"):
        M.outer_product_scatter_add(t["A"], t["B"], t["indices_output"], 10)
    d = workloads.hpe(I=64, N=10, J=20)
    d["indices_A"][7, 2] = -1
    t = to_dev(d, np.float64)
    with pytest.raises(M.MopsError, match="Index array indices_A"):
        M.homogeneous_polynomial_evaluation(t["A"], t["C"], t["indices_A"])
    d = workloads.sap(I=64)
    d["indices_B"][3] = 6
    t = to_dev(d, np.float64)
    with pytest.raises(M.MopsError, match="Index array indices_B"):
        M.sparse_accumulation_of_products(t["A"], t["B"], t["C"], t["indices_A"], t["indices_B"],
                                          t["indices_output"], 50)
    # the library keeps working afterwards
    d = workloads.sap(I=64)
    t = to_dev(d, np.float64)
    M.sparse_accumulation_of_products(t["A"], t["B"], t["C"], t["indices_A"], t["indices_B"],
                                      t["indices_output"], 50)


def test_runs_are_bitwise_reproducible():
    """Kernels that use no atomics give identical bits on every run."""
    for op in ("hpe", "sap", "opsa"):
        d = to_dev(workloads.GENERATORS[op](), np.float64)
        a, b = run_library(op, d), run_library(op, d)
        for k in a:
            assert np.array_equal(a[k], b[k]), f"{op}/{k}"
    d = to_dev(workloads.opsaw(), np.float64)
    a, b = run_library("opsaw", d), run_library("opsaw", d)
    for k in ("output", "grad_A", "grad_B"):
        assert np.array_equal(a[k], b[k]), f"opsaw/{k}"


def test_host_arrays_round_trip(oracle):
    """NumPy in, NumPy out: staged through the GPU (there is no CPU implementation)."""
    import mops_b200 as M
    d = workloads.opsa(J=3000, nO=50)
    out = M.outer_product_scatter_add(d["A"], d["B"], d["indices_output"], 50)
    assert isinstance(out, np.ndarray)
    assert_parity(out, oracle.opsa(d["A"], d["B"], d["indices_output"], 50), "numpy opsa")


def test_host_queue_overlaps_calls_and_matches_the_oracle(oracle):
    """Host arrays through ``HostQueue``: forward and VJP of three operations queued back to
    back (shared operands copied once), results valid after the block; NumPy and pinned
    torch inputs."""
    import torch
    import mops_b200 as M
    d1, d2, d3 = workloads.opsa(J=5000, nO=80), workloads.sap(I=300), workloads.sasaw(E=900, n=30)
    pin = lambda d: {k: (torch.from_numpy(v).pin_memory() if isinstance(v, np.ndarray) else v)
                     for k, v in d.items()}
    p2 = pin(d2)
    with M.HostQueue() as q:
        O1 = M.outer_product_scatter_add(d1["A"], d1["B"], d1["indices_output"], 80)
        gA1, gB1 = M.outer_product_scatter_add_vjp(d1["grad_output"], d1["A"], d1["B"],
                                                   d1["indices_output"])
        idx = (p2["indices_A"], p2["indices_B"], p2["indices_output"])
        O2 = M.sparse_accumulation_of_products(p2["A"], p2["B"], p2["C"], *idx, 50)
        gA2, gB2 = M.sparse_accumulation_of_products_vjp(p2["grad_output"], p2["A"], p2["B"],
                                                         p2["C"], *idx)
        i3 = (d3["indices_A"], d3["indices_W_1"], d3["indices_W_2"], d3["indices_output_1"],
              d3["indices_output_2"])
        O3 = M.sparse_accumulation_scatter_add_with_weights(d3["A"], d3["B"], d3["C"], d3["W"],
                                                            *i3, 9)
        g3 = M.sparse_accumulation_scatter_add_with_weights_vjp(d3["grad_output"], d3["A"],
                                                                d3["B"], d3["C"], d3["W"], *i3)
        assert len(q._operands) == 4 + 7 + 10  # every distinct host array is copied once
    assert isinstance(O1, np.ndarray) and isinstance(O2, torch.Tensor) and O2.is_pinned()
    w1 = run_checker(oracle, "opsa", d1, np.float64)
    w2 = run_checker(oracle, "sap", d2, np.float64)
    w3 = run_checker(oracle, "sasaw", d3, np.float64)
    for got, want, what in ((O1, w1["output"], "O1"), (gA1, w1["grad_A"], "gA1"),
                            (gB1, w1["grad_B"], "gB1"), (O2.numpy(), w2["output"], "O2"),
                            (gA2.numpy(), w2["grad_A"], "gA2"), (gB2.numpy(), w2["grad_B"], "gB2"),
                            (O3, w3["output"], "O3"), (g3[0], w3["grad_A"], "gA3"),
                            (g3[1], w3["grad_B"], "gB3"), (g3[2], w3["grad_W"], "gW3")):
        assert_parity(got, want, "host queue " + what)
    # outside a queue the same call is synchronous again
    out = M.outer_product_scatter_add(d1["A"], d1["B"], d1["indices_output"], 80)
    assert_parity(out, w1["output"], "after the queue")


def test_host_queues_in_a_row_reuse_device_memory():
    """Queues that follow each other run on the same streams, so torch's caching allocator
    hands the arrays of one queue to the next: the memory it has reserved does not grow."""
    import torch
    import mops_b200 as M
    d = workloads.sap(I=200_000)
    pin = {k: (torch.from_numpy(v).pin_memory() if isinstance(v, np.ndarray) else v)
           for k, v in d.items()}
    idx = (pin["indices_A"], pin["indices_B"], pin["indices_output"])
    reserved = []
    for _ in range(8):
        with M.HostQueue():
            M.sparse_accumulation_of_products(pin["A"], pin["B"], pin["C"], *idx, 50)
            M.sparse_accumulation_of_products_vjp(pin["grad_output"], pin["A"], pin["B"],
                                                  pin["C"], *idx)
        reserved.append(torch.cuda.memory_reserved())
    assert reserved[-1] == reserved[1], reserved


# ---------------------------------------------------------------- the timed configurations
@pytest.mark.parametrize("name", ["hpe", "sap", "opsa", "opsa_f32", "opsaw", "sasaw"])
def test_timed_configurations_against_oracle_subranges(oracle, name):
    """The six configurations bench.py times, at their full per-GPU size (I = 2^20 / 2^22
    rows, J = 2^24 entries, E = 2^22 edges over 2^16 nodes): blocks of rows / output segments
    against the oracle, grad_W on a 2^16-edge slice of the same problem, and the adjoint
    identity over the whole result (tests/subrange.py). 1e-12 (f64) / 1e-5 (f32) of the
    largest magnitude of each compared block."""
    import bench
    import subrange
    op, dtype = bench.CASES[name][0], bench.CASES[name][1]
    d = bench.generate(name, 0)
    t = to_dev(d, dtype)
    results = run_library(op, t, to_host=False)

    def library_vjp(sub):
        return run_library(op, to_dev(sub, dtype), to_host=False)["grad_W"]

    report = subrange.check_case(oracle, op, d, results, inputs=t, library_vjp=library_vjp)
    assert len(report) >= 6, report


# ---------------------------------------------------------------- full-size properties
def test_full_size_properties():
    """At the scaled sizes the oracle is too slow; check size-independent properties:
    linearity in A, agreement of the forward with a sum of two halves of the entries, and
    <gO, O(A,B)> == <gA, A> (the VJP is the adjoint of a map that is linear in A)."""
    import torch
    import mops_b200 as M
    torch.manual_seed(5)
    J, K, L, nO = 1 << 21, 13, 20, 1 << 15
    f = dict(device="cuda", dtype=torch.float64)
    A, B = torch.randn(J, K, **f), torch.randn(J, L, **f)
    P = torch.sort(torch.randint(0, nO, (J,), device="cuda", dtype=torch.int32)).values
    O = M.outer_product_scatter_add(A, B, P, nO)
    O2 = M.outer_product_scatter_add(2.5 * A, B, P, nO)
    assert torch.allclose(O2, 2.5 * O, rtol=1e-13, atol=1e-12)
    h = J // 2
    while P[h] == P[h - 1]:
        h += 1
    Oa = M.outer_product_scatter_add(A[:h], B[:h], P[:h], nO)
    Ob = M.outer_product_scatter_add(A[h:].contiguous(), B[h:].contiguous(), P[h:].contiguous(), nO)
    # (not bitwise: the streaming kernel groups a row's entries by where its chunks fall)
    assert torch.allclose(Oa + Ob, O, rtol=1e-13, atol=1e-12)
    gO = torch.randn(nO, K, L, **f)
    gA, gB = M.outer_product_scatter_add_vjp(gO, A, B, P)
    lhs, rhs = float((gO * O).sum()), float((gA * A).sum())
    assert abs(lhs - rhs) <= 1e-10 * max(abs(lhs), 1.0)
    rhs_b = float((gB * B).sum())
    assert abs(lhs - rhs_b) <= 1e-10 * max(abs(lhs), 1.0)

    I = 1 << 18
    d = workloads.sap(I=8)
    C = torch.from_numpy(d["C"]).cuda()
    idx = [torch.from_numpy(d[k]).cuda() for k in ("indices_A", "indices_B", "indices_output")]
    A, B = torch.rand(I, 20, **f), torch.rand(I, 6, **f)
    O = M.sparse_accumulation_of_products(A, B, C, *idx, 50)
    gO = torch.randn(I, 50, **f)
    gA, gB = M.sparse_accumulation_of_products_vjp(gO, A, B, C, *idx)
    lhs = float((gO * O).sum())
    assert abs(lhs - float((gA * A).sum())) <= 1e-10 * max(abs(lhs), 1.0)
    assert abs(lhs - float((gB * B).sum())) <= 1e-10 * max(abs(lhs), 1.0)
    # rows are independent: any block of rows equals the same rows computed alone
    sub = M.sparse_accumulation_of_products(A[1000:1100].contiguous(), B[1000:1100].contiguous(),
                                            C, *idx, 50)
    assert torch.equal(sub, O[1000:1100])


# ---------------------------------------------------------------- plans
def test_plan_reuses_tables_and_results_do_not_change(oracle):
    """With a plan bound, the first call of every kind builds its table and later calls reuse
    it (forward and VJP of a scatter op share the segment table); results equal the oracle's
    and, bit for bit, those of the same calls without a plan."""
    import mops_b200 as M
    for op in ("hpe", "sap", "opsa", "opsaw", "sasaw"):
        d = workloads.GENERATORS[op]()
        t = to_dev(d, np.float64)
        plain = run_library(op, t)
        want = run_checker(oracle, op, d, np.float64)
        plan = M.Plan()
        with plan:
            first = run_library(op, t)
            held = plan.tables
            assert held >= 1, op
            again = run_library(op, t)
            assert plan.tables == held, f"{op}: a repeated call built another table"
        for k in want:
            assert_parity(first[k], want[k], f"plan/{op}/{k}")
            if not (op in ("opsaw", "sasaw") and k == "grad_W"):  # RED order is free
                assert np.array_equal(first[k], plain[k]), f"plan/{op}/{k} differs from no plan"
                assert np.array_equal(again[k], plain[k]), f"plan/{op}/{k} differs on reuse"
        if op in ("opsa", "opsaw"):
            assert held == 1, f"{op}: forward and VJP must share one segment table, got {held}"
        plan.close()
    # outside the block nothing is bound
    assert M._lib.library().mops_b200_plan_bound() is None


def test_plan_does_not_keep_tables_of_bad_or_unsorted_indices(oracle):
    import mops_b200 as M
    d = workloads.opsa(J=3000, nO=40)
    d["indices_output"] = np.random.default_rng(2).permutation(d["indices_output"])
    t = to_dev(d, np.float64)
    want = run_checker(oracle, "opsa", d, np.float64)
    with M.Plan() as plan:
        for _ in range(2):
            got = run_library("opsa", t)
            for k in want:
                assert_parity(got[k], want[k], f"unsorted with plan/{k}")
        assert plan.tables == 0
    d = workloads.hpe(I=64, N=10, J=20)
    d["indices_A"][7, 2] = 12
    t = to_dev(d, np.float64)
    with M.Plan() as plan:
        for _ in range(2):
            with pytest.raises(M.MopsError, match="Index array indices_A"):
                M.homogeneous_polynomial_evaluation(t["A"], t["C"], t["indices_A"])
        assert plan.tables == 0


def test_plan_second_order_calls_are_not_cached_from_temporaries(oracle):
    """HPE's second-order path derives tables from temporaries; a bound plan must not keep
    them (two different problems in a row would otherwise share a stale table)."""
    import mops_b200 as M
    r = np.random.default_rng(5)
    alive = []  # the contract: arrays a plan has seen stay alive and unchanged
    with M.Plan():
        for seed in (1, 2):
            d = workloads.hpe(I=80, N=9, J=30, K=3, seed=seed)
            d["grad_grad_A"] = r.standard_normal(d["A"].shape)
            alive.append(to_dev(d, np.float64))
            got = run_library("hpe", alive[-1], second_order=True)
            want = run_checker(oracle, "hpe", d, np.float64, second_order=True)
            for k in want:
                assert_parity(got[k], want[k], f"hpe second order with plan/{k}")


# ---------------------------------------------------------------- sorting the scatter index
@pytest.mark.parametrize("n,n_rows", [(1, 1), (33, 7), (5000, 300), (70001, 1 << 16),
                                      (300000, 70000), (1 << 20, 1 << 18), (4097, 1 << 24)])
def test_sort_indices_is_a_stable_sort(n, n_rows):
    import torch
    import mops_b200 as M
    r = np.random.default_rng(n)
    idx = r.integers(0, n_rows, n, dtype=np.int32)
    got, perm = M.sort_indices(torch.from_numpy(idx).cuda(), n_rows)
    want_perm = np.argsort(idx, kind="stable").astype(np.int32)
    assert np.array_equal(perm.cpu().numpy(), want_perm)
    assert np.array_equal(got.cpu().numpy(), idx[want_perm])
    # host arrays are staged
    got_h, perm_h = M.sort_indices(idx, n_rows)
    assert isinstance(got_h, np.ndarray) and np.array_equal(perm_h, want_perm)


def test_sort_indices_then_scatter_matches_the_oracle_on_unsorted_input(oracle):
    """The intended use: sort once on the device, permute the rows, run the segmented kernels
    (a plan then knows the index is sorted); same result as the oracle on the unsorted input."""
    import torch
    import mops_b200 as M
    d = workloads.opsaw(E=20000, n=300)
    shuffle = np.random.default_rng(9).permutation(20000)
    for k in ("A", "B", "indices_W", "indices_output"):
        d[k] = d[k][shuffle]
    want = run_checker(oracle, "opsaw", d, np.float64)
    t = to_dev(d, np.float64)
    PO, perm = M.sort_indices(t["indices_output"], 300)
    perm = perm.long()
    A, B, PW = t["A"][perm].contiguous(), t["B"][perm].contiguous(), t["indices_W"][perm].contiguous()
    with M.Plan() as plan:
        O = M.outer_product_scatter_add_with_weights(A, B, t["W"], PW, PO)
        gA, gB, gW = M.outer_product_scatter_add_with_weights_vjp(t["grad_output"], A, B, t["W"], PW, PO)
        assert plan.tables == 1
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(perm.numel(), device=perm.device)
    assert_parity(O.cpu().numpy(), want["output"], "sorted opsaw output")
    assert_parity(gA[inverse].cpu().numpy(), want["grad_A"], "sorted opsaw grad_A")
    assert_parity(gB[inverse].cpu().numpy(), want["grad_B"], "sorted opsaw grad_B")
    assert_parity(gW.cpu().numpy(), want["grad_W"], "sorted opsaw grad_W")


def test_sort_indices_reports_values_out_of_range():
    import torch
    import mops_b200 as M
    idx = torch.tensor([3, 1, 9, 2], dtype=torch.int32, device="cuda")
    with pytest.raises(M.MopsError, match="Index array indices in operation cuda_sort_index"):
        M.sort_indices(idx, 9)
