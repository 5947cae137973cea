"""Parity of results computed at sizes the CPU oracle cannot afford in full.

Test infrastructure (the checker role): compares results of the library under test with the
CPU oracle on sub-ranges, using the independence the five operations have.

* HPE, SAP: batch rows are independent, so the oracle is run on three blocks of rows (the
  first rows, a block in the middle, the last, ragged, rows).
* OPSA: with a sorted scatter index a range of output rows owns a contiguous range of
  entries; the oracle is run on those entries with the index rebased to the range's first
  row. grad_A / grad_B of the same entries need only the range's rows of grad_output.
* OPSAW, SASAW: W is gathered by an unrelated index, so the oracle gets the whole W and a
  full-size output (rows outside the range stay zero) but only the range's entries.
* grad_W of OPSAW / SASAW sums over all entries: it is checked by running the library and
  the oracle on a slice of at most 2^16 entries (same W, same grad_output), and at full
  size through the adjoint identity <grad_output, O> = <grad_W, W> (the forward is linear
  in W, and in A and in B).

``results`` may hold torch tensors on any device or NumPy arrays; only the compared
sub-ranges are copied to the host.
"""
import numpy as np

TOL = {np.dtype("float64"): 1e-12, np.dtype("float32"): 1e-5}
# the adjoint identity compares two sums of ~1e8 products, each carrying the kernels' rounding
ADJOINT_TOL = {np.dtype("float64"): 1e-9, np.dtype("float32"): 1e-4}

ROW_BLOCK = 4096      # batch rows per block (HPE, SAP)
SEGMENT_BLOCK = 256   # output rows per block (scatter ops)
GRAD_W_SLICE = 1 << 16


class Mismatch(AssertionError):
    pass


def _np(x, sl=None):
    if x is None:
        return None
    if sl is not None:
        x = x[sl]
    if isinstance(x, np.ndarray):
        return np.ascontiguousarray(x)
    return np.ascontiguousarray(x.detach().cpu().numpy())


def compare(actual, expected, what, report):
    actual, expected = np.asarray(actual), np.asarray(expected)
    if actual.shape != expected.shape or actual.dtype != expected.dtype:
        raise Mismatch(f"{what}: {actual.dtype}{actual.shape} != {expected.dtype}{expected.shape}")
    if expected.size == 0:
        return
    tol = TOL[expected.dtype]
    scale = float(np.max(np.abs(expected)))
    err = float(np.max(np.abs(actual.astype(np.float64) - expected.astype(np.float64))))
    report.append({"what": what, "max_abs_err": err, "scale": scale, "n": int(expected.size)})
    if not np.isfinite(actual).all():
        raise Mismatch(f"{what}: non-finite values")
    if err > tol * max(scale, 1e-300):
        raise Mismatch(f"{what}: max|diff| = {err:.3e} > {tol:g} * {scale:.3e}")


def row_blocks(n, size):
    """First, middle and last (ragged: deliberately not aligned to `size`) blocks of [0, n)."""
    if n <= 3 * size:
        return [(0, n)]
    mid = (n // 2) // 32 * 32 + 5
    return [(0, size), (mid, mid + size), (n - size + 37, n)]


def _entries(index, r0, r1):
    return int(np.searchsorted(index, r0, side="left")), int(np.searchsorted(index, r1, side="left"))


def _is_sorted(index):
    return index.size == 0 or not bool(np.any(index[1:] < index[:-1]))


def check_hpe(oracle, d, results, report):
    I = d["A"].shape[0]
    for a, b in row_blocks(I, ROW_BLOCK):
        A, gO = d["A"][a:b], d["grad_output"][a:b]
        if "output" in results:
            compare(_np(results["output"], slice(a, b)), oracle.hpe(A, d["C"], d["indices_A"]),
                    f"hpe output rows [{a},{b})", report)
        if "grad_A" in results:
            compare(_np(results["grad_A"], slice(a, b)),
                    oracle.hpe_vjp(gO, A, d["C"], d["indices_A"]), f"hpe grad_A rows [{a},{b})",
                    report)


def check_sap(oracle, d, results, report):
    I = d["A"].shape[0]
    idx = (d["indices_A"], d["indices_B"], d["indices_output"])
    for a, b in row_blocks(I, ROW_BLOCK):
        A, B, gO = d["A"][a:b], d["B"][a:b], d["grad_output"][a:b]
        if "output" in results:
            compare(_np(results["output"], slice(a, b)),
                    oracle.sap(A, B, d["C"], *idx, d["output_size"]),
                    f"sap output rows [{a},{b})", report)
        if "grad_A" in results:
            gA, gB = oracle.sap_vjp(gO, A, B, d["C"], *idx)
            compare(_np(results["grad_A"], slice(a, b)), gA, f"sap grad_A rows [{a},{b})", report)
            compare(_np(results["grad_B"], slice(a, b)), gB, f"sap grad_B rows [{a},{b})", report)


def check_opsa(oracle, d, results, report):
    P, nO = d["indices_output"], d["output_size"]
    assert _is_sorted(P), "sub-range checks need a sorted scatter index"
    for r0, r1 in row_blocks(nO, SEGMENT_BLOCK):
        lo, hi = _entries(P, r0, r1)
        A, B, Ploc = d["A"][lo:hi], d["B"][lo:hi], (P[lo:hi] - r0).astype(np.int32)
        if "output" in results:
            compare(_np(results["output"], slice(r0, r1)), oracle.opsa(A, B, Ploc, r1 - r0),
                    f"opsa output rows [{r0},{r1}) entries [{lo},{hi})", report)
        if "grad_A" in results:
            gA, gB = oracle.opsa_vjp(d["grad_output"][r0:r1], A, B, Ploc)
            compare(_np(results["grad_A"], slice(lo, hi)), gA, f"opsa grad_A entries [{lo},{hi})",
                    report)
            compare(_np(results["grad_B"], slice(lo, hi)), gB, f"opsa grad_B entries [{lo},{hi})",
                    report)


def check_opsaw(oracle, d, results, report):
    PO, PW, n = d["indices_output"], d["indices_W"], d["W"].shape[0]
    assert _is_sorted(PO), "sub-range checks need a sorted scatter index"
    for r0, r1 in row_blocks(n, SEGMENT_BLOCK):
        lo, hi = _entries(PO, r0, r1)
        A, B = d["A"][lo:hi], d["B"][lo:hi]
        if "output" in results:
            want = oracle.opsaw(A, B, d["W"], PW[lo:hi], PO[lo:hi])
            compare(_np(results["output"], slice(r0, r1)), want[r0:r1],
                    f"opsaw output rows [{r0},{r1}) entries [{lo},{hi})", report)
        if "grad_A" in results:
            gA, gB, _ = oracle.opsaw_vjp(d["grad_output"], A, B, d["W"], PW[lo:hi], PO[lo:hi],
                                         need=(True, True, False))
            compare(_np(results["grad_A"], slice(lo, hi)), gA, f"opsaw grad_A entries [{lo},{hi})",
                    report)
            compare(_np(results["grad_B"], slice(lo, hi)), gB, f"opsaw grad_B entries [{lo},{hi})",
                    report)


def _sasaw_idx(d, lo, hi):
    return (d["indices_A"], d["indices_W_1"][lo:hi], d["indices_W_2"],
            d["indices_output_1"][lo:hi], d["indices_output_2"])


def check_sasaw(oracle, d, results, report):
    Io, n = d["indices_output_1"], d["W"].shape[0]
    assert _is_sorted(Io), "sub-range checks need a sorted scatter index"
    for r0, r1 in row_blocks(n, SEGMENT_BLOCK):
        lo, hi = _entries(Io, r0, r1)
        A, B = d["A"][lo:hi], d["B"][lo:hi]
        if "output" in results:
            want = oracle.sasaw(A, B, d["C"], d["W"], *_sasaw_idx(d, lo, hi), d["output_size"])
            compare(_np(results["output"], slice(r0, r1)), want[r0:r1],
                    f"sasaw output rows [{r0},{r1}) entries [{lo},{hi})", report)
        if "grad_A" in results:
            gA, gB, _ = oracle.sasaw_vjp(d["grad_output"], A, B, d["C"], d["W"],
                                         *_sasaw_idx(d, lo, hi), need=(True, True, False))
            compare(_np(results["grad_A"], slice(lo, hi)), gA, f"sasaw grad_A entries [{lo},{hi})",
                    report)
            compare(_np(results["grad_B"], slice(lo, hi)), gB, f"sasaw grad_B entries [{lo},{hi})",
                    report)


def grad_w_slice(op, d):
    """Inputs of the same problem restricted to a contiguous slice of at most 2^16 entries
    that starts in the middle of the entry range (W, grad_output and the coupling table
    whole): small enough for the oracle, and large enough that the gathered W rows and the
    scattered grad_W rows spread over the whole of W."""
    E = d["A"].shape[0]
    n = min(GRAD_W_SLICE, E)
    lo = (E - n) // 2
    sl = slice(lo, lo + n)
    per_entry = {"opsaw": ("A", "B", "indices_W", "indices_output"),
                 "sasaw": ("A", "B", "indices_W_1", "indices_output_1")}[op]
    return {k: (v[sl] if k in per_entry else v) for k, v in d.items()}, (lo, lo + n)


def check_grad_w_slice(oracle, op, d, library_vjp, report):
    """``library_vjp(sub)`` -> grad_W of the library under test for the sliced problem."""
    sub, (lo, hi) = grad_w_slice(op, d)
    got = _np(library_vjp(sub))
    if op == "opsaw":
        _, _, want = oracle.opsaw_vjp(sub["grad_output"], sub["A"], sub["B"], sub["W"],
                                      sub["indices_W"], sub["indices_output"],
                                      need=(False, False, True))
    else:
        _, _, want = oracle.sasaw_vjp(sub["grad_output"], sub["A"], sub["B"], sub["C"], sub["W"],
                                      sub["indices_A"], sub["indices_W_1"], sub["indices_W_2"],
                                      sub["indices_output_1"], sub["indices_output_2"],
                                      need=(False, False, True))
    compare(got, want, f"{op} grad_W of entries [{lo},{hi})", report)


def _dot(x, y):
    if isinstance(x, np.ndarray):
        return float(np.sum(x.astype(np.float64) * np.asarray(y, dtype=np.float64)))
    import torch
    if not isinstance(y, torch.Tensor):
        y = torch.from_numpy(np.ascontiguousarray(y)).to(x.device)
    return float((x.double() * y.double()).sum())


def check_adjoint(op, d, results, report, inputs=None):
    """<grad_output, O> equals <grad_X, X> for every operand X the forward is linear in.
    ``inputs`` may hold device copies of the operands (else the host arrays are used)."""
    if "output" not in results or "grad_A" not in results:
        return
    src = inputs if inputs is not None else d
    dtype = np.dtype(d["A"].dtype)
    lhs = _dot(results["output"], src["grad_output"])
    pairs = {"hpe": (), "sap": ("A", "B"), "opsa": ("A", "B"), "opsaw": ("A", "B", "W"),
             "sasaw": ("A", "B", "W")}[op]
    for name in pairs:
        if "grad_" + name not in results:
            continue
        rhs = _dot(results["grad_" + name], src[name])
        rel = abs(lhs - rhs) / max(abs(lhs), 1.0)
        report.append({"what": f"{op} <gO,O> = <grad_{name},{name}>", "max_abs_err": abs(lhs - rhs),
                       "scale": abs(lhs), "n": 1})
        if rel > ADJOINT_TOL[dtype]:
            raise Mismatch(f"{op}: <gO,O> = {lhs!r} but <grad_{name},{name}> = {rhs!r}")


CHECKS = {"hpe": check_hpe, "sap": check_sap, "opsa": check_opsa, "opsaw": check_opsaw,
          "sasaw": check_sasaw}


def check_case(oracle, op, d, results, inputs=None, library_vjp=None):
    """All sub-range checks of one case. ``d``: host inputs (NumPy); ``results``: name ->
    array (device or host) with keys output / grad_A / grad_B / grad_W. Returns the list of
    comparisons made; raises Mismatch on the first one out of tolerance."""
    report = []
    CHECKS[op](oracle, d, results, report)
    check_adjoint(op, d, results, report, inputs)
    if op in ("opsaw", "sasaw") and library_vjp is not None:
        check_grad_w_slice(oracle, op, d, library_vjp, report)
    return report
