"""Seeded synthetic inputs for the five operations.

The reference measures on no public dataset; its benchmark programs draw random arrays
of fixed shapes (``mops/benchmarks/*.cpp``, ``python/mops/benchmarks/*.py``). The shapes
here follow those and the neighbour-list statistics of atomistic models (about 60
neighbours per atom). ``numpy.random.default_rng(seed)``; arrays are drawn in the order
listed in each function; "sorted" index arrays are ``np.sort`` of a uniform draw, so
rows receive Binomial(J, 1/n) ~ Poisson(J/n) entries and empty rows do occur.
``grad_output`` is drawn last. f32 variants are the f64 draws cast to f32.
"""
import numpy as np

SEEDS = {"hpe": 1001, "sap": 1002, "opsa": 1003, "opsaw": 1004, "sasaw": 1005}


def _f(x, dtype):
    return np.ascontiguousarray(x, dtype=dtype)


def hpe(I=1000, N=100, J=2000, K=4, dtype=np.float64, seed=SEEDS["hpe"]):
    r = np.random.default_rng(seed)
    A = r.uniform(-1, 1, (I, N))
    C = r.standard_normal(J)
    P = r.integers(0, N, (J, K), dtype=np.int32)
    gO = r.standard_normal(I)
    return dict(A=_f(A, dtype), C=_f(C, dtype), indices_A=P, grad_output=_f(gO, dtype))


def sap(I=1000, nA=20, nB=6, nO=50, K=1000, dtype=np.float64, seed=SEEDS["sap"]):
    r = np.random.default_rng(seed)
    A = r.uniform(-1, 1, (I, nA))
    B = r.uniform(-1, 1, (I, nB))
    C = r.standard_normal(K)
    PA = r.integers(0, nA, K, dtype=np.int32)
    PB = r.integers(0, nB, K, dtype=np.int32)
    PO = np.sort(r.integers(0, nO, K, dtype=np.int32))
    gO = r.standard_normal((I, nO))
    return dict(A=_f(A, dtype), B=_f(B, dtype), C=_f(C, dtype), indices_A=PA, indices_B=PB,
                indices_output=PO, output_size=nO, grad_output=_f(gO, dtype))


def opsa(J=60000, K=13, L=20, nO=1000, dtype=np.float64, seed=SEEDS["opsa"]):
    r = np.random.default_rng(seed)
    A = r.standard_normal((J, K))
    B = r.standard_normal((J, L))
    P = np.sort(r.integers(0, nO, J, dtype=np.int32))
    gO = r.standard_normal((nO, K, L))
    return dict(A=_f(A, dtype), B=_f(B, dtype), indices_output=P, output_size=nO,
                grad_output=_f(gO, dtype))


def opsaw(E=60000, K=13, L=32, n=1000, dtype=np.float64, seed=SEEDS["opsaw"]):
    r = np.random.default_rng(seed)
    A = r.standard_normal((E, K))
    B = r.standard_normal((E, L))
    W = r.standard_normal((n, L))
    PO = np.sort(r.integers(0, n, E, dtype=np.int32))
    PW = r.integers(0, n, E, dtype=np.int32)
    gO = r.standard_normal((n, K, L))
    return dict(A=_f(A, dtype), B=_f(B, dtype), W=_f(W, dtype), indices_W=PW,
                indices_output=PO, grad_output=_f(gO, dtype))


def sasaw(E=60000, nA=9, L=32, n=1000, N=500, nW2=9, nO2=9, dtype=np.float64,
          seed=SEEDS["sasaw"]):
    r = np.random.default_rng(seed)
    A = r.standard_normal((E, nA))
    B = r.standard_normal((E, L))
    W = r.standard_normal((n, nW2, L))
    Io = np.sort(r.integers(0, n, E, dtype=np.int32))
    Jw = r.integers(0, n, E, dtype=np.int32)
    C = r.standard_normal(N)
    M1 = r.integers(0, nA, N, dtype=np.int32)
    M2 = r.integers(0, nW2, N, dtype=np.int32)
    M3 = np.sort(r.integers(0, nO2, N, dtype=np.int32))
    gO = r.standard_normal((n, nO2, L))
    return dict(A=_f(A, dtype), B=_f(B, dtype), C=_f(C, dtype), W=_f(W, dtype), indices_A=M1,
                indices_W_1=Jw, indices_W_2=M2, indices_output_1=Io, indices_output_2=M3,
                output_size=nO2, grad_output=_f(gO, dtype))


GENERATORS = {"hpe": hpe, "sap": sap, "opsa": opsa, "opsaw": opsaw, "sasaw": sasaw}


def s_(dtype):
    return np.dtype(dtype).itemsize


def algorithmic_bytes(op, level, w):
    """Bytes one call must move: every input read once, every output written once, index
    arrays included, gathered W rows counted once. ``w`` is a dict made by a generator
    above; ``level`` is ``"fwd"`` or ``"vjp"``."""
    s = w["A"].dtype.itemsize
    if op == "hpe":
        I, N = w["A"].shape
        J, K = w["indices_A"].shape
        return s * (I * N + J + I) + 4 * J * K if level == "fwd" else \
            s * (2 * I * N + I + J) + 4 * J * K
    if op == "sap":
        I, nA = w["A"].shape
        nB, nO, K = w["B"].shape[1], w["output_size"], w["C"].shape[0]
        return s * I * (nA + nB + nO) + K * (s + 12) if level == "fwd" else \
            s * I * (nO + 2 * nA + 2 * nB) + K * (s + 12)
    if op == "opsa":
        J, K = w["A"].shape
        L, nO = w["B"].shape[1], w["output_size"]
        return s * J * (K + L) + 4 * J + s * nO * K * L if level == "fwd" else \
            s * nO * K * L + 2 * s * J * (K + L) + 4 * J
    if op == "opsaw":
        E, K = w["A"].shape
        L, n = w["B"].shape[1], w["W"].shape[0]
        fwd = s * E * (K + L) + 8 * E + s * n * L + s * n * K * L
        return fwd if level == "fwd" else fwd + s * E * (K + L) + s * n * L
    if op == "sasaw":
        E, nA = w["A"].shape
        L, N = w["B"].shape[1], w["C"].shape[0]
        Wn = w["W"].size
        On = w["W"].shape[0] * w["output_size"] * L
        fwd = s * E * (nA + L) + 8 * E + s * Wn + N * (s + 12) + s * On
        return fwd if level == "fwd" else fwd + s * E * (nA + L) + s * Wn
    raise KeyError(op)


def items(op, w):
    """Units one call processes: batch rows for HPE/SAP, entries (edges) for the scatter ops."""
    return w["A"].shape[0]


def useful_flops(op, level, w):
    """Floating-point operations one call needs when the work is organised the way the kernels
    organise it (multiply-add = 2). Only SASAW differs from the naive count: the coupling table
    is first contracted with the edge's A row into a dense nO2 x nW2 matrix T_e (2*cells*nA),
    which is then applied to the 32-wide rows (2*nO2*nW2*L per product)."""
    if op != "sasaw":
        raise KeyError(op)
    E, nA = w["A"].shape
    L = w["B"].shape[1]
    nW2, nO2 = w["W"].shape[1], w["output_size"]
    cells = nW2 * nO2
    contract = 2 * cells * nA          # T_e = D a_e   (and grad_A_e = D^T U_e)
    product = 2 * cells * L            # one nO2 x nW2 by nW2 x L product (or its transposes)
    scale_b = nW2 * L                  # B[e,:] * W[J_e]
    if level == "fwd":
        return E * (contract + product + scale_b)
    # VJP: T_e, X = T_e^T gO (grad_B, grad_W), U = gO (B*W)^T, grad_A = D^T U, and the
    # element-wise products that turn X into grad_B / grad_W
    return E * (2 * contract + 2 * product + 3 * scale_b)
