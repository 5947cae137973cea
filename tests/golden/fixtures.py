"""Inputs of the golden-vector cases.

Shapes and the seed are those of the reference's own test fixtures
(python/mops/tests/{hpe,sap,opsa,opsaw,sasaw}{,_vjp}.py: ``np.random.seed(0xDEADBEEF)``,
``np.random.rand`` / ``randint``; batch 99 exercises the reference's SIMD remainder path;
scatter indices are unsorted; OPSA/OPSAW have a variant that leaves output row 1 empty).
NumPy's legacy ``RandomState`` stream is frozen, so the inputs are regenerated here and
only the expected outputs are stored in ``golden.npz``.
"""
import numpy as np

SEED = 0xDEADBEEF


def _rs():
    return np.random.RandomState(SEED)


def hpe():
    r = _rs()
    d = dict(A=r.rand(99, 20), C=r.rand(200),
             indices_A=r.randint(20, size=(200, 4)).astype(np.int32), grad_output=r.rand(99))
    d["grad_grad_A"] = r.rand(99, 20)
    return d


def sap():
    r = _rs()
    d = dict(A=r.rand(99, 20), B=r.rand(99, 6), C=r.rand(30),
             indices_A=r.randint(20, size=30).astype(np.int32),
             indices_B=r.randint(6, size=30).astype(np.int32),
             indices_output=r.randint(35, size=30).astype(np.int32), output_size=35)
    d["grad_output"] = r.rand(99, 35)
    d["grad_grad_A"] = r.rand(99, 20)
    d["grad_grad_B"] = r.rand(99, 6)
    return d


def opsa(empty_row=False):
    r = _rs()
    d = dict(A=r.rand(100, 10), B=r.rand(100, 5),
             indices_output=r.randint(10, size=100).astype(np.int32), output_size=10)
    d["grad_output"] = r.rand(10, 10, 5)
    d["grad_grad_A"] = r.rand(100, 10)
    d["grad_grad_B"] = r.rand(100, 5)
    if empty_row:
        d["indices_output"][d["indices_output"] == 1] = 2
    return d


def opsaw(empty_row=False):
    r = _rs()
    d = dict(A=r.rand(100, 10), B=r.rand(100, 5), W=r.rand(20, 5),
             indices_W=r.randint(20, size=100).astype(np.int32),
             indices_output=r.randint(20, size=100).astype(np.int32))
    d["grad_output"] = r.rand(20, 10, 5)
    if empty_row:
        d["indices_output"][d["indices_output"] == 1] = 2
    return d


def sasaw():
    r = _rs()
    d = dict(A=r.rand(100, 20), B=r.rand(100, 200), W=r.rand(25, 13, 200), C=r.rand(50),
             indices_output_1=r.randint(25, size=100).astype(np.int32),
             indices_W_1=r.randint(25, size=100).astype(np.int32), output_size=15,
             indices_A=r.randint(20, size=50).astype(np.int32),
             indices_W_2=r.randint(13, size=50).astype(np.int32),
             indices_output_2=r.randint(15, size=50).astype(np.int32))
    d["grad_output"] = r.rand(25, 15, 200)
    return d


CASES = {
    "hpe": hpe, "sap": sap,
    "opsa": opsa, "opsa_empty_row": lambda: opsa(True),
    "opsaw": opsaw, "opsaw_empty_row": lambda: opsaw(True),
    "sasaw": sasaw,
}
