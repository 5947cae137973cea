"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol that
include/mops.h declares, keeps the reference's status/error convention, and rejects bad
shapes with the reference's messages before touching a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from mops_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_all_61_reference_symbols():
    lib = _lib.library()
    names = _lib.abi_symbols()
    assert len(names) == 61 and len(set(names)) == 61
    for n in names:
        assert hasattr(lib, n), n


def test_header_and_library_agree():
    """Every prototype the header generates is exported, and nothing else with a mops_ prefix."""
    header = open(os.path.join(ROOT, "include", "mops.h")).read()
    ops = re.findall(r"^\s+X\((\w+), MOPS_ARGS_\w+\)", header, flags=re.M)
    assert len(ops) == 15
    declared = {f"mops_{dev}{op}_{dt}" for op in ops for dev in ("", "cuda_") for dt in ("f32", "f64")}
    declared |= set(re.findall(r"MOPS_EXPORT [\w\s\*]+?(mops_\w+)\(", header))
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True,
                         text=True, check=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l and l.split()[-1].startswith("mops_")}
    assert declared == exported, (declared ^ exported)


def test_host_entry_points_report_that_this_build_is_cuda_only():
    A = np.zeros((3, 2))
    out = np.zeros((2, 2, 2))
    P = np.zeros(3, np.int32)
    s = [_lib.make_struct(out.ctypes.data, out.shape), _lib.make_struct(A.ctypes.data, A.shape),
         _lib.make_struct(A.ctypes.data, A.shape), _lib.make_struct(P.ctypes.data, P.shape)]
    with pytest.raises(_lib.MopsError, match="CUDA .* implementations only") as e:
        _lib.call("mops_outer_product_scatter_add_f64", s)
    assert e.value.status == 1


def test_second_order_entry_points_without_a_kernel_say_so():
    z2, z3, i1 = _lib.null_struct(2), _lib.null_struct(3), _lib.null_struct(1)
    with pytest.raises(_lib.MopsError, match="Not implemented"):
        _lib.call("mops_cuda_outer_product_scatter_add_with_weights_vjp_vjp_f64",
                  [z3, z2, z2, z2, z2, z2, z2, z3, z2, z2, z2, i1, i1])
    # OPSA's second order exists (all outputs skipped: returns without touching the device)
    _lib.call("mops_cuda_outer_product_scatter_add_vjp_vjp_f64",
              [z3, z2, z2, z2, z2, z3, z2, z2, i1])
    z1, i2 = _lib.null_struct(1), _lib.null_struct(2)
    _lib.call("mops_cuda_homogeneous_polynomial_evaluation_vjp_vjp_f32",
              [z1, z2, z2, z1, z2, z1, i2])  # likewise for HPE


def _fake(shape):
    """A struct with a non-null but never-dereferenced pointer: shape checks come first."""
    return _lib.make_struct(0x1000, shape)


@pytest.mark.parametrize("symbol,structs,message", [
    ("mops_cuda_homogeneous_polynomial_evaluation_f64",
     [(99,), (99, 20), (200,), (199, 4)],
     "Dimension mismatch: the sizes of C along dimension 0 and indices_A along dimension 0 "
     "must match in cuda_homogeneous_polynomial_evaluation"),
    ("mops_cuda_sparse_accumulation_of_products_f32",
     [(99, 35), (99, 20), (98, 6), (30,), (30,), (30,), (30,)],
     "Dimension mismatch: the sizes of A along dimension 0 and B along dimension 0 must match "
     "in cuda_sparse_accumulation_of_products"),
    ("mops_cuda_outer_product_scatter_add_f64",
     [(10, 10, 5), (100, 10), (100, 5), (101,)],
     "Dimension mismatch: the sizes of A along dimension 0 and indices_output along dimension 0 "
     "must match in cuda_outer_product_scatter_add"),
    ("mops_cuda_outer_product_scatter_add_with_weights_f64",
     [(20, 10, 5), (100, 10), (100, 5), (20, 6), (100,), (100,)],
     "Dimension mismatch: the sizes of B along dimension 1 and W along dimension 1 must match "
     "in cuda_outer_product_scatter_add_with_weights"),
    ("mops_cuda_sparse_accumulation_scatter_add_with_weights_f64",
     [(25, 15, 200), (100, 20), (100, 200), (50,), (25, 13, 200), (50,), (100,), (49,), (100,), (50,)],
     "Dimension mismatch: the sizes of C along dimension 0 and indices_W_2 along dimension 0 "
     "must match in cuda_sparse_accumulation_scatter_add_with_weights"),
    ("mops_cuda_outer_product_scatter_add_vjp_f64",
     [(100, 11), (100, 5), (10, 10, 5), (100, 10), (100, 5), (100,)],
     "Dimension mismatch: the sizes of grad_A along dimension 1 and A along dimension 1 must "
     "match in cuda_outer_product_scatter_add_vjp"),
])
def test_shape_errors_match_the_reference_text(symbol, structs, message):
    with pytest.raises(_lib.MopsError) as e:
        _lib.call(symbol, [_fake(s) for s in structs])
    assert e.value.status == 1
    assert str(e.value) == message
    assert _lib.last_error() == message


def test_negative_shape_is_rejected():
    with pytest.raises(_lib.MopsError, match="integer value '-3' does not fit in size_t"):
        _lib.call("mops_cuda_outer_product_scatter_add_f64",
                  [_fake((10, 10, 5)), _fake((-3, 10)), _fake((100, 5)), _fake((100,))])


def test_front_end_argument_checks():
    """Same exception types and texts as python/mops/tests/*.py expect."""
    import mops_b200 as M
    A, C, P = np.zeros((9, 4)), np.zeros(7), np.zeros((7, 3), np.int32)
    with pytest.raises(TypeError, match="Wrong dtype for A in homogeneous_polynomial_evaluation: got int32"):
        M.homogeneous_polynomial_evaluation(A.astype(np.int32), C, P)
    with pytest.raises(ValueError, match="`A` must be a 2D array in homogeneous_polynomial_evaluation, "
                                         "got a 3D array instead"):
        M.homogeneous_polynomial_evaluation(A[..., None], C, P)
    with pytest.raises(TypeError, match="Wrong dtype for indices_output in outer_product_scatter_add"):
        M.outer_product_scatter_add(A, A, np.zeros(9), 3)


def test_stream_and_wait_extensions():
    lib = _lib.library()
    assert lib.mops_b200_get_wait() == 1
    lib.mops_b200_set_wait(0)
    assert lib.mops_b200_get_wait() == 0
    lib.mops_b200_set_wait(1)
    assert lib.mops_b200_get_stream() in (None, 0)
    assert b"sm_100a" in lib.mops_b200_version()
