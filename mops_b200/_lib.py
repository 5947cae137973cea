"""Loads ``libmops.so`` (the sm_100a kernels behind the mops C ABI) and binds every symbol.

Mirrors python/mops/src/mops/_c_lib.py and _c_api.py of the reference: all 61 ABI symbols
are resolved at load, so a library that lacks one fails here, loudly, and not at first use.
There is no fallback of any kind: without the built library this module raises ImportError.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmops.so")

OPERATIONS = (
    "homogeneous_polynomial_evaluation",
    "sparse_accumulation_of_products",
    "outer_product_scatter_add",
    "outer_product_scatter_add_with_weights",
    "sparse_accumulation_scatter_add_with_weights",
)
LEVELS = ("", "_vjp", "_vjp_vjp")
DTYPES = ("f32", "f64")


def abi_symbols():
    """The 60 operation entry points + the error getter, as the reference ABI names them."""
    names = [f"mops_{dev}{op}{lvl}_{dt}" for op in OPERATIONS for lvl in LEVELS
             for dev in ("", "cuda_") for dt in DTYPES]
    return names + ["mops_get_last_error_message"]


EXTENSION_SYMBOLS = ("mops_b200_set_stream", "mops_b200_get_stream", "mops_b200_set_wait",
                     "mops_b200_get_wait", "mops_b200_version", "mops_b200_last_kernels",
                     "mops_b200_plan_create", "mops_b200_plan_destroy", "mops_b200_plan_bind",
                     "mops_b200_plan_bound", "mops_b200_plan_tables", "mops_b200_cuda_sort_index",
                     "mops_b200_cuda_sparse_accumulation_scatter_add_with_weights_noalloc_f64")


class MopsError(Exception):
    """Raised for every non-zero status of the C ABI (python/mops/src/mops/status.py:4-16)."""

    def __init__(self, message, status=None):
        super().__init__(message)
        self.message = message
        self.status = status


_LIB = None


def library():
    global _LIB
    if _LIB is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: build it with `python -m mops_b200.build` "
                "(there is no CPU or pure-Python fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name in abi_symbols() + list(EXTENSION_SYMBOLS):
            getattr(lib, name)  # AttributeError here = incomplete ABI
        lib.mops_get_last_error_message.restype = ctypes.c_char_p
        lib.mops_b200_version.restype = ctypes.c_char_p
        lib.mops_b200_last_kernels.restype = ctypes.c_char_p
        lib.mops_b200_plan_create.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        lib.mops_b200_plan_destroy.argtypes = [ctypes.c_void_p]
        lib.mops_b200_plan_bind.argtypes = [ctypes.c_void_p]
        lib.mops_b200_plan_bind.restype = None
        lib.mops_b200_plan_bound.restype = ctypes.c_void_p
        lib.mops_b200_plan_tables.argtypes = [ctypes.c_void_p]
        lib.mops_b200_set_stream.argtypes = [ctypes.c_void_p]
        lib.mops_b200_get_stream.restype = ctypes.c_void_p
        lib.mops_b200_set_wait.argtypes = [ctypes.c_int]
        _LIB = lib
    return _LIB


def last_kernels():
    """Main kernels (with template arguments) of this thread's last call, as a list."""
    text = library().mops_b200_last_kernels().decode("utf8")
    return [k for k in text.split("; ") if k]


def last_error():
    return library().mops_get_last_error_message().decode("utf8")


def check_status(status):
    if status != 0:
        raise MopsError(last_error(), status)


def _struct(ndim):
    class Tensor(ctypes.Structure):
        _fields_ = [("data", ctypes.c_void_p), ("shape", ctypes.c_int64 * ndim)]
    return Tensor


TENSOR = {n: _struct(n) for n in (1, 2, 3)}


def make_struct(ptr, shape):
    t = TENSOR[len(shape)]()
    t.data = ptr
    for d, s in enumerate(shape):
        t.shape[d] = s
    return t


def null_struct(ndim):
    """``{NULL, {0,...}}``: "do not compute this gradient" (python/mops/src/mops/utils.py:81-109)."""
    t = TENSOR[ndim]()
    t.data = None
    return t


def call(symbol, structs):
    fn = getattr(library(), symbol)
    fn.restype = ctypes.c_int
    fn.argtypes = [type(s) for s in structs]
    check_status(fn(*structs))
