"""mops_b200: the five mops sparse operations on B200 (sm_100a), behind the reference's API.

This package mirrors the Python front end of lab-cosmo/mops (python/mops/src/mops): the same
fifteen functions with the same names, argument order, keyword arguments, return values and
error types, calling the same C ABI (``mops_cuda_*``) of the library built from
``mops_b200/csrc``.

Accepted arrays
  * ``torch.Tensor`` on a CUDA device: used in place (device pointers), results are CUDA
    tensors on the same device. Runs on torch's current stream and returns when complete.
  * ``numpy.ndarray`` (or CPU ``torch.Tensor``): the reference would run its CPU code; this
    build has none, so host arrays are staged to the current CUDA device, the same kernels
    run, and the result comes back as a host array of the same kind. This is the
    "host buffers in, host buffers out" path timed as ``e2e`` by ``bench.py``.

  * Inside ``with mops_b200.HostQueue():`` calls on host arrays do not wait: their copies
    in, kernels and copies out are queued on three CUDA streams and overlap across calls;
    results are valid when the block ends.

Differences from the reference front end: no CuPy dispatch (CuPy is replaced by torch CUDA
tensors); OPSAW and SASAW run on the GPU instead of raising "CUDA implementation does not
exist yet".
"""
import ctypes
import threading

import numpy as np

from . import _lib
from ._lib import MopsError  # noqa: F401

__all__ = [f"{op}{lvl}" for op in _lib.OPERATIONS for lvl in _lib.LEVELS] + [
    "MopsError", "HostQueue", "Plan", "sort_indices"]


def _torch():
    import torch
    return torch


# ----------------------------------------------------------------------------- array handling
def _is_array(x):
    if isinstance(x, np.ndarray):
        return True
    torch = _torch()
    return isinstance(x, torch.Tensor)


def _dtype_name(x):
    return str(x.dtype).replace("torch.", "")


def _is_floating(x):
    if isinstance(x, np.ndarray):
        return np.issubdtype(x.dtype, np.floating)
    return x.dtype.is_floating_point


def _is_integer(x):
    if isinstance(x, np.ndarray):
        return np.issubdtype(x.dtype, np.integer)
    torch = _torch()
    return x.dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


def _check(array, ndim, kind, operation, name):
    """Same checks and messages as python/mops/src/mops/checks.py:9-35."""
    if not _is_array(array):
        raise TypeError(f"`{name}` must be an array in {operation}, got {type(array)}")
    if len(array.shape) != ndim:
        raise ValueError(f"`{name}` must be a {ndim}D array in {operation}, "
                         f"got a {len(array.shape)}D array instead")
    ok = _is_floating(array) if kind == "f" else _is_integer(array)
    if not ok:
        raise TypeError(f"Wrong dtype for {name} in {operation}: got {_dtype_name(array)}")


def _check_scalar(value, operation, name):
    if not isinstance(value, (int, np.integer)) or isinstance(value, bool):
        raise TypeError(f"`{name}` must be a scalar in {operation}, got {type(value)}")


def sort_indices(indices, n_rows):
    """Stable sort of a scatter index on the GPU: returns ``(sorted, permutation)`` with
    ``sorted == indices[permutation]`` ascending and equal values in input order, as int32
    arrays of the kind given (CUDA tensor in, CUDA tensors out; host arrays are staged through
    the current device). Permute the rows of ``A``, ``B`` (and ``indices_W``) with
    ``permutation`` to get the sorted problem the scatter operations run fastest on."""
    op = "sort_indices"
    _check(indices, 1, "i", op, "indices")
    _check_scalar(n_rows, op, "n_rows")
    torch = _torch()
    numpy_in = isinstance(indices, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(indices)) if numpy_in else indices
    was_cuda = t.is_cuda
    if not torch.cuda.is_available():
        raise MopsError("no CUDA device available")
    dev = t.device if was_cuda else torch.device("cuda", torch.cuda.current_device())
    t = t.to(dev).to(torch.int32).contiguous()
    out, perm = torch.empty_like(t), torch.empty_like(t)
    lib = _lib.library()
    fn = lib.mops_b200_cuda_sort_index
    structs = [_lib.make_struct(x.data_ptr(), x.shape) for x in (out, perm, t)]
    fn.restype, fn.argtypes = ctypes.c_int, [type(s) for s in structs] + [ctypes.c_int64]
    with torch.cuda.device(dev):
        previous = lib.mops_b200_get_stream()
        lib.mops_b200_set_stream(torch.cuda.current_stream().cuda_stream)
        try:
            _lib.check_status(fn(*structs, int(n_rows)))
        finally:
            lib.mops_b200_set_stream(previous)
    if was_cuda:
        return out, perm
    out, perm = out.cpu(), perm.cpu()
    return (out.numpy(), perm.numpy()) if numpy_in else (out, perm)


class Plan:
    """Device tables built once and reused (``mops_b200_plan_*`` of the C ABI).

    Inside ``with plan:`` every operation called on CUDA tensors builds the table it derives
    from its index (and coefficient) arrays only the first time it sees those arrays (same
    device addresses and sizes) and reuses it afterwards: the segment offsets of a sorted
    scatter index are shared by the forward and the VJP of one graph, HPE / SAP / SASAW
    coupling tables are not rebuilt, and sorted scatter calls no longer stop mid-way to ask
    the device whether the index was sorted. The caller must keep the index tensors alive and
    unchanged while the plan holds tables for them. Binding is per thread: operations that
    run on another thread (torch's autograd engine) do not see it."""

    def __init__(self):
        handle = ctypes.c_void_p()
        _lib.check_status(_lib.library().mops_b200_plan_create(ctypes.byref(handle)))
        self._handle = handle
        self._previous = None

    def __enter__(self):
        lib = _lib.library()
        self._previous = lib.mops_b200_plan_bound()
        lib.mops_b200_plan_bind(self._handle)
        return self

    def __exit__(self, *exc):
        _lib.library().mops_b200_plan_bind(self._previous)
        return False

    @property
    def tables(self):
        """Number of tables the plan holds."""
        return int(_lib.library().mops_b200_plan_tables(self._handle))

    def close(self):
        if self._handle is not None:
            _lib.library().mops_b200_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostQueue:
    """Overlaps the host<->device traffic of consecutive calls on host arrays.

    Inside ``with HostQueue() as q:`` every operation called with host arrays (NumPy arrays or
    CPU torch tensors; pinned memory makes the copies asynchronous) is queued instead of
    waited for: operands are copied in on one stream, the kernels run on a second, results
    are copied out to pinned host memory on a third, chained by events. While one call
    computes, the next call's operands arrive and the previous call's results leave (PCIe is
    full duplex). A host array that several queued calls share (the operands of a forward and
    of its VJP) is copied once. The arrays a call returns are filled when ``q.wait()``
    returns or the block ends; until then their contents are undefined, and the operands
    must not be modified. Like ``mops_b200_set_wait(0)``, queued calls do not report index
    errors found on the device.
    """

    _local = threading.local()

    def __init__(self, device=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise MopsError("no CUDA device available")
        index = torch.cuda.current_device() if device is None else torch.device(device).index
        self.device = torch.device("cuda", index)
        # The three streams are made once per thread and device and shared by the queues that
        # follow each other: torch's caching allocator keeps freed device memory per stream, so
        # a queue on fresh streams could not reuse what the previous queue's arrays occupied
        # (28 GB per step of the benchmark: the device filled up within a few steps and every
        # so often a step stalled for half a second while the allocator emptied its cache).
        streams = getattr(HostQueue._local, "streams", None)
        if streams is None:
            streams = HostQueue._local.streams = {}
        if index not in streams:
            streams[index] = tuple(torch.cuda.Stream(device=self.device) for _ in range(3))
        self.copy_in, self.compute, self.copy_out = streams[index]
        self._operands = {}  # (address, bytes, dtype) -> (device tensor, event, host array)
        self._keep = []

    @classmethod
    def current(cls):
        return getattr(cls._local, "queue", None)

    def __enter__(self):
        if HostQueue.current() is not None:
            raise MopsError("HostQueue blocks do not nest")
        HostQueue._local.queue = self
        return self

    def __exit__(self, *exc):
        HostQueue._local.queue = None
        self.wait()
        return False

    def wait(self):
        """Returns when every queued call is complete and its results are in host memory."""
        self.copy_out.synchronize()
        self.compute.synchronize()
        self.copy_in.synchronize()
        self._operands.clear()
        self._keep.clear()

    def operand(self, host_tensor, convert=None):
        """Device copy of a host tensor (made once per wait() period) and its ready event."""
        torch = _torch()
        key = (host_tensor.data_ptr(), host_tensor.numel() * host_tensor.element_size(),
               host_tensor.dtype, convert)
        hit = self._operands.get(key)
        if hit is None:
            with torch.cuda.stream(self.copy_in):
                dev = host_tensor.to(self.device, non_blocking=True)
                if convert is not None:
                    dev = dev.to(convert)
                ready = torch.cuda.Event()
                ready.record(self.copy_in)
            hit = (dev.contiguous(), ready, host_tensor)
            self._operands[key] = hit
        return hit[0], hit[1]


class _Arena:
    """Moves one call's arrays to the device and its results back to where the inputs live."""

    def __init__(self, first):
        torch = _torch()
        if not torch.cuda.is_available():
            raise MopsError("no CUDA device available: this build of mops runs on the GPU only "
                            "(there is no CPU implementation to fall back to)")
        self.torch = torch
        self.numpy = isinstance(first, np.ndarray)
        self.pinned = (not self.numpy) and (not first.is_cuda) and first.is_pinned()
        self.queue = None
        if self.numpy or not first.is_cuda:
            self.queue = HostQueue.current()
            self.device = (self.queue.device if self.queue is not None
                           else torch.device("cuda", torch.cuda.current_device()))
            self.host = True
            self.ready = []
            self.done = None
        else:
            self.device = first.device
            self.host = False
        if isinstance(first, np.ndarray):
            self.dtype = {np.dtype("float32"): torch.float32,
                          np.dtype("float64"): torch.float64}.get(first.dtype)
        else:
            self.dtype = first.dtype if first.dtype in (torch.float32, torch.float64) else None
        if self.dtype is None:
            raise TypeError("Unsupported dtype detected. Only float32 and float64 are supported")
        self.suffix = "f32" if self.dtype == torch.float32 else "f64"

    def floats(self, x):
        t = self.torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x
        if t.dtype != self.dtype:
            raise TypeError("all floating-point arrays of one call must have the same dtype")
        if self.queue is not None and not t.is_cuda:
            dev, ready = self.queue.operand(t.contiguous())
            self.ready.append(ready)
            return dev
        return t.to(self.device, non_blocking=True).contiguous()

    def ints(self, x):
        t = self.torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x
        if self.queue is not None and not t.is_cuda:
            dev, ready = self.queue.operand(t.contiguous(), convert=self.torch.int32)
            self.ready.append(ready)
            return dev
        return t.to(self.device, non_blocking=True).to(self.torch.int32).contiguous()

    def empty(self, shape):
        shape = tuple(int(s) for s in shape)
        if self.queue is not None:
            with self.torch.cuda.stream(self.queue.compute):
                t = self.torch.empty(shape, dtype=self.dtype, device=self.device)
            self.queue._keep.append(t)
            return t
        return self.torch.empty(shape, dtype=self.dtype, device=self.device)

    def back(self, t):
        """Result to where the inputs live. Pinned host inputs get pinned host results (from
        torch's caching host allocator), so the copy back runs at full PCIe speed."""
        if t is None:
            return None
        if not self.host:
            return t
        if self.queue is not None:
            q = self.queue
            q.copy_out.wait_event(self.done)
            with self.torch.cuda.stream(q.copy_out):
                out = self.torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                out.copy_(t, non_blocking=True)
            return out.numpy() if self.numpy else out
        if self.pinned:
            out = self.torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            out.copy_(t, non_blocking=True)
            self.torch.cuda.current_stream(self.device).synchronize()
            return out
        t = t.cpu()
        return t.numpy() if self.numpy else t

    def run(self, name, tensors):
        """tensors: list of torch tensors, or ``(None, ndim)`` for a skipped gradient."""
        torch = self.torch
        structs = []
        for t in tensors:
            if isinstance(t, tuple):
                structs.append(_lib.null_struct(t[1]))
            else:
                structs.append(_lib.make_struct(t.data_ptr(), t.shape))
        lib = _lib.library()
        if self.queue is not None:
            q = self.queue
            for ready in self.ready:
                q.compute.wait_event(ready)
            with torch.cuda.device(self.device), torch.cuda.stream(q.compute):
                previous, waited = lib.mops_b200_get_stream(), lib.mops_b200_get_wait()
                lib.mops_b200_set_stream(q.compute.cuda_stream)
                lib.mops_b200_set_wait(0)
                try:
                    _lib.call(f"mops_cuda_{name}_{self.suffix}", structs)
                finally:
                    lib.mops_b200_set_stream(previous)
                    lib.mops_b200_set_wait(waited)
                self.done = torch.cuda.Event()
                self.done.record(q.compute)
            return
        with torch.cuda.device(self.device):
            previous = lib.mops_b200_get_stream()
            lib.mops_b200_set_stream(torch.cuda.current_stream().cuda_stream)
            try:
                _lib.call(f"mops_cuda_{name}_{self.suffix}", structs)
            finally:
                lib.mops_b200_set_stream(previous)


def _opt(arena, x, ndim):
    return (None, ndim) if x is None else arena.floats(x)


# ------------------------------------------------------------------------------------- HPE
def homogeneous_polynomial_evaluation(A, C, indices_A):
    op = "homogeneous_polynomial_evaluation"
    _check(A, 2, "f", op, "A"); _check(C, 1, "f", op, "C"); _check(indices_A, 2, "i", op, "indices_A")
    m = _Arena(A)
    A_, C_, P_ = m.floats(A), m.floats(C), m.ints(indices_A)
    out = m.empty((A_.shape[0],))
    m.run(op, [out, A_, C_, P_])
    return m.back(out)


def homogeneous_polynomial_evaluation_vjp(grad_output, A, C, indices_A, compute_grad_A=True):
    op = "homogeneous_polynomial_evaluation_vjp"
    _check(grad_output, 1, "f", op, "grad_output")
    _check(A, 2, "f", op, "A"); _check(C, 1, "f", op, "C"); _check(indices_A, 2, "i", op, "indices_A")
    m = _Arena(A)
    g_, A_, C_, P_ = m.floats(grad_output), m.floats(A), m.floats(C), m.ints(indices_A)
    grad_A = m.empty(A_.shape) if compute_grad_A else None
    m.run(op, [grad_A if compute_grad_A else (None, 2), g_, A_, C_, P_])
    return m.back(grad_A)


def homogeneous_polynomial_evaluation_vjp_vjp(grad_grad_A, grad_output, A, C, indices_A,
                                              compute_grad_grad_output=True,
                                              compute_grad_A_2=True):
    op = "homogeneous_polynomial_evaluation_vjp_vjp"
    _check(grad_output, 1, "f", op, "grad_output")
    _check(A, 2, "f", op, "A"); _check(C, 1, "f", op, "C"); _check(indices_A, 2, "i", op, "indices_A")
    m = _Arena(A)
    g_, A_, C_, P_ = m.floats(grad_output), m.floats(A), m.floats(C), m.ints(indices_A)
    ggO = m.empty(g_.shape) if compute_grad_grad_output else None
    gA2 = m.empty(A_.shape) if compute_grad_A_2 else None
    # C prototype order: (grad_grad_output, grad_A_2, grad_grad_A, ...), mops/include/mops/hpe.h:46-54
    m.run(op, [ggO if ggO is not None else (None, 1), gA2 if gA2 is not None else (None, 2),
               _opt(m, grad_grad_A, 2), g_, A_, C_, P_])
    return m.back(ggO), m.back(gA2)


# ------------------------------------------------------------------------------------- SAP
def _sap_common(op, A, B, C, indices_A, indices_B, indices_output):
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B"); _check(C, 1, "f", op, "C")
    _check(indices_A, 1, "i", op, "indices_A"); _check(indices_B, 1, "i", op, "indices_B")
    _check(indices_output, 1, "i", op, "indices_output")


def sparse_accumulation_of_products(A, B, C, indices_A, indices_B, indices_output, output_size):
    op = "sparse_accumulation_of_products"
    _sap_common(op, A, B, C, indices_A, indices_B, indices_output)
    _check_scalar(output_size, op, "output_size")
    m = _Arena(A)
    A_, B_, C_ = m.floats(A), m.floats(B), m.floats(C)
    out = m.empty((A_.shape[0], output_size))
    m.run(op, [out, A_, B_, C_, m.ints(indices_A), m.ints(indices_B), m.ints(indices_output)])
    return m.back(out)


def sparse_accumulation_of_products_vjp(grad_output, A, B, C, indices_A, indices_B,
                                        indices_output, compute_grad_A=True, compute_grad_B=True):
    op = "sparse_accumulation_of_products_vjp"
    _check(grad_output, 2, "f", op, "grad_output")
    _sap_common(op, A, B, C, indices_A, indices_B, indices_output)
    m = _Arena(A)
    g_, A_, B_, C_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(C)
    gA = m.empty(A_.shape) if compute_grad_A else None
    gB = m.empty(B_.shape) if compute_grad_B else None
    m.run(op, [gA if gA is not None else (None, 2), gB if gB is not None else (None, 2), g_, A_,
               B_, C_, m.ints(indices_A), m.ints(indices_B), m.ints(indices_output)])
    return m.back(gA), m.back(gB)


def sparse_accumulation_of_products_vjp_vjp(grad_grad_A, grad_grad_B, grad_output, A, B, C,
                                            indices_A, indices_B, indices_output,
                                            compute_grad_grad_output=True, compute_grad_A_2=True,
                                            compute_grad_B_2=True):
    op = "sparse_accumulation_of_products_vjp_vjp"
    _check(grad_output, 2, "f", op, "grad_output")
    _sap_common(op, A, B, C, indices_A, indices_B, indices_output)
    m = _Arena(A)
    g_, A_, B_, C_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(C)
    ggO = m.empty(g_.shape) if compute_grad_grad_output else None
    gA2 = m.empty(A_.shape) if compute_grad_A_2 else None
    gB2 = m.empty(B_.shape) if compute_grad_B_2 else None
    m.run(op, [ggO if ggO is not None else (None, 2), gA2 if gA2 is not None else (None, 2),
               gB2 if gB2 is not None else (None, 2), _opt(m, grad_grad_A, 2),
               _opt(m, grad_grad_B, 2), g_, A_, B_, C_, m.ints(indices_A), m.ints(indices_B),
               m.ints(indices_output)])
    return m.back(ggO), m.back(gA2), m.back(gB2)


# ------------------------------------------------------------------------------------ OPSA
def outer_product_scatter_add(A, B, indices_output, output_size):
    op = "outer_product_scatter_add"
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B")
    _check(indices_output, 1, "i", op, "indices_output")
    _check_scalar(output_size, op, "output_size")
    m = _Arena(A)
    A_, B_ = m.floats(A), m.floats(B)
    out = m.empty((output_size, A_.shape[1], B_.shape[1]))
    m.run(op, [out, A_, B_, m.ints(indices_output)])
    return m.back(out)


def outer_product_scatter_add_vjp(grad_output, A, B, indices_output, compute_grad_A=True,
                                  compute_grad_B=True):
    op = "outer_product_scatter_add_vjp"
    _check(grad_output, 3, "f", op, "grad_output")
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B")
    _check(indices_output, 1, "i", op, "indices_output")
    m = _Arena(A)
    g_, A_, B_ = m.floats(grad_output), m.floats(A), m.floats(B)
    gA = m.empty(A_.shape) if compute_grad_A else None
    gB = m.empty(B_.shape) if compute_grad_B else None
    m.run(op, [gA if gA is not None else (None, 2), gB if gB is not None else (None, 2), g_, A_,
               B_, m.ints(indices_output)])
    return m.back(gA), m.back(gB)


def outer_product_scatter_add_vjp_vjp(grad_grad_A, grad_grad_B, grad_output, A, B, indices_output,
                                      compute_grad_grad_output=True, compute_grad_A_2=True,
                                      compute_grad_B_2=True):
    op = "outer_product_scatter_add_vjp_vjp"
    _check(grad_output, 3, "f", op, "grad_output")
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B")
    _check(indices_output, 1, "i", op, "indices_output")
    m = _Arena(A)
    g_, A_, B_ = m.floats(grad_output), m.floats(A), m.floats(B)
    ggO = m.empty(g_.shape) if compute_grad_grad_output else None
    gA2 = m.empty(A_.shape) if compute_grad_A_2 else None
    gB2 = m.empty(B_.shape) if compute_grad_B_2 else None
    m.run(op, [ggO if ggO is not None else (None, 3), gA2 if gA2 is not None else (None, 2),
               gB2 if gB2 is not None else (None, 2), _opt(m, grad_grad_A, 2),
               _opt(m, grad_grad_B, 2), g_, A_, B_, m.ints(indices_output)])
    return m.back(ggO), m.back(gA2), m.back(gB2)


# ----------------------------------------------------------------------------------- OPSAW
def outer_product_scatter_add_with_weights(A, B, W, indices_W, indices_output):
    op = "outer_product_scatter_add_with_weights"
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B"); _check(W, 2, "f", op, "W")
    _check(indices_W, 1, "i", op, "indices_W"); _check(indices_output, 1, "i", op, "indices_output")
    m = _Arena(A)
    A_, B_, W_ = m.floats(A), m.floats(B), m.floats(W)
    out = m.empty((W_.shape[0], A_.shape[1], B_.shape[1]))
    m.run(op, [out, A_, B_, W_, m.ints(indices_W), m.ints(indices_output)])
    return m.back(out)


def outer_product_scatter_add_with_weights_vjp(grad_output, A, B, W, indices_W, indices_output,
                                               compute_grad_A=True, compute_grad_B=True,
                                               compute_grad_W=True):
    op = "outer_product_scatter_add_with_weights_vjp"
    _check(grad_output, 3, "f", op, "grad_output")
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B"); _check(W, 2, "f", op, "W")
    _check(indices_W, 1, "i", op, "indices_W"); _check(indices_output, 1, "i", op, "indices_output")
    m = _Arena(A)
    g_, A_, B_, W_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(W)
    gA = m.empty(A_.shape) if compute_grad_A else None
    gB = m.empty(B_.shape) if compute_grad_B else None
    gW = m.empty(W_.shape) if compute_grad_W else None
    m.run(op, [gA if gA is not None else (None, 2), gB if gB is not None else (None, 2),
               gW if gW is not None else (None, 2), g_, A_, B_, W_, m.ints(indices_W),
               m.ints(indices_output)])
    return m.back(gA), m.back(gB), m.back(gW)


def outer_product_scatter_add_with_weights_vjp_vjp(grad_grad_A, grad_grad_B, grad_grad_W,
                                                   grad_output, A, B, W, indices_W,
                                                   indices_output, compute_grad_grad_output=True,
                                                   compute_grad_A_2=True, compute_grad_B_2=True,
                                                   compute_grad_W_2=True):
    op = "outer_product_scatter_add_with_weights_vjp_vjp"
    m = _Arena(A)
    g_, A_, B_, W_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(W)
    m.run(op, [(None, 3), (None, 2), (None, 2), (None, 2), _opt(m, grad_grad_A, 2),
               _opt(m, grad_grad_B, 2), _opt(m, grad_grad_W, 2), g_, A_, B_, W_,
               m.ints(indices_W), m.ints(indices_output)])


# ----------------------------------------------------------------------------------- SASAW
def _sasaw_common(op, A, B, C, W, indices_A, indices_W_1, indices_W_2, indices_output_1,
                  indices_output_2):
    _check(A, 2, "f", op, "A"); _check(B, 2, "f", op, "B"); _check(C, 1, "f", op, "C")
    _check(W, 3, "f", op, "W")
    for name, idx in (("indices_A", indices_A), ("indices_W_1", indices_W_1),
                      ("indices_W_2", indices_W_2), ("indices_output_1", indices_output_1),
                      ("indices_output_2", indices_output_2)):
        _check(idx, 1, "i", op, name)


def sparse_accumulation_scatter_add_with_weights(A, B, C, W, indices_A, indices_W_1, indices_W_2,
                                                 indices_output_1, indices_output_2, output_size):
    op = "sparse_accumulation_scatter_add_with_weights"
    _sasaw_common(op, A, B, C, W, indices_A, indices_W_1, indices_W_2, indices_output_1,
                  indices_output_2)
    _check_scalar(output_size, op, "output_size")
    m = _Arena(A)
    A_, B_, C_, W_ = m.floats(A), m.floats(B), m.floats(C), m.floats(W)
    out = m.empty((W_.shape[0], output_size, B_.shape[1]))
    m.run(op, [out, A_, B_, C_, W_, m.ints(indices_A), m.ints(indices_W_1), m.ints(indices_W_2),
               m.ints(indices_output_1), m.ints(indices_output_2)])
    return m.back(out)


def sparse_accumulation_scatter_add_with_weights_vjp(grad_output, A, B, C, W, indices_A,
                                                     indices_W_1, indices_W_2, indices_output_1,
                                                     indices_output_2, compute_grad_A=True,
                                                     compute_grad_B=True, compute_grad_W=True):
    op = "sparse_accumulation_scatter_add_with_weights_vjp"
    _check(grad_output, 3, "f", op, "grad_output")
    _sasaw_common(op, A, B, C, W, indices_A, indices_W_1, indices_W_2, indices_output_1,
                  indices_output_2)
    m = _Arena(A)
    g_, A_, B_, C_, W_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(C), m.floats(W)
    gA = m.empty(A_.shape) if compute_grad_A else None
    gB = m.empty(B_.shape) if compute_grad_B else None
    gW = m.empty(W_.shape) if compute_grad_W else None
    m.run(op, [gA if gA is not None else (None, 2), gB if gB is not None else (None, 2),
               gW if gW is not None else (None, 3), g_, A_, B_, C_, W_, m.ints(indices_A),
               m.ints(indices_W_1), m.ints(indices_W_2), m.ints(indices_output_1),
               m.ints(indices_output_2)])
    return m.back(gA), m.back(gB), m.back(gW)


def sparse_accumulation_scatter_add_with_weights_vjp_vjp(grad_grad_A, grad_grad_B, grad_grad_W,
                                                         grad_output, A, B, C, W, indices_A,
                                                         indices_W_1, indices_W_2,
                                                         indices_output_1, indices_output_2,
                                                         compute_grad_grad_output=True,
                                                         compute_grad_A_2=True,
                                                         compute_grad_B_2=True,
                                                         compute_grad_W_2=True):
    op = "sparse_accumulation_scatter_add_with_weights_vjp_vjp"
    m = _Arena(A)
    g_, A_, B_, C_, W_ = m.floats(grad_output), m.floats(A), m.floats(B), m.floats(C), m.floats(W)
    # grad_grad_W is 2-D in the C prototype (mops/include/mops/sasaw.h:84)
    m.run(op, [(None, 3), (None, 2), (None, 2), (None, 3), _opt(m, grad_grad_A, 2),
               _opt(m, grad_grad_B, 2), (None, 2), g_, A_, B_, C_, W_, m.ints(indices_A),
               m.ints(indices_W_1), m.ints(indices_W_2), m.ints(indices_output_1),
               m.ints(indices_output_2)])
