"""The allocation-free SASAW forward entry point, for callers that cannot allocate device
memory at the time they call (a host program whose own pool has reserved the whole device, so
that a library's cudaMalloc fails or fragments it; latency-critical loops, where a driver
allocation may block): called through the C ABI and compared with the CPU oracle and with
the regular entry point.

This file sorts last on purpose, so that a run which stops at the first failure has already
been through every other test."""
import numpy as np
import pytest

from conftest import assert_parity
from helpers import run_checker
from mops_b200 import _lib, workloads

NOALLOC = "mops_b200_cuda_sparse_accumulation_scatter_add_with_weights_noalloc_f64"
REGULAR = "mops_cuda_sparse_accumulation_scatter_add_with_weights_f64"
ORDER = ("A", "B", "C", "W", "indices_A", "indices_W_1", "indices_W_2", "indices_output_1",
         "indices_output_2")


def _structs(out, t):
    return [_lib.make_struct(out.data_ptr(), out.shape)] + \
        [_lib.make_struct(t[k].data_ptr(), t[k].shape) for k in ORDER]


@pytest.mark.gpu
def test_noalloc_matches_oracle_and_regular_entry_point_on_consecutive_calls(oracle):
    """Two calls in a row on different problems (the second smaller, so stale contents of the
    shared scratch array would show), then an unsorted one; each against the CPU oracle and
    against the regular entry point, within the f64 parity tolerance."""
    import torch
    from helpers import to_dev
    cases = [workloads.sasaw(E=4000, n=64, N=500),
             workloads.sasaw(E=900, n=31, N=37, nA=4, L=33, nW2=3, nO2=5, seed=77)]
    unsorted = workloads.sasaw(E=700, n=20, N=120, seed=78)
    unsorted["indices_output_1"] = np.random.default_rng(1).permutation(unsorted["indices_output_1"])
    cases.append(unsorted)
    expected = [run_checker(oracle, "sasaw", d, np.float64)["output"] for d in cases]
    for round_ in range(2):
        for d, want_cpu in zip(cases, expected):
            t = to_dev(d, np.float64)
            shape = (t["W"].shape[0], d["output_size"], t["B"].shape[1])
            want = torch.full(shape, float("nan"), dtype=torch.float64, device="cuda")
            got = torch.full(shape, float("nan"), dtype=torch.float64, device="cuda")
            _lib.call(REGULAR, _structs(want, t))
            _lib.call(NOALLOC, _structs(got, t))
            assert_parity(got.cpu().numpy(), want_cpu, f"noalloc vs oracle, round {round_}")
            assert_parity(got.cpu().numpy(), want.cpu().numpy(), f"noalloc vs regular, round {round_}")


@pytest.mark.gpu
def test_noalloc_leaves_device_memory_untouched():
    """The property the entry point exists for: after a warm-up call (which may make the
    driver load kernel code), further calls change neither the free device memory nor
    torch's own reservations, whereas the table of the regular entry point comes from a
    memory pool."""
    import torch
    from helpers import to_dev
    d = workloads.sasaw(E=3000, n=50, N=400)
    t = to_dev(d, np.float64)
    out = torch.empty((50, 9, 32), dtype=torch.float64, device="cuda")
    structs = _structs(out, t)
    _lib.call(NOALLOC, structs)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        _lib.call(NOALLOC, structs)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before


@pytest.mark.gpu
def test_noalloc_reports_bad_indices():
    from helpers import to_dev
    import torch
    d = workloads.sasaw(E=500, n=16, N=50)
    d["indices_W_2"][3] = 9
    t = to_dev(d, np.float64)
    out = torch.empty((16, 9, 32), dtype=torch.float64, device="cuda")
    with pytest.raises(_lib.MopsError, match="Index array indices_W_2"):
        _lib.call(NOALLOC, _structs(out, t))


def test_noalloc_handles_an_empty_cell_grid_on_the_host():
    """W.shape[1] == 0 with a non-empty coupling table means every indices_W_2 entry is out of
    range: reported before any CUDA call (fake pointers, runs without a GPU), like the regular
    entry point reports it."""
    fake = lambda shape: _lib.make_struct(0x1000, shape)
    E, n, N = 10, 4, 7
    with pytest.raises(_lib.MopsError, match="Index array indices_W_2"):
        _lib.call(NOALLOC, [fake((n, 9, 32)), fake((E, 9)), fake((E, 32)), fake((N,)),
                            fake((n, 0, 32)), fake((N,)), fake((E,)), fake((N,)), fake((E,)),
                            fake((N,))])


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    """Checked on the host before any CUDA call: runs without a GPU."""
    fake = lambda shape: _lib.make_struct(0x1000, shape)
    E, n, N = 10, 4, 5000
    with pytest.raises(_lib.MopsError, match="at most 4096 coupling entries and 1024"):
        _lib.call(NOALLOC, [fake((n, 9, 32)), fake((E, 9)), fake((E, 32)), fake((N,)),
                            fake((n, 9, 32)), fake((N,)), fake((E,)), fake((N,)), fake((E,)),
                            fake((N,))])
    with pytest.raises(_lib.MopsError, match="at most 4096 coupling entries and 1024"):
        _lib.call(NOALLOC, [fake((n, 40, 32)), fake((E, 9)), fake((E, 32)), fake((7,)),
                            fake((n, 40, 32)), fake((7,)), fake((E,)), fake((7,)), fake((E,)),
                            fake((7,))])
