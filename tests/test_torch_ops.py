"""The torch operators (torch.ops.mops.*): registration and argument checks on CPU; on the
GPU, forward parity with the CPU oracle, finite-difference gradient checks in f64 (the VJP
checked against the forward, independent of any reference VJP; the reference does the same
in python/mops-torch/tests/*.py), second derivatives for HPE, SAP and OPSA, and a TorchScript round trip."""
import io

import numpy as np
import pytest
import torch

import fixtures
from conftest import assert_parity

import mops_b200.torch as mt


def _t(x, device="cuda", grad=False):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(device)
    return t.requires_grad_(True) if grad else t


def test_operators_are_registered_with_the_reference_schemas():
    schemas = {
        "homogeneous_polynomial_evaluation":
            "mops::homogeneous_polynomial_evaluation(Tensor A, Tensor C, Tensor indices_A) -> Tensor",
        "outer_product_scatter_add":
            "mops::outer_product_scatter_add(Tensor A, Tensor B, Tensor indices_output, "
            "int output_size) -> Tensor",
        "sparse_accumulation_of_products":
            "mops::sparse_accumulation_of_products(Tensor A, Tensor B, Tensor C, Tensor indices_A, "
            "Tensor indices_B, Tensor indices_output, int output_size) -> Tensor",
        "outer_product_scatter_add_with_weights":
            "mops::outer_product_scatter_add_with_weights(Tensor A, Tensor B, Tensor W, "
            "Tensor indices_W, Tensor indices_output) -> Tensor",
        "sparse_accumulation_scatter_add_with_weights":
            "mops::sparse_accumulation_scatter_add_with_weights(Tensor A, Tensor B, Tensor C, "
            "Tensor W, Tensor indices_A, Tensor indices_W_1, Tensor indices_W_2, "
            "Tensor indices_output_1, Tensor indices_output_2, int output_size) -> Tensor",
    }
    for name, schema in schemas.items():
        op = getattr(torch.ops.mops, name)
        assert str(op.default._schema) == schema


def test_argument_checks_and_cpu_rejection():
    A, B = torch.zeros(5, 3, dtype=torch.float64), torch.zeros(5, 2, dtype=torch.float64)
    idx = torch.zeros(5, dtype=torch.int32)
    with pytest.raises(ValueError, match="is not implemented for device cpu"):
        mt.outer_product_scatter_add(A, B, idx, 4)
    with pytest.raises(TypeError, match="All index tensors must be of type int32"):
        mt.outer_product_scatter_add(A, B, idx.long(), 4)
    with pytest.raises(TypeError, match="All floating point tensors must be of the same dtype"):
        mt.outer_product_scatter_add(A, B.float(), idx, 4)
    with pytest.raises(ValueError, match="Expected A to have 2 dimensions"):
        mt.outer_product_scatter_add(A[0], B, idx, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_forward_matches_oracle(oracle, dtype):
    c = lambda x: np.ascontiguousarray(x, dtype=dtype)
    d = fixtures.hpe()
    out = mt.homogeneous_polynomial_evaluation(_t(c(d["A"])), _t(c(d["C"])), _t(d["indices_A"]))
    assert_parity(out.cpu().numpy(), oracle.hpe(c(d["A"]), c(d["C"]), d["indices_A"]), "hpe")
    d = fixtures.sap()
    out = mt.sparse_accumulation_of_products(
        _t(c(d["A"])), _t(c(d["B"])), _t(c(d["C"])), _t(d["indices_A"]), _t(d["indices_B"]),
        _t(d["indices_output"]), d["output_size"])
    assert_parity(out.cpu().numpy(), oracle.sap(c(d["A"]), c(d["B"]), c(d["C"]), d["indices_A"],
                                                d["indices_B"], d["indices_output"], 35), "sap")
    d = fixtures.opsa(True)
    out = mt.outer_product_scatter_add(_t(c(d["A"])), _t(c(d["B"])), _t(d["indices_output"]), 10)
    assert_parity(out.cpu().numpy(), oracle.opsa(c(d["A"]), c(d["B"]), d["indices_output"], 10), "opsa")
    d = fixtures.opsaw()
    out = mt.outer_product_scatter_add_with_weights(
        _t(c(d["A"])), _t(c(d["B"])), _t(c(d["W"])), _t(d["indices_W"]), _t(d["indices_output"]))
    assert_parity(out.cpu().numpy(), oracle.opsaw(c(d["A"]), c(d["B"]), c(d["W"]), d["indices_W"],
                                                  d["indices_output"]), "opsaw")
    d = fixtures.sasaw()
    idx = [d[k] for k in ("indices_A", "indices_W_1", "indices_W_2", "indices_output_1",
                          "indices_output_2")]
    out = mt.sparse_accumulation_scatter_add_with_weights(
        _t(c(d["A"])), _t(c(d["B"])), _t(c(d["C"])), _t(c(d["W"])), *[_t(i) for i in idx], 15)
    assert_parity(out.cpu().numpy(),
                  oracle.sasaw(c(d["A"]), c(d["B"]), c(d["C"]), c(d["W"]), *idx, 15), "sasaw")


@pytest.mark.gpu
def test_gradcheck_all_operations():
    g = torch.Generator().manual_seed(0xDEADBEEF)
    rand = lambda *s: torch.rand(*s, dtype=torch.float64, generator=g).cuda().requires_grad_(True)
    ri = lambda n, *s: torch.randint(n, s, dtype=torch.int32, generator=g).cuda()

    A, C, P = rand(30, 8), torch.rand(40, dtype=torch.float64, generator=g).cuda(), ri(8, 40, 3)
    assert torch.autograd.gradcheck(mt.homogeneous_polynomial_evaluation, (A, C, P), fast_mode=True)
    assert torch.autograd.gradgradcheck(mt.homogeneous_polynomial_evaluation, (A, C, P),
                                        fast_mode=True)

    A, B = rand(20, 7), rand(20, 5)
    Csap = torch.rand(30, dtype=torch.float64, generator=g).cuda()
    args = (A, B, Csap, ri(7, 30), ri(5, 30), ri(9, 30), 9)
    assert torch.autograd.gradcheck(mt.sparse_accumulation_of_products, args, fast_mode=True)
    assert torch.autograd.gradgradcheck(mt.sparse_accumulation_of_products, args, fast_mode=True)

    A, B = rand(60, 6), rand(60, 5)
    idx = torch.sort(ri(10, 60)).values
    idx[idx == 1] = 2  # an empty output row, as in python/mops-torch/tests/opsa.py:28-32
    assert torch.autograd.gradcheck(mt.outer_product_scatter_add, (A, B, idx, 10), fast_mode=True)
    assert torch.autograd.gradgradcheck(mt.outer_product_scatter_add, (A, B, idx, 10),
                                        fast_mode=True)

    A, B, W = rand(60, 6), rand(60, 5), rand(10, 5)
    # unsorted indices, as in python/mops-torch/tests/opsaw.py:45-47
    # grad_W is accumulated with atomics (indices_W is unsorted), so repeated backward
    # passes may differ in the last bits
    assert torch.autograd.gradcheck(mt.outer_product_scatter_add_with_weights,
                                    (A, B, W, ri(10, 60), ri(10, 60)), fast_mode=True,
                                    nondet_tol=1e-12)

    A, B, W = rand(40, 5), rand(40, 6), rand(8, 4, 6)
    Cs = torch.rand(25, dtype=torch.float64, generator=g).cuda()
    args = (A, B, Cs, W, ri(5, 25), ri(8, 40), ri(4, 25), ri(8, 40), ri(3, 25), 3)
    assert torch.autograd.gradcheck(mt.sparse_accumulation_scatter_add_with_weights, args,
                                    fast_mode=True, nondet_tol=1e-12)


@pytest.mark.gpu
def test_second_derivatives_without_a_kernel_raise():
    A = torch.rand(20, 6, dtype=torch.float64, device="cuda", requires_grad=True)
    B = torch.rand(20, 5, dtype=torch.float64, device="cuda", requires_grad=True)
    W = torch.rand(4, 5, dtype=torch.float64, device="cuda", requires_grad=True)
    idx = torch.sort(torch.randint(4, (20,), dtype=torch.int32, device="cuda")).values
    out = mt.outer_product_scatter_add_with_weights(A, B, W, idx, idx)
    (gA,) = torch.autograd.grad(out.sum(), A, create_graph=True)
    with pytest.raises(NotImplementedError, match="second derivatives are not supported"):
        gA.sum().backward()


@pytest.mark.gpu
def test_torchscript_round_trip():
    class M(torch.nn.Module):
        def forward(self, A: torch.Tensor, B: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
            return torch.ops.mops.outer_product_scatter_add(A, B, idx, 7)

    A = torch.rand(50, 4, dtype=torch.float64, device="cuda", requires_grad=True)
    B = torch.rand(50, 3, dtype=torch.float64, device="cuda")
    idx = torch.sort(torch.randint(7, (50,), dtype=torch.int32, device="cuda")).values
    eager = M()(A, B, idx)
    scripted = torch.jit.script(M())
    buf = io.BytesIO()
    torch.jit.save(scripted, buf)
    buf.seek(0)
    loaded = torch.jit.load(buf)
    out = loaded(A, B, idx)
    assert torch.equal(out, eager)
    (g1,) = torch.autograd.grad(out.sum(), A)
    (g2,) = torch.autograd.grad(M()(A, B, idx).sum(), A)
    assert torch.equal(g1, g2)


@pytest.mark.gpu
def test_runs_on_the_current_stream_and_device():
    side = torch.cuda.Stream()
    A = torch.rand(5000, 6, dtype=torch.float64, device="cuda")
    B = torch.rand(5000, 5, dtype=torch.float64, device="cuda")
    idx = torch.sort(torch.randint(100, (5000,), dtype=torch.int32, device="cuda")).values
    ref = mt.outer_product_scatter_add(A, B, idx, 100)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        out = mt.outer_product_scatter_add(A, B, idx, 100)
    side.synchronize()
    assert torch.equal(out, ref)
