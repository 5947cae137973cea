"""Shared by the GPU parity tests: runs every level of an op through the library under test
(``mops_b200``, i.e. through the C ABI) and through a CPU checker with the same call shape."""
import numpy as np


def to_dev(d, dtype, device="cuda"):
    import torch
    out = {}
    for k, v in d.items():
        if isinstance(v, np.ndarray):
            if np.issubdtype(v.dtype, np.floating):
                v = v.astype(dtype)
            out[k] = torch.from_numpy(np.ascontiguousarray(v)).to(device)
        else:
            out[k] = v
    return out


def host(x):
    return None if x is None else x.cpu().numpy()


def run_library(op, d, second_order=False, to_host=True):
    """All levels of ``op`` on a dict of CUDA tensors -> {name: numpy array} (or the CUDA
    tensors themselves with ``to_host=False``)."""
    import mops_b200 as M
    out = {}
    if op == "hpe":
        out["output"] = M.homogeneous_polynomial_evaluation(d["A"], d["C"], d["indices_A"])
        out["grad_A"] = M.homogeneous_polynomial_evaluation_vjp(
            d["grad_output"], d["A"], d["C"], d["indices_A"])
        if second_order:
            out["grad_grad_output"], out["grad_A_2"] = M.homogeneous_polynomial_evaluation_vjp_vjp(
                d["grad_grad_A"], d["grad_output"], d["A"], d["C"], d["indices_A"])
    elif op == "sap":
        idx = (d["indices_A"], d["indices_B"], d["indices_output"])
        out["output"] = M.sparse_accumulation_of_products(d["A"], d["B"], d["C"], *idx,
                                                         d["output_size"])
        out["grad_A"], out["grad_B"] = M.sparse_accumulation_of_products_vjp(
            d["grad_output"], d["A"], d["B"], d["C"], *idx)
        if second_order:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = \
                M.sparse_accumulation_of_products_vjp_vjp(
                    d["grad_grad_A"], d["grad_grad_B"], d["grad_output"], d["A"], d["B"], d["C"],
                    *idx)
    elif op == "opsa":
        out["output"] = M.outer_product_scatter_add(d["A"], d["B"], d["indices_output"],
                                                   d["output_size"])
        out["grad_A"], out["grad_B"] = M.outer_product_scatter_add_vjp(
            d["grad_output"], d["A"], d["B"], d["indices_output"])
        if second_order:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = \
                M.outer_product_scatter_add_vjp_vjp(
                    d["grad_grad_A"], d["grad_grad_B"], d["grad_output"], d["A"], d["B"],
                    d["indices_output"])
    elif op == "opsaw":
        idx = (d["indices_W"], d["indices_output"])
        out["output"] = M.outer_product_scatter_add_with_weights(d["A"], d["B"], d["W"], *idx)
        out["grad_A"], out["grad_B"], out["grad_W"] = \
            M.outer_product_scatter_add_with_weights_vjp(d["grad_output"], d["A"], d["B"], d["W"],
                                                         *idx)
    elif op == "sasaw":
        idx = (d["indices_A"], d["indices_W_1"], d["indices_W_2"], d["indices_output_1"],
               d["indices_output_2"])
        out["output"] = M.sparse_accumulation_scatter_add_with_weights(
            d["A"], d["B"], d["C"], d["W"], *idx, d["output_size"])
        out["grad_A"], out["grad_B"], out["grad_W"] = \
            M.sparse_accumulation_scatter_add_with_weights_vjp(
                d["grad_output"], d["A"], d["B"], d["C"], d["W"], *idx)
    else:
        raise KeyError(op)
    return {k: host(v) for k, v in out.items()} if to_host else out


def run_checker(impl, op, d, dtype, second_order=False):
    """Same, through an oracle/reference object of oracle.mops_oracle."""
    c = lambda x: np.ascontiguousarray(x, dtype=dtype)
    out = {}
    if op == "hpe":
        out["output"] = impl.hpe(c(d["A"]), c(d["C"]), d["indices_A"])
        out["grad_A"] = impl.hpe_vjp(c(d["grad_output"]), c(d["A"]), c(d["C"]), d["indices_A"])
        if second_order:
            out["grad_grad_output"], out["grad_A_2"] = impl.hpe_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_output"]), c(d["A"]), c(d["C"]), d["indices_A"])
    elif op == "sap":
        idx = (d["indices_A"], d["indices_B"], d["indices_output"])
        out["output"] = impl.sap(c(d["A"]), c(d["B"]), c(d["C"]), *idx, d["output_size"])
        out["grad_A"], out["grad_B"] = impl.sap_vjp(c(d["grad_output"]), c(d["A"]), c(d["B"]),
                                                    c(d["C"]), *idx)
        if second_order:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = impl.sap_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_grad_B"]), c(d["grad_output"]), c(d["A"]),
                c(d["B"]), c(d["C"]), *idx)
    elif op == "opsa":
        out["output"] = impl.opsa(c(d["A"]), c(d["B"]), d["indices_output"], d["output_size"])
        out["grad_A"], out["grad_B"] = impl.opsa_vjp(c(d["grad_output"]), c(d["A"]), c(d["B"]),
                                                     d["indices_output"])
        if second_order:
            out["grad_grad_output"], out["grad_A_2"], out["grad_B_2"] = impl.opsa_vjp_vjp(
                c(d["grad_grad_A"]), c(d["grad_grad_B"]), c(d["grad_output"]), c(d["A"]),
                c(d["B"]), d["indices_output"])
    elif op == "opsaw":
        idx = (d["indices_W"], d["indices_output"])
        out["output"] = impl.opsaw(c(d["A"]), c(d["B"]), c(d["W"]), *idx)
        out["grad_A"], out["grad_B"], out["grad_W"] = impl.opsaw_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), c(d["W"]), *idx)
    elif op == "sasaw":
        idx = (d["indices_A"], d["indices_W_1"], d["indices_W_2"], d["indices_output_1"],
               d["indices_output_2"])
        out["output"] = impl.sasaw(c(d["A"]), c(d["B"]), c(d["C"]), c(d["W"]), *idx,
                                   d["output_size"])
        out["grad_A"], out["grad_B"], out["grad_W"] = impl.sasaw_vjp(
            c(d["grad_output"]), c(d["A"]), c(d["B"]), c(d["C"]), c(d["W"]), *idx)
    else:
        raise KeyError(op)
    return out
