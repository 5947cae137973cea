"""``torch.ops.mops.*`` backed by the sm_100a kernels.

Mirrors python/mops-torch/src/mops/torch/__init__.py of the reference: importing this module
loads the operator library, after which the five operations are available both as
``torch.ops.mops.<name>`` and as attributes of this module, differentiable through autograd
and usable from TorchScript. CUDA tensors only.
"""
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libmops_torch.so")

if not os.path.isfile(LIB_PATH):
    raise ImportError(f"{LIB_PATH} not found: build it with `python -m mops_b200.build`")
torch.ops.load_library(LIB_PATH)

homogeneous_polynomial_evaluation = torch.ops.mops.homogeneous_polynomial_evaluation
sparse_accumulation_of_products = torch.ops.mops.sparse_accumulation_of_products
outer_product_scatter_add = torch.ops.mops.outer_product_scatter_add
outer_product_scatter_add_with_weights = torch.ops.mops.outer_product_scatter_add_with_weights
sparse_accumulation_scatter_add_with_weights = (
    torch.ops.mops.sparse_accumulation_scatter_add_with_weights
)

__all__ = [
    "homogeneous_polynomial_evaluation",
    "sparse_accumulation_of_products",
    "outer_product_scatter_add",
    "outer_product_scatter_add_with_weights",
    "sparse_accumulation_scatter_add_with_weights",
]
