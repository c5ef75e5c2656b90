"""Operators of the FP8 MoE expert path under the reference's module names
(`dlblas.kernels.*`).  Importing this package registers `topk_gating` with the op registry."""
from . import topk_gating  # noqa: F401  (registration side effect, as in dlblas/kernels/__init__.py)
