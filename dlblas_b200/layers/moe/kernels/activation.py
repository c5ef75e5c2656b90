"""`dlblas.layers.moe.kernels.activation.silu_and_mul`
(dlblas/layers/moe/kernels/activation.py:61-95 of the reference)."""
from ....kernels.activation import silu_and_mul  # noqa: F401
