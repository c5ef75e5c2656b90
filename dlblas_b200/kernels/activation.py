"""`dlblas.kernels.activation.silu_and_mul` (dlblas/kernels/activation.py:89-131 of the reference)."""
import torch

from .. import ops


def silu_and_mul(gate_up: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """out = silu(gate_up[:, :N]) * gate_up[:, N:], computed in fp32, stored in the input dtype."""
    assert gate_up.dim() == 2
    return ops.silu_and_mul(gate_up, out)
