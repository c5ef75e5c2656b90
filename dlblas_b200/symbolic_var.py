"""Symbolic shapes used when an operator is registered (dlblas/symbolic_var.py:134-177 of the
reference): a named dimension and a tensor placeholder that only carries shape symbols,
a device prefix and a dtype."""
import torch


class SymVar:
    def __init__(self, name):
        assert isinstance(name, str)
        self.name = name

    def __eq__(self, value) -> bool:
        return isinstance(value, SymVar) and self.name == value.name

    def __hash__(self) -> int:
        return hash(self.name)

    def __repr__(self):
        return f"SymVar({self.name!r})"


class Tensor:
    """Placeholder for a tensor argument at registration time; nothing is allocated."""

    def __init__(self, shape, *, device: str, dtype: torch.dtype):
        for arg in shape:
            assert isinstance(arg, SymVar), f"expect a SymVar, but got {arg}"
        self._shape, self._device, self._dtype = tuple(shape), device, dtype

    shape = property(lambda self: self._shape)
    device = property(lambda self: self._device)
    dtype = property(lambda self: self._dtype)
