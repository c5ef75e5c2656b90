"""Helpers shared by the MoE layers."""
import sys
from typing import Union

import torch


class DisposibleTensor:
    """Owner handle for a large buffer that should be given back before its Python name goes out of scope.

    Public contract of `dlblas.utils.utils.DisposibleTensor` (dlblas/utils/utils.py:173-235 of the reference), which
    the low-latency layer relies on for the dispatch buffers: `.value` is the tensor while it is held;
    `.dispose()` lets go of it and insists that this handle was the last owner (otherwise the memory would not
    actually return to the allocator); `.shape`, `.device` and `.dtype` stay readable afterwards unless the
    caller opted out; the two `maybe_*` helpers accept plain tensors as well."""

    __slots__ = ("_held", "_facts")
    _KEPT_FACTS = ("shape", "device", "dtype")

    def __init__(self, value: torch.Tensor):
        self._held = value
        self._facts = None

    @property
    def is_disposed(self) -> bool:
        return self._held is None

    @property
    def value(self) -> torch.Tensor:
        assert self._held is not None, "the tensor was disposed"
        return self._held

    def dispose(self, backup_metadata: bool = True):
        assert self._held is not None, "the tensor was disposed already"
        if not torch.compiler.is_compiling():
            # one reference from this handle and one from the argument of getrefcount itself
            owners = sys.getrefcount(self._held)
            assert owners == 2, f"refcount={owners}"
        self._facts = {name: getattr(self._held, name) for name in self._KEPT_FACTS} if backup_metadata else None
        self._held = None

    def __getattr__(self, name):
        # only reached for names that are not slots: the tensor facts that outlive the tensor
        if name in DisposibleTensor._KEPT_FACTS:
            if self._held is not None:
                return getattr(self._held, name)
            assert self._facts is not None, "Use backup_metadata flag if you want to use metadata after dispose"
            return self._facts[name]
        raise AttributeError(name)

    @staticmethod
    def maybe_unwrap(value: "MaybeDisposibleTensor") -> torch.Tensor:
        return value.value if isinstance(value, DisposibleTensor) else value

    @staticmethod
    def maybe_dispose(value: "MaybeDisposibleTensor") -> None:
        if isinstance(value, DisposibleTensor):
            value.dispose()


MaybeDisposibleTensor = Union[torch.Tensor, DisposibleTensor]
