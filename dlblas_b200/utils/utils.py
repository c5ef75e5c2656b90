"""Helpers shared by the MoE layers."""
import sys
from typing import Any, Dict, Optional, Union

import torch


class DisposibleTensor:
    """Wrapper that lets the owner free a large buffer early (dlblas/utils/utils.py:173-235 of
    the reference): `dispose()` drops the only reference (checked through the refcount) and keeps
    shape / device / dtype readable afterwards."""

    _BACKUP_METADATA_KEYS = ["shape", "device", "dtype"]

    def __init__(self, value: torch.Tensor):
        self._value = value
        self._backup_metadata: Optional[Dict[str, Any]] = None

    @property
    def value(self):
        assert not self.is_disposed
        return self._value

    def dispose(self, backup_metadata: bool = True):
        assert not self.is_disposed
        if not torch.compiler.is_compiling():
            refcount = sys.getrefcount(self._value)
            assert refcount == 2, f"refcount={refcount}"
        if backup_metadata:
            self._backup_metadata = {k: getattr(self._value, k) for k in self._BACKUP_METADATA_KEYS}
        self._value = None

    @property
    def is_disposed(self):
        return self._value is None

    @staticmethod
    def maybe_unwrap(value):
        return value.value if isinstance(value, DisposibleTensor) else value

    @staticmethod
    def maybe_dispose(value):
        if isinstance(value, DisposibleTensor):
            value.dispose()

    def _meta(self, name):
        if not self.is_disposed:
            return getattr(self._value, name)
        assert self._backup_metadata is not None, "Use backup_metadata flag if you want to use metadata after dispose"
        return self._backup_metadata[name]

    shape = property(lambda self: self._meta("shape"))
    device = property(lambda self: self._meta("device"))
    dtype = property(lambda self: self._meta("dtype"))


MaybeDisposibleTensor = Union[torch.Tensor, DisposibleTensor]
