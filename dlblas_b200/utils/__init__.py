"""`dlblas.utils` surface kept by this package (dlblas/utils/__init__.py:8-23 of the reference)."""
from ..op_registry import op_registry
from ..op_struct import OpImpl, OpParams
from ..symbolic_var import SymVar, Tensor
from .logger import get_logger
from .utils import DisposibleTensor

register_dlblas_op = op_registry.register


def get_list_op_names():
    return op_registry.get_list_op_names()


def get_args_from_op_name(name: str):
    return op_registry.get_args_from_op_name(name)


def get_op(name: str, args):
    """Returns the OpImpl (callable) registered under `name` that matches `args`."""
    return op_registry.get_op(name, args)
