"""`dlblas.utils` surface kept by this package (dlblas/utils/__init__.py:8-23 of the reference):
`register_dlblas_op`, `get_op`, `get_list_op_names`, `get_args_from_op_name`, all thin views of the one
registry object, plus the symbolic argument types operators are registered with."""
from ..op_registry import op_registry as _registry
from ..op_struct import OpImpl, OpParams  # noqa: F401
from ..symbolic_var import SymVar, Tensor  # noqa: F401
from .logger import get_logger  # noqa: F401
from .utils import DisposibleTensor  # noqa: F401

op_registry = _registry

# bound methods of the registry: same callables, same signatures as the reference's module-level functions
register_dlblas_op = _registry.register
get_list_op_names = _registry.get_list_op_names
get_args_from_op_name = _registry.get_args_from_op_name
get_op = _registry.get_op
