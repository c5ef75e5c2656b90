"""Operator records and argument matching (dlblas/op_struct.py:14-161 of the reference)."""
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from .symbolic_var import Tensor


@dataclass(frozen=True)
class OpParams:
    n_args: int
    args_types: tuple
    args: tuple

    def __eq__(self, other) -> bool:
        assert isinstance(other, OpParams)
        return self.n_args == other.n_args and tuple(self.args_types) == tuple(other.args_types)

    def __hash__(self):
        return hash((self.n_args, tuple(str(t) for t in self.args_types)))


@dataclass
class OpImpl:
    params: OpParams
    file_path: Optional[str]
    src: Optional[str]
    spaces: Any
    call: Callable
    bench_fn: Optional[Callable]
    kernel: Any

    def __call__(self, *args, **kwargs):
        return self.call(*args, **kwargs)

    def bench(self, *args, **kwargs):
        return self.bench_fn(*args, **kwargs)


def parse_args(args: tuple) -> OpParams:
    types = []
    for i, arg in enumerate(args):
        if isinstance(arg, Tensor):
            types.append("tensor")
        elif isinstance(arg, str):
            types.append("str")
        elif isinstance(arg, int) or arg is torch.SymInt:
            types.append("int")
        elif arg is torch.SymFloat or arg is torch.SymBool:
            types.append(arg)
        else:
            raise TypeError(f"arg {i} has unsupported type {type(arg)}")
    return OpParams(n_args=len(args), args_types=tuple(types), args=tuple(args))


_PY_TYPES = {"str": str, "int": int, torch.SymFloat: float, torch.SymBool: bool}


def match(user_args, op_params: OpParams) -> bool:
    """True if the call arguments fit the registered signature: positional count, Python
    types, tensor dtype, device prefix, and equal sizes wherever one symbol is reused."""
    if not isinstance(user_args, tuple):
        raise TypeError(f"user_args must be a tuple, but got {type(user_args)}")
    if not isinstance(op_params, OpParams):
        raise TypeError(f"op_params must be an OpParams, but got {type(op_params)}")
    if len(user_args) != op_params.n_args:
        return False
    bound = {}
    for want, spec, arg in zip(op_params.args_types, op_params.args, user_args):
        if arg is None:
            continue
        if want == "tensor":
            if not isinstance(arg, torch.Tensor) or arg.dtype != spec.dtype:
                return False
            if not str(arg.device).startswith(spec.device):
                return False
            if len(arg.shape) < len(spec.shape):
                return False
            for sym, size in zip(spec.shape, arg.shape):
                if bound.setdefault(sym, size) != size:
                    return False
        else:
            py = _PY_TYPES[want]
            if not isinstance(arg, py) or (py is int and isinstance(arg, bool)):
                return False
    return True
