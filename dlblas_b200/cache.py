"""In-process operator cache keyed by name + per-argument dtype/shape
(dlblas/cache.py:58-138 of the reference; key format of `gen_key`, :63-75)."""
import pickle
from typing import Optional

import torch

from .op_struct import OpImpl

_DTYPE_NAMES = {torch.float16: "f16", torch.float32: "f32", torch.bfloat16: "bf16", torch.int32: "i32",
                torch.int64: "i64", torch.float8_e4m3fn: "f8e4m3"}


def convert_dtype(t: torch.Tensor) -> str:
    return _DTYPE_NAMES.get(t.dtype, str(t.dtype).replace("torch.", ""))


def convert_shapes(t: torch.Tensor) -> str:
    return "x".join(str(s) for s in t.shape)


class Cache:
    def __init__(self):
        self._cache = {}

    def gen_key(self, op_name, args) -> str:
        key = op_name
        for i, arg in enumerate(args):
            key += "-" + str(i) + ":"
            key += (convert_dtype(arg) + "_" + convert_shapes(arg)) if isinstance(arg, torch.Tensor) else str(arg)
        return key

    def put(self, op: OpImpl, op_name, args, cache_key=None):
        self._cache[self.gen_key(op_name, args) if cache_key is None else cache_key] = op

    def get(self, op_name, args, cache_key=None) -> Optional[OpImpl]:
        return self._cache.get(self.gen_key(op_name, args) if cache_key is None else cache_key)

    def __len__(self):
        return len(self._cache)

    def to_file(self, fname):
        with open(f"{fname}.pkl", "wb") as fh:
            pickle.dump({k: (v.params.n_args, getattr(v.call, "__name__", "")) for k, v in self._cache.items()}, fh)
