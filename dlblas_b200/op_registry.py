"""Name -> implementation registry behind `get_op` (dlblas/op_registry.py:19-162 of the
reference).  Differences, on purpose: there is no autotuner and no benchmark-based selection
(the reference times every candidate with 200 kernel runs on the first call of a shape,
op_registry.py:124-136); the first matching candidate is taken, and nothing imports Triton."""
from dataclasses import dataclass, field
from typing import Optional

from .cache import Cache
from .op_struct import OpImpl, match, parse_args


@dataclass
class OpRegistry:
    ops: dict = field(default_factory=dict)
    cache: Cache = field(default_factory=Cache)

    def register(self, name, spaces, args, call, bench_fn, kernel):
        params = parse_args(args)
        impl = OpImpl(params, getattr(call, "__module__", None), None, spaces, call, bench_fn, kernel)
        if name in self.ops:
            assert self.ops[name][0].params == params, \
                f"Multiple implementations of a kernel:{name} must have the same parameters."
            self.ops[name].append(impl)
        else:
            self.ops[name] = [impl]

    def get_op_count(self, name):
        return len(self.ops[name])

    def get_list_op_names(self):
        return list(self.ops.keys())

    def get_args_from_op_name(self, op_name: str):
        return [i.params for i in self.ops[op_name]]

    def look_up_cache(self, op_name: str, args: tuple, cache_key=None) -> Optional[OpImpl]:
        return self.cache.get(op_name, args, cache_key)

    def get_op(self, op_name: str, args: tuple, configs=None, cache_key=None) -> OpImpl:
        if op_name not in self.ops:
            raise NameError(f"op {op_name} not found")
        op = self.look_up_cache(op_name, args, cache_key)
        if op is not None:
            return op
        candidates = [op for op in self.ops[op_name] if match(args, op.params)]
        if not candidates:
            raise LookupError(f"no candidates for op {op_name} with args")
        self.cache.put(candidates[0], op_name, args, cache_key)
        return candidates[0]


op_registry = OpRegistry()
