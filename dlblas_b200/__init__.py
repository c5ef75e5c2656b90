"""dlblas_b200 — the FP8 MoE expert path of DLBlas, written for B200 (sm_100a).

The package keeps the reference's module layout for this path, so `dlblas_b200.X` stands in for
`dlblas.X`:

    dlblas_b200.topk_gating                                   (dlblas/__init__.py:15-25)
    dlblas_b200.utils.get_op / register_dlblas_op             (dlblas/utils/__init__.py:8-23)
    dlblas_b200.kernels.fp8_gemm.fp8_gemm                     (dlblas/kernels/fp8_gemm.py:68)
    dlblas_b200.kernels.fp8.per_token_group_quant_fp8         (dlblas/kernels/fp8.py:108)
    dlblas_b200.kernels.moe.{quant_fp8, biased_grouped_topk, silu_and_mul_masked_post_quant_fwd}
    dlblas_b200.kernels.fused_moe_v3.{ep_scatter, ep_gather, fused_moe_v3}
    dlblas_b200.layers.moe.ep_moe.{DlblasTritonFusedMoEBlockedF8Impl, FusedMoENormal,
                                   FusedMoELowLatency, build_deepep_moe}

`install_as_dlblas()` additionally publishes the package under the name `dlblas` so existing
`import dlblas...` call sites of this path resolve to it.  All arithmetic runs in the CUDA
extension `_dlblas_b200.so` (C ABI in include/dlblas_b200.h); importing the package needs
neither a GPU nor the extension, calling an operator needs both.
"""
import sys
from typing import Tuple

from torch import Tensor

from . import kernels  # noqa: F401  registers the ops, like `import dlblas.kernels` in the reference
from .utils import get_op

__version__ = "0.0.7+b200"


def topk_gating(logits: Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2,
                higher_precision: bool = False) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Capacity-limited top-k gating; returns (l_aux, token_rearranged_ec_idx, token_exp_weights,
    expert_select_token_idx).  Dispatched through the op registry like the reference."""
    op = get_op("topk_gating", (logits, k, capacity_factor, min_capacity, higher_precision))
    return op(logits, k, capacity_factor, min_capacity, higher_precision)


class _AliasFinder:
    """Resolves `dlblas` and every `dlblas.<sub>` import to the module object of `dlblas_b200.<sub>`, so that
    the two names share one module (one registry, one library handle, one set of module-level state)."""

    def __init__(self, alias: str, target: str):
        self.alias, self.target = alias, target

    def find_spec(self, fullname, path=None, target=None):
        if fullname != self.alias and not fullname.startswith(self.alias + "."):
            return None
        import importlib.machinery
        return importlib.machinery.ModuleSpec(fullname, self)

    def create_module(self, spec):
        import importlib
        module = importlib.import_module(self.target + spec.name[len(self.alias):])
        self._specs = getattr(self, "_specs", {})
        self._specs[id(module)] = getattr(module, "__spec__", None)
        return module

    def exec_module(self, module):
        # already executed under its own name; the import system has just stamped the alias spec on it
        original = getattr(self, "_specs", {}).pop(id(module), None)
        if original is not None:
            module.__spec__ = original


def install_as_dlblas():
    """Make `import dlblas` and `import dlblas.<anything on this path>` resolve to this package."""
    me = sys.modules[__name__]
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder("dlblas", __name__))
    sys.modules.setdefault("dlblas", me)
    return me
