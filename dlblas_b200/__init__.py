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


def install_as_dlblas():
    """Make `import dlblas` (and the sub-modules of this path) resolve to this package."""
    import importlib
    me = sys.modules[__name__]
    sys.modules.setdefault("dlblas", me)
    for sub in ("utils", "op_registry", "op_struct", "symbolic_var", "cache", "kernels", "kernels.fp8_gemm",
                "kernels.fp8", "kernels.moe", "kernels.activation", "kernels.quant_dequant", "kernels.fused_moe_v3",
                "kernels.topk_gating", "layers", "layers.moe", "layers.moe.ep_moe", "layers.moe.token_dispatcher",
                "layers.moe.kernels", "layers.moe.kernels.fused_moe", "layers.moe.kernels.blocked_fp8_fused_moe",
                "layers.moe.kernels.activation", "utils.logger", "utils.utils", "utils.device_utils"):
        sys.modules.setdefault("dlblas." + sub, importlib.import_module(__name__ + "." + sub))
    return me
