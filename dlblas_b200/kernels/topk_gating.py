"""`dlblas.topk_gating` (dlblas/kernels/topk_gating.py:245-317 of the reference), forward and backward:
capacity-limited softmax top-k gating, registered with the op registry under 'topk_gating'."""
import math
import struct

import torch

from .. import ops
from ..symbolic_var import SymVar
from ..symbolic_var import Tensor as FakeTensor
from ..utils import register_dlblas_op


def _capacity(num_tokens: int, num_experts: int, capacity_factor: float, min_capacity: int) -> int:
    """ceil(T / E * capacity_factor), at least min_capacity (topk_gating.py:15-24), computed on the host from the
    shape: no device round trip.  The reference multiplies the Python float T / E by a float32 tensor and takes
    the ceiling in float32; the same single-precision product is formed here, because a double-precision one
    lands on the other side of an integer for some shapes (e.g. T = 50290, E = 8, factor 2.4)."""
    prod = struct.unpack("f", struct.pack("f", num_tokens / num_experts))[0] * \
        struct.unpack("f", struct.pack("f", capacity_factor))[0]
    prod = struct.unpack("f", struct.pack("f", prod))[0]      # the product of two floats, rounded to float
    return max(int(math.ceil(prod)), int(min_capacity))


class TopKGatingFunc(torch.autograd.Function):
    """dlblas/kernels/topk_gating.py:245-285.  The backward always differentiates the auxiliary loss
    (topk_gating_bwd.py:13-68); with higher_precision it also differentiates token_exp_weights.  The
    reference's code for that second path cannot run (it picks the gradient of the integer index output) and
    scales its coupling term by an extra 1 / denominator; the gradient here is the exact one."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2,
                higher_precision: bool = False):
        t, e = logits.shape
        capacity = _capacity(t, e, capacity_factor * k, min_capacity)
        l_aux, ec_idx, w, sel, ws = ops.topk_gating(logits.contiguous(), k, capacity, return_workspace=True)
        ctx.save_for_backward(ws)
        ctx.meta = (logits.dtype, t, e, k, capacity, bool(higher_precision))
        ctx.mark_non_differentiable(ec_idx, sel)
        return l_aux, ec_idx, w, sel

    @staticmethod
    def backward(ctx, grad_l_aux, _grad_ec_idx, grad_weights, _grad_sel):
        (ws,) = ctx.saved_tensors
        dtype, t, e, k, capacity, hp = ctx.meta
        if grad_l_aux is None:
            grad_l_aux = torch.zeros((), dtype=dtype, device=ws.device)
        gw = grad_weights if hp else None
        return ops.topk_gating_bwd(ws, dtype, t, e, k, capacity, grad_l_aux, gw), None, None, None, None


def call(logits: torch.Tensor, k: int, capacity_factor: float = 1.0, min_capacity: int = 2,
         enable_token_rearrange_opt: bool = False):
    """Returns (l_aux, token_rearranged_ec_idx int32 [k*T], token_exp_weights [k*T],
    expert_select_token_idx int64 [E*capacity]).  Both settings of the last flag give the same
    four outputs in the reference (:256-268); it selects how much the backward differentiates."""
    if logits.requires_grad and torch.is_grad_enabled():
        return TopKGatingFunc.apply(logits, k, capacity_factor, min_capacity, enable_token_rearrange_opt)
    t, e = logits.shape
    capacity = _capacity(t, e, capacity_factor * k, min_capacity)
    return ops.topk_gating(logits.contiguous(), k, capacity)


def bench_fn(logits, k, capacity_factor=1.0, min_capacity=2, enable_token_rearrange_opt=False):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        call(logits, k, capacity_factor, min_capacity, enable_token_rearrange_opt)
    start.record()
    for _ in range(10):
        call(logits, k, capacity_factor, min_capacity, enable_token_rearrange_opt)
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / 10


name = "topk_gating"
for _dtype in [torch.float16, torch.float32]:
    _logits = FakeTensor((SymVar("seqLen"), SymVar("experts")), dtype=_dtype, device="cuda")
    register_dlblas_op(name, None, (_logits, torch.SymInt, torch.SymFloat, torch.SymInt, torch.SymBool), call, bench_fn,
                       call)
