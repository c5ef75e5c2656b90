"""Token permutation for MoE training, forward and backward
(dlblas/kernels/permute/moe_triton_kernels.py of the reference; the autograd wrappers follow
tests/kernels/permute/triton_ops.py).

permute:    rows of `input` are replicated top_k times and ordered by expert (stable: ascending flat slot
            index inside an expert; slots routed to -1 are dropped).  `row_id_map` int32 [top_k * tokens],
            k-major, gives the destination row of every (token, slot), -1 for dropped slots.
unpermute:  out[t] = sum_k prob[t, k] * permuted[row_id_map[k, t]], rounded to the tensor type after every
            product and add (the reference accumulates in the tensor type).
The module keeps its reference name although nothing here is Triton: the kernels are the library's sort,
fan-out copy and un-permute kernels.
"""
from typing import List, Optional, Tuple

import torch

from ... import ops
from ..._C import check, dtype_code, lib, ptr, require_cuda, stream


def _destinations(indices: torch.Tensor):
    """(sorted slot ids, destination row per flat slot or -1, number of dropped slots as a 0-d tensor)."""
    num_experts_bound = int(indices.max().item()) + 1 if indices.numel() else 1
    sidx, _, _, pos = ops.sort_by_expert(indices.contiguous(), max(num_experts_bound, 1), want_pos=True)
    dropped = (pos < 0).sum()
    dest = torch.where(pos >= 0, pos - dropped.to(pos.dtype), torch.full_like(pos, -1))
    return sidx, dest.to(torch.int32), dropped


def moe_permute_topk_op_triton(input_tensor: torch.Tensor, indices: torch.Tensor, num_out_tokens: int,
                               workspace: List[torch.Tensor], max_expanded_token_num: int,
                               num_negative_one_in_indices: int, permuted_output: torch.Tensor,
                               row_id_map: torch.Tensor):
    """Reference signature (:62-137).  Fills `permuted_output` [num_out_tokens, H] and `row_id_map`; returns
    (permuted_output, row_id_map, sorted_row_id, workspace).  Entries of row_id_map for dropped slots are set
    to -1 (the reference leaves them unwritten)."""
    require_cuda(input_tensor, indices)
    t, k = indices.shape
    h = input_tensor.shape[1]
    if num_out_tokens <= 0:
        num_out_tokens = t * k - num_negative_one_in_indices
    assert permuted_output.shape == (num_out_tokens, h), "permuted_output shape mismatch"
    assert row_id_map.numel() == t * k, "row_id_map size mismatch"
    sidx, dest, _ = _destinations(indices)
    dest_k = torch.where(dest < num_out_tokens, dest, torch.full_like(dest, -1))
    x = input_tensor.contiguous()
    row_bytes = h * x.element_size()
    check(lib().dlb_permute_rows(ptr(x), row_bytes, 0, 0, t, ptr(dest_k), k, ptr(permuted_output), 0, stream(x.device)))
    row_id_map.view(k, t).copy_(dest_k.view(t, k).t())
    return permuted_output, row_id_map, sidx, workspace


def moe_recover_topk_op_triton(input_tensor: torch.Tensor, row_id_map: torch.Tensor, prob: Optional[torch.Tensor],
                               num_tokens: int, num_topK: int) -> torch.Tensor:
    """Weighted gather back to token order (:274-301); prob None = plain sum."""
    require_cuda(input_tensor, row_id_map)
    x = input_tensor.contiguous()
    h = x.shape[1]
    out = torch.empty(num_tokens, h, dtype=x.dtype, device=x.device)
    p = None if prob is None else prob.to(torch.float32).contiguous()
    check(lib().dlb_unpermute(ptr(x), dtype_code(x.dtype), ptr(row_id_map.contiguous()), 0 if p is None else ptr(p),
                              num_tokens, num_topK, h, ptr(out), stream(x.device)))
    return out


def moe_permute_topk_bwd_op(permuted_act_grad: torch.Tensor, sorted_row_id: torch.Tensor, original_shape, num_topK: int):
    """Gradient of permute (:190-213): act_grad[t] = sum over the token's slots of permuted_act_grad[row].
    `sorted_row_id` lists the flat slot of every permuted row (rows of dropped slots must not be included)."""
    require_cuda(permuted_act_grad)
    t = original_shape[0]
    rows = permuted_act_grad.shape[0]
    sid = sorted_row_id.to(torch.int64)[-rows:] if sorted_row_id.numel() > rows else sorted_row_id.to(torch.int64)
    rmap = torch.full((num_topK * t,), -1, dtype=torch.int32, device=permuted_act_grad.device)
    rmap[(sid % num_topK) * t + sid // num_topK] = torch.arange(rows, dtype=torch.int32, device=rmap.device)
    return moe_recover_topk_op_triton(permuted_act_grad, rmap, None, t, num_topK)


def moe_recover_topk_bwd_op_triton(input_bwd: torch.Tensor, input_fwd: torch.Tensor, row_id_map: torch.Tensor,
                                   prob: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gradient of unpermute (:480-528): (act_grad fp32 [rows, H], prob_grad fp32 [tokens, top_k])."""
    require_cuda(input_bwd, input_fwd)
    t, k = prob.shape
    h = input_bwd.shape[1]
    go, fw = input_bwd.contiguous(), input_fwd.contiguous()
    act_grad = torch.zeros(fw.shape, dtype=torch.float32, device=fw.device)
    prob_grad = torch.empty(t, k, dtype=torch.float32, device=fw.device)
    check(lib().dlb_unpermute_bwd(ptr(go), ptr(fw), dtype_code(go.dtype), ptr(row_id_map.contiguous()),
                                  ptr(prob.to(torch.float32).contiguous()), t, k, h, ptr(act_grad), ptr(prob_grad),
                                  stream(fw.device)))
    return act_grad, prob_grad


class _Permute(torch.autograd.Function):
    workspace: List[torch.Tensor] = []

    @staticmethod
    def forward(ctx, input_act: torch.Tensor, indices: torch.Tensor):
        if not input_act.numel():
            return input_act, None
        if indices.dim() == 1:
            indices = indices.view(-1, 1)
        if not input_act.is_cuda or not indices.is_cuda:
            raise RuntimeError("permute needs CUDA tensors")
        if input_act.size(0) != indices.size(0):
            raise RuntimeError(f"token count mismatch: {input_act.size(0)} vs {indices.size(0)}")
        t, k = indices.shape
        dropped = int((indices == -1).sum().item())
        out = torch.zeros(t * k - dropped, input_act.size(1), dtype=input_act.dtype, device=input_act.device)
        rmap = torch.empty(t * k, dtype=torch.int32, device=input_act.device)
        out, rmap, _, _Permute.workspace = moe_permute_topk_op_triton(input_act, indices, t * k - dropped,
                                                                      _Permute.workspace, t * k, dropped, out, rmap)
        ctx.save_for_backward(rmap)
        ctx.shape, ctx.k = input_act.shape, k
        ctx.mark_non_differentiable(rmap)
        return out, rmap

    @staticmethod
    def backward(ctx, grad_permuted, _):
        if not grad_permuted.numel():
            return grad_permuted, None
        (rmap,) = ctx.saved_tensors
        return moe_recover_topk_op_triton(grad_permuted.contiguous(), rmap, None, ctx.shape[0], ctx.k), None


class _Unpermute(torch.autograd.Function):

    @staticmethod
    def forward(ctx, input_act: torch.Tensor, row_id_map: torch.Tensor, probs: Optional[torch.Tensor]):
        if not input_act.numel():
            ctx.probs = probs
            return input_act
        t = probs.size(0) if probs is not None else row_id_map.numel()
        k = probs.size(1) if probs is not None else 1
        out = moe_recover_topk_op_triton(input_act, row_id_map, probs, t, k)
        ctx.save_for_backward(input_act, row_id_map, probs)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        if not grad_out.numel():
            return grad_out, None, ctx.probs
        input_act, rmap, probs = ctx.saved_tensors
        if probs is None:
            ones = torch.ones(rmap.numel(), 1, dtype=torch.float32, device=grad_out.device)
            act_grad, _ = moe_recover_topk_bwd_op_triton(grad_out, input_act, rmap, ones)
            return act_grad.to(input_act.dtype), None, None
        act_grad, prob_grad = moe_recover_topk_bwd_op_triton(grad_out, input_act, rmap, probs)
        return act_grad.to(input_act.dtype), None, (prob_grad.to(probs.dtype) if ctx.needs_input_grad[2] else None)


def permute(input_act: torch.Tensor, indices: torch.Tensor):
    """(permuted activations [routed slots, H], row_id_map); differentiable in `input_act`."""
    return _Permute.apply(input_act, indices)


def unpermute(input_act: torch.Tensor, row_id_map: torch.Tensor, probs: Optional[torch.Tensor] = None):
    """Weighted combine back to token order; differentiable in `input_act` and `probs`."""
    return _Unpermute.apply(input_act, row_id_map, probs)
