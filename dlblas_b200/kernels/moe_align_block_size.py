"""`dlblas.kernels.moe_align_block_size` of the reference (vLLM's block-aligned token layout,
dlblas/kernels/moe_align_block_size.py:138-210).

Every expert's slots are laid out contiguously and padded to a multiple of `block_size`:
sorted_ids int32 [max padded] holds flat slot indices (t * top_k + j) grouped by expert in ascending slot
order, padding entries = topk_ids.numel(); expert_ids int32 [blocks] = expert of every block (0 for blocks
past the end); num_tokens_post_pad int32 [1].  Built from the library's stable sort (counts and rank inside the
expert) and index arithmetic on the device, no host round trip.
"""
from typing import Optional, Tuple

import torch

from .. import ops


def ceil_div(a: int, b: int) -> int:
    return -(a // -b)


def round_up(x: int, y: int) -> int:
    return ((x + y - 1) // y) * y


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int, num_local_experts: int,
                         expert_map: Optional[torch.Tensor] = None,
                         pad_sorted_ids: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Same contract as the reference, including its side effect: negative ids in `topk_ids` are replaced
    in place by `num_local_experts` (the "not on this rank" id, :178-180).  Ids >= num_experts are ignored."""
    numel = topk_ids.numel()
    dev = topk_ids.device
    topk_ids[topk_ids < 0] = num_local_experts
    max_padded = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_padded = round_up(max_padded, block_size)
    max_blocks = ceil_div(max_padded, block_size)
    _, _, _, rank, counts = ops.sort_by_expert(topk_ids, num_experts, want_rank=True, want_counts=True)
    padded = (counts.to(torch.int64) + (block_size - 1)) // block_size * block_size
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    sorted_ids = torch.full((max_padded,), numel, dtype=torch.int32, device=dev)
    flat = topk_ids.reshape(-1).to(torch.int64)
    ok = flat < num_experts
    dest = starts[flat.clamp(max=num_experts - 1)] + rank.to(torch.int64)
    slots = torch.arange(numel, dtype=torch.int32, device=dev)
    sorted_ids[dest[ok]] = slots[ok]
    block_start = torch.arange(max_blocks, dtype=torch.int64, device=dev) * block_size
    expert_ids = torch.searchsorted(ends, block_start, right=True)
    expert_ids = torch.where(expert_ids < num_experts, expert_ids, torch.zeros_like(expert_ids)).to(torch.int32)
    num_tokens_post_pad = ends[-1:].to(torch.int32)
    if expert_map is not None:
        expert_ids = expert_map[expert_ids.long()]
    return sorted_ids, expert_ids, num_tokens_post_pad
