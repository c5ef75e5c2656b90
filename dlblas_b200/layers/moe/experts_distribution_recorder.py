"""Per-layer expert load statistics for the load balancer.

Counterpart of dlblas/layers/moe/experts_distribution_recorder.py:12-54 of the reference: `record()` is called once
per MoE layer and step with the routing ids; token counts per expert accumulate per (layer, expert count) key, are
summed over the ranks of the default process group, and one rank writes them as JSON `[layers][experts]` (layers in
ascending order) at most once per minute whose number is a multiple of DLBLAS_EPLB_DUMP_FREQUENCY.  The file is what
`EPLBMetadata.init` reads through EPLB_EXPERTS_STATISTIC_FILE.  Unlike the reference, slots routed to -1 are ignored
(`bincount` would reject them) and tensors stay on the device of the ids instead of a hard-coded 'cuda'."""
import json
import os
from datetime import datetime
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ...utils.logger import get_logger

logger = get_logger(__name__)


def _layer_of(key: str) -> int:
    return int(key.split("_", 1)[0])


class ExpertsDistributionRecorder:

    def __init__(self, output_dir: str):
        self.output_dir = output_dir
        self.dump_frequency = int(os.getenv("DLBLAS_EPLB_DUMP_FREQUENCY", 5))
        self.dump_rank = int(os.getenv("DLBLAS_EPLB_DUMP_RANK", 0))
        self.last_dump_minute = -1
        # all three keyed by "<layer>_<num_experts>", as in the reference
        self.dispatch_count: Dict[str, int] = {}
        self.accum_token_counts: Dict[str, torch.Tensor] = {}
        self.global_token_counts: Dict[str, torch.Tensor] = {}

    def map_to_sorted_2d_array(self, data_map):
        """Rows of `data_map` as nested lists, ordered by layer number."""
        return [data_map[k].cpu().tolist() for k in sorted(data_map, key=_layer_of)]

    def _accumulate(self, key: str, topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
        routed = topk_ids.reshape(-1)
        routed = routed[routed >= 0]
        step = torch.bincount(routed, minlength=num_experts)[:num_experts]
        total = self.accum_token_counts.get(key)
        total = step.to(torch.int64) if total is None else total + step
        self.accum_token_counts[key] = total
        return total

    def _dump_due(self, rank: int, now: datetime) -> bool:
        return rank == self.dump_rank and now.minute % self.dump_frequency == 0 and now.minute != self.last_dump_minute

    def record(self, topk_ids: torch.Tensor, layer_index: int, num_experts: int,
               now: Optional[datetime] = None) -> Optional[str]:
        """Returns the path of the dump written by this call, if any.  `now` is for tests."""
        key = f"{layer_index}_{num_experts}"
        step_no = self.dispatch_count[key] = self.dispatch_count.get(key, 0) + 1
        over_ranks = self._accumulate(key, topk_ids, num_experts).clone()
        multi = dist.is_available() and dist.is_initialized()
        if multi:
            dist.all_reduce(over_ranks, op=dist.ReduceOp.SUM)
        self.global_token_counts[key] = over_ranks
        rank = dist.get_rank() if multi else 0
        now = now or datetime.now()
        if not self._dump_due(rank, now):
            return None
        self.last_dump_minute = now.minute
        os.makedirs(self.output_dir, exist_ok=True)
        path = os.path.join(self.output_dir, f"rank{rank}_step{step_no}_experts_counts.json")
        with open(path, "w") as fh:
            json.dump(self.map_to_sorted_2d_array(self.global_token_counts), fh, indent=2)
        logger.info(f"[EPLB] Experts distribution dumped to {path}")
        return path
