"""Per-layer expert load statistics for the load balancer
(dlblas/layers/moe/experts_distribution_recorder.py:12-54 of the reference): token counts per expert,
accumulated over steps, summed over ranks, dumped as JSON [layers][experts] every few minutes by one rank.
The dump is the file `EPLBMetadata.init` reads through EPLB_EXPERTS_STATISTIC_FILE."""
import json
import os
from datetime import datetime

import torch
import torch.distributed as dist

from ...utils.logger import get_logger

logger = get_logger(__name__)


class ExpertsDistributionRecorder:

    def __init__(self, output_dir: str):
        self.output_dir = output_dir
        self.dispatch_count = {}
        self.accum_token_counts = {}
        self.global_token_counts = {}
        self.last_dump_minute = -1
        self.dump_frequency = int(os.getenv("DLBLAS_EPLB_DUMP_FREQUENCY", 5))
        self.dump_rank = int(os.getenv("DLBLAS_EPLB_DUMP_RANK", 0))

    def map_to_sorted_2d_array(self, data_map):
        keys = sorted(data_map.keys(), key=lambda k: int(k.split("_")[0]))
        return [data_map[k].cpu().tolist() for k in keys]

    def record(self, topk_ids: torch.Tensor, layer_index: int, num_experts: int, now: datetime = None):
        key = f"{layer_index}_{num_experts}"
        self.dispatch_count[key] = self.dispatch_count.get(key, 0) + 1
        if key not in self.accum_token_counts:
            self.accum_token_counts[key] = torch.zeros(num_experts, dtype=torch.int64, device=topk_ids.device)
        flat = topk_ids.reshape(-1)
        flat = flat[flat >= 0]                                  # slots masked with -1 carry no load
        self.accum_token_counts[key] += torch.bincount(flat, minlength=num_experts)[:num_experts]
        total = self.accum_token_counts[key].clone()
        if dist.is_initialized():
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
        self.global_token_counts[key] = total
        rank = dist.get_rank() if dist.is_initialized() else 0
        now = now or datetime.now()
        if rank == self.dump_rank and now.minute % self.dump_frequency == 0 and now.minute != self.last_dump_minute:
            self.last_dump_minute = now.minute
            os.makedirs(self.output_dir, exist_ok=True)
            path = os.path.join(self.output_dir, f"rank{rank}_step{self.dispatch_count[key]}_experts_counts.json")
            with open(path, "w") as f:
                json.dump(self.map_to_sorted_2d_array(self.global_token_counts), f, indent=2)
            logger.info(f"[EPLB] Experts distribution dumped to {path}")
            return path
        return None
