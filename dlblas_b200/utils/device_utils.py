"""Device probe (dlblas/utils/device_utils.py:21-45 of the reference), CUDA only and lazy:
importing this module never touches the GPU."""
import functools

import torch


@functools.lru_cache(maxsize=None)
def get_device_props(device_idx: int = 0):
    p = torch.cuda.get_device_properties(device_idx)
    return {"multi_processor_count": p.multi_processor_count, "warps_per_sm": 64,
            "capability": (p.major, p.minor), "total_memory": p.total_memory}


def infer_device() -> str:
    return "cuda"
