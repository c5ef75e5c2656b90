"""Expert-parallel load balancer: placement tables for replicated ("redundant") experts.

Same tables as dlblas/layers/moe/eplb.py of the reference (itself DeepSeek's EPLB as carried by sglang):
`rebalance_experts` (:90-108) = group packing onto nodes, replication of the hottest experts inside a
node, packing of the replicas onto GPUs (:53-87), or plain replication when groups do not divide over
nodes; `compute_logical_to_rank_dispatch_physical_map` (:130-170) = for every rank the replica it sends a
logical expert to (its own GPU's replica when there is one).  All of it is host arithmetic on small
integer tables, written on numpy; tensors in, tensors out, on the device of the input.

Ties: the greedy steps take the first best candidate (lowest pack index, lowest expert index), like
`min(..., key=)` and `Tensor.max(dim).indices` in the reference; items of equal load are visited in the
order of the reference's (unstable) `torch.sort` call on the host.
"""
import os
import random
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch


def _pack_greedy(load: np.ndarray, num_packs: int) -> Tuple[np.ndarray, np.ndarray]:
    """Heaviest-first assignment of `n` items to `num_packs` packs of exactly n / num_packs items:
    every item goes to the lightest pack that still has room.  Returns (pack of item, slot inside pack)."""
    rows, n = load.shape
    assert n % num_packs == 0
    room = n // num_packs
    if room == 1:
        return np.tile(np.arange(n, dtype=np.int64), (rows, 1)), np.zeros((rows, n), dtype=np.int64)
    pack_of = np.full((rows, n), -1, dtype=np.int64)
    slot_of = np.full((rows, n), -1, dtype=np.int64)
    # equal loads are structural (the replicas of one expert): keep the order the reference's own call,
    # an unstable torch.sort on fp32, gives them on the host
    order = torch.from_numpy(np.ascontiguousarray(load, dtype=np.float32)).sort(-1, descending=True).indices.numpy()
    for r in range(rows):
        weight = np.zeros(num_packs, dtype=np.float64)
        used = np.zeros(num_packs, dtype=np.int64)
        for item in order[r]:
            open_packs = np.flatnonzero(used < room)
            p = open_packs[np.argmin(weight[open_packs])]
            pack_of[r, item] = p
            slot_of[r, item] = used[p]
            weight[p] += float(load[r, item])
            used[p] += 1
    return pack_of, slot_of


def balanced_packing(weight: torch.Tensor, num_packs: int) -> Tuple[torch.Tensor, torch.Tensor]:
    p, s = _pack_greedy(weight.detach().cpu().float().numpy(), num_packs)
    return torch.from_numpy(p).to(weight.device), torch.from_numpy(s).to(weight.device)


def _replicate(load: np.ndarray, num_phy: int):
    """Adds num_phy - num_log replicas one at a time, each to the expert whose load per replica is highest."""
    rows, num_log = load.shape
    assert num_phy >= num_log
    load = load.astype(np.float32)
    phy2log = np.tile(np.arange(num_phy, dtype=np.int64), (rows, 1))
    rank = np.zeros((rows, num_phy), dtype=np.int64)
    count = np.ones((rows, num_log), dtype=np.int64)
    rr = np.arange(rows)
    for slot in range(num_log, num_phy):
        hot = np.argmax(load / count.astype(np.float32), axis=1)
        phy2log[:, slot] = hot
        rank[:, slot] = count[rr, hot]
        count[rr, hot] += 1
    return phy2log, rank, count


def replicate_experts(weight: torch.Tensor, num_phy: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    out = _replicate(weight.detach().cpu().float().numpy(), num_phy)
    return tuple(torch.from_numpy(o).to(weight.device) for o in out)


def _invert(perm: np.ndarray) -> np.ndarray:
    inv = np.empty_like(perm)
    np.put_along_axis(inv, perm, np.tile(np.arange(perm.shape[1], dtype=np.int64), (perm.shape[0], 1)), axis=1)
    return inv


def _rebalance_hierarchical(load: np.ndarray, num_phy: int, num_groups: int, num_nodes: int, num_gpus: int):
    layers, num_log = load.shape
    assert num_log % num_groups == 0 and num_groups % num_nodes == 0
    assert num_gpus % num_nodes == 0 and num_phy % num_gpus == 0
    group_size = num_log // num_groups
    groups_per_node = num_groups // num_nodes
    phy_per_gpu = num_phy // num_gpus
    log_per_node = num_log // num_nodes
    # 1. whole expert groups onto nodes, balancing the nodes' load
    group_load = load.reshape(layers, num_groups, group_size).sum(-1)
    g_pack, g_slot = _pack_greedy(group_load, num_nodes)
    log2mlog = (((g_pack * groups_per_node + g_slot) * group_size)[:, :, None] +
                np.arange(group_size, dtype=np.int64)).reshape(layers, num_log)
    mlog2log = _invert(log2mlog)
    # 2. replicas inside each node
    node_load = np.take_along_axis(load, mlog2log, axis=1).reshape(layers * num_nodes, log_per_node)
    phy2mlog, phy_rank, mlog_cnt = _replicate(node_load, num_phy // num_nodes)
    # 3. replicas onto the node's GPUs
    per_phy = np.take_along_axis(node_load.astype(np.float32) / mlog_cnt.astype(np.float32), phy2mlog, axis=1)
    pack, slot = _pack_greedy(per_phy, num_gpus // num_nodes)
    pphy2phy = _invert(pack * phy_per_gpu + slot)
    pphy2mlog = np.take_along_axis(phy2mlog, pphy2phy, axis=1).reshape(layers, num_nodes, -1)
    pphy2mlog = (pphy2mlog + (np.arange(num_nodes, dtype=np.int64) * log_per_node)[None, :, None]).reshape(layers, -1)
    pphy2log = np.take_along_axis(mlog2log, pphy2mlog, axis=1)
    pphy_rank = np.take_along_axis(phy_rank, pphy2phy, axis=1).reshape(layers, -1)
    log_cnt = np.take_along_axis(mlog_cnt.reshape(layers, -1), log2mlog, axis=1)
    return pphy2log, pphy_rank, log_cnt


def rebalance_experts_hierarchical(weight: torch.Tensor, num_physical_experts: int, num_groups: int, num_nodes: int,
                                   num_gpus: int):
    out = _rebalance_hierarchical(weight.detach().cpu().float().numpy(), num_physical_experts, num_groups, num_nodes,
                                  num_gpus)
    return tuple(torch.from_numpy(o).to(weight.device) for o in out)


def rebalance_experts(weight: torch.Tensor, num_replicas: int, num_groups: int, num_nodes: int,
                      num_gpus: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """weight [layers, logical experts] = observed load.  Returns physical -> logical [layers, replicas],
    logical -> physical [layers, experts, max replicas] (-1 padded) and the replica count per logical expert."""
    load = weight.detach().cpu().float().numpy()
    layers, num_log = load.shape
    if num_groups % num_nodes == 0:
        phy2log, phy_rank, log_cnt = _rebalance_hierarchical(load, num_replicas, num_groups, num_nodes, num_gpus)
    else:
        phy2log, phy_rank, log_cnt = _replicate(load, num_replicas)
    width = int(log_cnt.max())
    log2phy = np.full((layers, num_log * width), -1, dtype=np.int64)
    np.put_along_axis(log2phy, phy2log * width + phy_rank,
                      np.tile(np.arange(num_replicas, dtype=np.int64), (layers, 1)), axis=1)
    dev = weight.device
    return (torch.from_numpy(phy2log).to(dev), torch.from_numpy(log2phy.reshape(layers, num_log, width)).to(dev),
            torch.from_numpy(log_cnt).to(dev))


def logical_to_all_physical_raw(logical_to_all_physical_map, layer_id: int, logical_expert_id: int) -> List[int]:
    return [p for p in logical_to_all_physical_map[layer_id, logical_expert_id].tolist() if p != -1]


def compute_logical_to_rank_dispatch_physical_map(logical_to_all_physical_map: torch.Tensor, num_gpus: int,
                                                  num_physical_experts: int, seed: int = 42):
    """[num_gpus, layers, logical experts]: the replica each rank dispatches to.  A rank that hosts a replica
    uses it (the first one); the others share the replicas evenly, in an order drawn from
    `random.Random(seed)` exactly as the reference draws it (whole rounds of all replicas, a sample for the
    remainder, one shuffle)."""
    rng = random.Random(seed)
    per_gpu = num_physical_experts // num_gpus
    table = logical_to_all_physical_map.detach().cpu().numpy()
    layers, num_log, _ = table.shape
    out = np.full((num_gpus, layers, num_log), -1, dtype=table.dtype)
    for layer in range(layers):
        for e in range(num_log):
            replicas = [int(p) for p in table[layer, e] if p != -1]
            col = out[:, layer, e]
            for p in reversed(replicas):          # the first replica on a GPU wins
                col[p // per_gpu] = p
            missing = np.flatnonzero(col == -1)
            if len(missing):
                rounds, rest = divmod(len(missing), len(replicas))
                picks = replicas * rounds + rng.sample(replicas, k=rest)
                rng.shuffle(picks)
                col[missing] = picks
    assert (out != -1).all()
    return torch.from_numpy(out).to(logical_to_all_physical_map.dtype)


@dataclass
class EPLBMetadata:
    physical_to_logical_map: torch.Tensor                 # (layers, physical experts)
    logical_to_all_physical_map: torch.Tensor             # (layers, logical experts, physical experts), -1 padded
    logical_to_all_physical_map_num_valid: torch.Tensor   # (layers, logical experts)
    logical_to_rank_dispatch_physical_map: torch.Tensor   # (gpus, layers, logical experts)

    def num_physical_experts(self) -> int:
        return self.physical_to_logical_map.shape[1]

    def __post_init__(self):
        layers, phys = self.physical_to_logical_map.shape
        l1, logical, p1 = self.logical_to_all_physical_map.shape
        l2, e2 = self.logical_to_all_physical_map_num_valid.shape
        _, l3, e3 = self.logical_to_rank_dispatch_physical_map.shape
        assert layers == l1 == l2 == l3
        assert logical == e2 == e3
        assert phys == p1

    @staticmethod
    def _init_raw(ep_size: int, physical_to_logical_map: torch.Tensor, logical_to_all_physical_map: torch.Tensor):
        phys = physical_to_logical_map.shape[1]
        padded = torch.nn.functional.pad(logical_to_all_physical_map,
                                         (0, phys - logical_to_all_physical_map.shape[-1]), value=-1)
        return EPLBMetadata(
            physical_to_logical_map=physical_to_logical_map,
            logical_to_all_physical_map=padded,
            logical_to_all_physical_map_num_valid=torch.count_nonzero(logical_to_all_physical_map != -1, dim=-1),
            logical_to_rank_dispatch_physical_map=compute_logical_to_rank_dispatch_physical_map(
                logical_to_all_physical_map, num_gpus=ep_size, num_physical_experts=phys))

    @staticmethod
    def init(ep_size: int, num_routed_experts: int, num_hidden_layers: int, device=None):
        """Environment as in the reference (:217-252): EPLB_NUM_GROUPS, EPLB_EXPERTS_STATISTIC_FILE (JSON
        [layers][experts]), RANKS_PER_NODES, EPLB_NUM_REDUNDANT_EXPERTS; without a statistics file the load is
        taken as descending in the expert index."""
        num_groups = int(os.getenv("EPLB_NUM_GROUPS", 4))
        stat_path = os.getenv("EPLB_EXPERTS_STATISTIC_FILE", None)
        ranks_per_node = int(os.getenv("RANKS_PER_NODES", 8))
        redundant = int(os.getenv("EPLB_NUM_REDUNDANT_EXPERTS", 32))
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        if stat_path is None:
            stat = torch.arange(num_routed_experts, dtype=torch.int32, device=device).flip(dims=(0,)).expand(
                num_hidden_layers, -1)
        else:
            try:
                import json
                with open(stat_path, "r") as f:
                    stat = torch.tensor(json.load(f), dtype=torch.float32, device=device)
            except Exception:
                raise RuntimeError(f"Load eplb experts statistic data failed, path: {stat_path}")
            want = torch.Size([num_hidden_layers, num_routed_experts])
            assert stat.shape == want, f"Shape of {stat_path} must be {want}"
        num_nodes = 1 if ep_size < ranks_per_node else ep_size // ranks_per_node
        phy2log, log2phy, _ = rebalance_experts(stat, num_routed_experts + redundant, num_groups, num_nodes, ep_size)
        return EPLBMetadata._init_raw(ep_size, phy2log, log2phy)


_global_eplb_metadata: Optional[EPLBMetadata] = None


def init_global_eplb_metadata(ep_size: int, num_routed_experts: int, num_hidden_layers: int):
    global _global_eplb_metadata
    assert _global_eplb_metadata is None
    _global_eplb_metadata = EPLBMetadata.init(ep_size, num_routed_experts, num_hidden_layers)


def get_global_eplb_metadata():
    assert _global_eplb_metadata is not None
    return _global_eplb_metadata


def get_eplb_phy2log_metadata_by_layer(layer_idx: int):
    assert _global_eplb_metadata is not None
    return _global_eplb_metadata.physical_to_logical_map[layer_idx]


@dataclass
class EPLBDispatchInfo:
    partial_logical_to_rank_dispatch_physical_map: torch.Tensor
    partial_logical_to_all_physical_map: torch.Tensor
    partial_logical_to_all_physical_map_num_valid: torch.Tensor

    @classmethod
    def init_new(cls, ep_rank: int, layer_idx: int):
        meta = get_global_eplb_metadata()
        return cls(meta.logical_to_rank_dispatch_physical_map[ep_rank, layer_idx, :],
                   meta.logical_to_all_physical_map[layer_idx, :],
                   meta.logical_to_all_physical_map_num_valid[layer_idx, :])


def topk_ids_logical_to_physical(topk_ids: torch.Tensor, info: Optional[EPLBDispatchInfo]) -> torch.Tensor:
    """Random replica per routed slot (:294-308): uniform over the replicas of the slot's logical expert."""
    if info is None:
        return topk_ids
    flat = topk_ids.flatten()
    valid = info.partial_logical_to_all_physical_map_num_valid.to(flat.device)[flat]
    pick = torch.randint(0, 65536, flat.shape, dtype=torch.int32, device=flat.device) % valid
    table = info.partial_logical_to_all_physical_map.to(flat.device)
    return table[flat, pick].view(topk_ids.shape)
