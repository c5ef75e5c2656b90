"""Expert-parallel load balancer: host tables against fixtures produced by the reference's own
dlblas/layers/moe/eplb.py, the hash oracle against the golden model of tests/kernels/test_eplb.py,
and the statistics recorder."""
import json
import os
from datetime import datetime

import pytest
import torch

from oracle import moe_oracle as O


def _hash_cases(golden):
    for c in golden("eplb.pt")["hash"]:
        if "topk_idx" in c:
            yield c["name"], c["topk_idx"], c, None
        else:
            topk = torch.full((c["num_tokens"], c["topk_rows"].shape[1]), -1, dtype=torch.int32)
            topk[c["rows"]] = c["topk_rows"]
            yield c["name"], topk, c, c["rows"]


def test_hash_oracle_matches_reference_model(golden):
    n = 0
    for name, topk, c, rows in _hash_cases(golden):
        got = O.eplb_hash_map(topk, c["log2phy"], c["logcnt"], c["seed"])
        if rows is None:
            assert torch.equal(got, c["model_out"]), name
        else:
            assert torch.equal(got[rows], c["model_out_rows"]), name   # token ids past 2^16: (t << 16) wraps
        n += 1
    assert n == 4


def test_rebalance_tables_match_reference(golden):
    from dlblas_b200.layers.moe import eplb
    tables = golden("eplb.pt")["tables"]
    assert len(tables) == 6
    for t in tables:
        phy2log, log2phy, logcnt = eplb.rebalance_experts(t["weight"], t["num_replicas"], t["num_groups"],
                                                          t["num_nodes"], t["num_gpus"])
        assert torch.equal(phy2log, t["phy2log"])
        assert torch.equal(log2phy, t["log2phy"])
        assert torch.equal(logcnt, t["logcnt"])
        disp = eplb.compute_logical_to_rank_dispatch_physical_map(log2phy, t["num_gpus"], t["num_replicas"], seed=42)
        assert torch.equal(disp, t["dispatch"])
        # every physical slot serves the logical expert that lists it
        for layer in range(phy2log.shape[0]):
            for p, e in enumerate(phy2log[layer].tolist()):
                assert p in log2phy[layer, e].tolist()
        assert int(logcnt.sum()) == phy2log.numel()


def test_metadata_and_dispatch_info(monkeypatch):
    from dlblas_b200.layers.moe import eplb
    monkeypatch.setenv("EPLB_NUM_REDUNDANT_EXPERTS", "8")
    monkeypatch.setenv("EPLB_NUM_GROUPS", "4")
    monkeypatch.setattr(eplb, "_global_eplb_metadata", None)
    meta = eplb.EPLBMetadata.init(ep_size=4, num_routed_experts=16, num_hidden_layers=2, device="cpu")
    assert meta.num_physical_experts() == 24
    assert meta.logical_to_all_physical_map.shape == (2, 16, 24)
    assert meta.logical_to_rank_dispatch_physical_map.shape == (4, 2, 16)
    monkeypatch.setattr(eplb, "_global_eplb_metadata", meta)
    info = eplb.EPLBDispatchInfo.init_new(ep_rank=1, layer_idx=0)
    ids = torch.randint(0, 16, (50, 4), generator=torch.Generator().manual_seed(0))
    phys = eplb.topk_ids_logical_to_physical(ids, info)
    assert phys.shape == ids.shape
    assert torch.equal(meta.physical_to_logical_map[0][phys], ids)       # a replica of the right expert
    assert eplb.topk_ids_logical_to_physical(ids, None) is ids
    assert torch.equal(eplb.get_eplb_phy2log_metadata_by_layer(1), meta.physical_to_logical_map[1])


def test_recorder_accumulates_and_dumps(tmp_path):
    from dlblas_b200.layers.moe.experts_distribution_recorder import ExpertsDistributionRecorder
    rec = ExpertsDistributionRecorder(str(tmp_path))
    ids = torch.tensor([[0, 1], [1, 2], [-1, 3]])
    assert rec.record(ids, layer_index=3, num_experts=4, now=datetime(2024, 1, 1, 10, 1)) is None   # minute 1: no dump
    path = rec.record(ids, layer_index=3, num_experts=4, now=datetime(2024, 1, 1, 10, 5))
    assert path is not None and os.path.exists(path)
    assert json.load(open(path)) == [[2, 4, 2, 2]]
    assert rec.record(ids, 3, 4, now=datetime(2024, 1, 1, 10, 5)) is None                           # once per minute
    assert rec.global_token_counts["3_4"].tolist() == [3, 6, 3, 3]


@pytest.mark.gpu
def test_hash_kernel_matches_oracle_and_reference_model(golden):
    from dlblas_b200.kernels.moe import map_logic_to_physical_idx_hash_random
    for name, topk, c, rows in _hash_cases(golden):
        for dt in (torch.int32, torch.int64):
            got = map_logic_to_physical_idx_hash_random(topk.to(dt).cuda(), c["log2phy"].cuda(), c["logcnt"].cuda(),
                                                        seed=c["seed"]).cpu()
            assert got.dtype == torch.int32
            assert torch.equal(got, O.eplb_hash_map(topk, c["log2phy"], c["logcnt"], c["seed"])), name
            if rows is None:
                assert torch.equal(got, c["model_out"]), name
            else:
                assert torch.equal(got[rows], c["model_out_rows"]), name
    empty = map_logic_to_physical_idx_hash_random(torch.empty(0, 2, dtype=torch.int32, device="cuda"),
                                                  c["log2phy"].cuda(), c["logcnt"].cuda())
    assert empty.shape == (0, 2)
