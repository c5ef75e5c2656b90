"""vLLM-style entry points: moe_align_block_size against fixtures from the reference's kernel, and
fused_moe (v2) against the oracle."""
import pytest
import torch

from oracle import moe_oracle as O

DEV = "cuda"


def test_align_oracle_against_reference(golden):
    cases = golden("align_block.pt")
    assert len(cases) == 4
    assert cases[0]["sorted_ids"][:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    for c in cases:
        s_ids, e_ids, n_post = O.moe_align_block_size(c["topk_ids"], c["block_size"], c["num_experts"],
                                                      c["pad_sorted_ids"])
        n = int(c["num_tokens_post_pad"])
        assert int(n_post) == n
        assert torch.equal(s_ids, c["sorted_ids"])
        assert torch.equal(e_ids[: n // c["block_size"]], c["expert_ids"][: n // c["block_size"]])


@pytest.mark.gpu
def test_align_kernel_path(golden):
    from dlblas_b200.kernels.moe_align_block_size import moe_align_block_size
    for c in golden("align_block.pt"):
        ids = c["topk_ids"].clone().to(DEV)
        s_ids, e_ids, n_post = moe_align_block_size(ids, c["block_size"], c["num_experts"], c["num_experts"], None,
                                                    c["pad_sorted_ids"])
        assert torch.equal(s_ids.cpu(), c["sorted_ids"]) and s_ids.dtype == torch.int32
        assert torch.equal(n_post.cpu(), c["num_tokens_post_pad"])
        assert torch.equal(e_ids.cpu(), c["expert_ids"])
    # negative ids become the "not local" id in place; an expert map translates block experts
    ids = torch.tensor([[0, -1], [1, 0], [-1, -1]], dtype=torch.int32, device=DEV)
    emap = torch.tensor([5, 6, -1], dtype=torch.int32, device=DEV)
    s_ids, e_ids, n_post = moe_align_block_size(ids, 4, 3, 2, emap)
    assert ids.cpu().tolist() == [[0, 2], [1, 0], [2, 2]]
    assert s_ids.cpu().tolist()[:12] == [0, 3, 6, 6, 2, 6, 6, 6, 1, 4, 5, 6] and int(n_post) == 12
    assert e_ids.cpu().tolist()[:3] == [5, 6, -1]


@pytest.mark.gpu
def test_fused_moe_v2_against_oracle():
    from dlblas_b200.kernels.fused_moe_v2 import fused_moe
    x, logits, w13, w13s, w2, w2s = O.make_layer_inputs(77, 256, 256, 8, seed=3)
    w, ids = O.softmax_topk(logits, 2, True)
    out = fused_moe(x.to(DEV), w13.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), use_fp8_w8a8=True,
                    w1_scale=w13s.to(DEV), w2_scale=w2s.to(DEV), block_shape=[128, 128])
    ref = O.fused_moe_v2(x, w13, w13s, w2, w2s, w, ids)
    assert out.dtype == torch.bfloat16 and O.rel_frobenius(out.cpu(), ref) < 2e-2
    # expert parallel shard: only experts 4..7 are local
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3], dtype=torch.int32)
    out_ep = fused_moe(x.to(DEV), w13[4:].to(DEV), w2[4:].to(DEV), w.to(DEV), ids.to(DEV), use_fp8_w8a8=True,
                       expert_map=emap.to(DEV), w1_scale=w13s[4:].to(DEV), w2_scale=w2s[4:].to(DEV),
                       block_shape=[128, 128])
    w_masked = torch.where(ids >= 4, w, torch.zeros_like(w))
    ref_ep = O.fused_moe_v2(x, w13, w13s, w2, w2s, w_masked, ids)
    assert O.rel_frobenius(out_ep.cpu(), ref_ep) < 2e-2
    with pytest.raises(AssertionError):               # e4m3 weights without use_fp8_w8a8: the unquantised mode wants 16-bit
        fused_moe(x.to(DEV), w13.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV))
    with pytest.raises(NotImplementedError):
        fused_moe(x.to(DEV), w13.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), use_int8_w8a8=True)
