"""Training-side permutation: oracle against fixtures produced by the reference's kernels
(dlblas/kernels/permute/moe_triton_kernels.py under the interpreter, fp32 data), and the CUDA path
against the oracle, forward and backward."""
import pytest
import torch

from oracle import moe_oracle as O

DEV = "cuda"


def _check_permutation(x, ids, permuted, rmap):
    """Properties every admissible permutation has (the reference's sort leaves the order inside an
    expert open): each routed slot's row is a copy of its token, rows are grouped by ascending expert."""
    t, k = ids.shape
    m = rmap.view(k, t)
    experts_of_rows = torch.full((permuted.shape[0],), -1, dtype=torch.int64)
    for j in range(k):
        ok = ids[:, j] >= 0
        assert bool((m[j][~ok] == -1).all())
        assert torch.equal(permuted[m[j][ok].long()], x[ok])
        experts_of_rows[m[j][ok].long()] = ids[ok, j].long()
    assert bool((experts_of_rows >= 0).all())
    assert bool((experts_of_rows[1:] >= experts_of_rows[:-1]).all())


def test_oracle_against_reference_kernels(golden):
    cases = golden("permute.pt")
    assert len(cases) == 2
    for c in cases:
        t, k = c["ids"].shape
        _check_permutation(c["x"], c["ids"], c["permuted"], c["row_id_map"])        # the reference's own output
        perm, rmap, order = O.permute_topk(c["x"], c["ids"])
        _check_permutation(c["x"], c["ids"], perm, rmap)
        assert torch.equal(c["ids"].flatten()[order], c["ids"].flatten()[c["sorted_row_id"]])
        assert torch.equal(O.unpermute_topk(c["y"], c["row_id_map"], c["probs"], t, k), c["unpermuted"])
        assert torch.equal(O.unpermute_topk(c["y"], c["row_id_map"], None, t, k), c["unpermuted_noprob"])
        act, pg = O.unpermute_topk_bwd(c["grad_out"], c["y"], c["row_id_map"], c["probs"])
        assert torch.equal(act, c["act_grad"])
        torch.testing.assert_close(pg, c["prob_grad"], rtol=1e-5, atol=1e-5)
        if "permute_bwd" in c:
            assert torch.equal(O.unpermute_topk(c["grad_permuted"], c["row_id_map"], None, t, k), c["permute_bwd"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_permute_unpermute_forward_backward(golden, dtype):
    from dlblas_b200.kernels.permute import (moe_permute_topk_bwd_op, moe_recover_topk_bwd_op_triton,
                                             moe_recover_topk_op_triton, permute, unpermute)
    for c in golden("permute.pt"):
        t, k = c["ids"].shape
        x = c["x"].to(dtype)
        xd = x.to(DEV).requires_grad_(True)
        perm, rmap = permute(xd, c["ids"].to(DEV))
        o_perm, o_rmap, _ = O.permute_topk(x, c["ids"])
        assert torch.equal(perm.detach().cpu(), o_perm) and torch.equal(rmap.cpu(), o_rmap)   # stable order, bit-exact
        y = c["y"].to(dtype)
        probs = c["probs"]
        yd = y.to(DEV).requires_grad_(True)
        pd = probs.to(DEV).requires_grad_(True)
        out = unpermute(yd, rmap, pd)
        # the oracle's map differs from the fixture's only inside experts; use ours throughout
        ref = O.unpermute_topk(y, o_rmap, probs, t, k)
        assert torch.equal(out.detach().cpu(), ref)
        assert torch.equal(moe_recover_topk_op_triton(y.to(DEV), rmap, None, t, k).cpu(),
                           O.unpermute_topk(y, o_rmap, None, t, k))
        go = c["grad_out"].to(dtype)
        out.backward(go.to(DEV))
        act, pg = O.unpermute_topk_bwd(go, y, o_rmap, probs)
        assert torch.equal(yd.grad.cpu(), act.to(dtype))
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        torch.testing.assert_close(pd.grad.cpu(), pg, rtol=tol, atol=tol * float(pg.abs().max()))
        a2, p2 = moe_recover_topk_bwd_op_triton(go.to(DEV), y.to(DEV), rmap, probs.to(DEV))
        assert a2.dtype == torch.float32 and torch.equal(a2.cpu(), act)
        # permute backward = plain sum over the token's slots
        gp = c["grad_permuted"].to(dtype)
        perm.backward(gp.to(DEV))
        assert torch.equal(xd.grad.cpu(), O.unpermute_topk(gp, o_rmap, None, t, k))
        if int((c["ids"] < 0).sum()) == 0:
            _, _, order = O.permute_topk(x, c["ids"])
            got = moe_permute_topk_bwd_op(gp.to(DEV), order.to(DEV), (t, x.shape[1]), k)
            assert torch.equal(got.cpu(), O.unpermute_topk(gp, o_rmap, None, t, k))
