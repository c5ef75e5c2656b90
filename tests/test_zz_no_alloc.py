"""The allocation-free sort entry point, called through the C ABI.

`dlb_sort_by_expert_static` serves callers that have no device memory left to give as a
workspace and may not call the allocator (an engine whose memory pool owns the whole GPU,
code on a path where an allocation's device-wide synchronisation is not tolerable).  Its
scratch is a fixed array inside the library, shared by all calls, never cleared.  The test
runs it twice in a row on different inputs — the second call sees the first call's leftovers
in the scratch — and requires bit-identical results to the workspace-taking entry point.
This file sorts last on purpose, so a `-x` run has executed every other test before it.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_both(ids, num_experts):
    from dlblas_b200 import _C
    lib = _C.lib()
    n = ids.numel()
    outs = []
    for static in (False, True):
        sidx = torch.full((n,), -7, dtype=torch.int64, device=DEV)
        se = torch.full((2, num_experts), -7, dtype=torch.int64, device=DEV)
        pos = torch.full((n,), -7, dtype=torch.int32, device=DEV)
        rank = torch.full((n,), -7, dtype=torch.int32, device=DEV)
        cnt = torch.full((num_experts,), -7, dtype=torch.int32, device=DEV)
        st = torch.cuda.current_stream().cuda_stream
        if static:
            rc = lib.dlb_sort_by_expert_static(ids.data_ptr(), _C.dtype_code(ids.dtype), n, num_experts, sidx.data_ptr(),
                                               se[0].data_ptr(), se[1].data_ptr(), pos.data_ptr(), rank.data_ptr(),
                                               cnt.data_ptr(), st)
        else:
            ws_bytes = lib.dlb_sort_by_expert_workspace_size(n, num_experts)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=DEV)
            rc = lib.dlb_sort_by_expert(ids.data_ptr(), _C.dtype_code(ids.dtype), n, num_experts, sidx.data_ptr(),
                                        se[0].data_ptr(), se[1].data_ptr(), pos.data_ptr(), rank.data_ptr(),
                                        cnt.data_ptr(), ws.data_ptr(), ws_bytes, st)
        _C.check(rc)
        torch.cuda.synchronize()
        outs.append((sidx, se, pos, rank, cnt))
    return outs


def test_static_scratch_sort_matches_workspace_sort_twice_in_a_row():
    from dlblas_b200 import _C
    lib = _C.lib()
    g = torch.Generator().manual_seed(123)
    # both inputs are large enough for the multi-kernel path, the one that uses scratch
    first = torch.randint(-1, 256, (40000 * 8,), generator=g, dtype=torch.int64).to(DEV)
    second = torch.randint(0, 64, (20001 * 6,), generator=g, dtype=torch.int32).to(DEV)
    for ids, e in ((first, 256), (second, 64)):
        assert lib.dlb_sort_by_expert_workspace_size(ids.numel(), e) > 0
        ref, got = _run_both(ids, e)
        for a, b in zip(ref, got):
            assert torch.equal(a, b)                      # integer outputs: bit-exact
        flat = ids.long().cpu()
        assert torch.equal(got[0].cpu(), torch.argsort(flat, stable=True))
    # a request beyond the built-in capacity is refused with a clear message, nothing is launched
    cap = lib.dlb_sort_by_expert_static_capacity()
    assert lib.dlb_sort_by_expert_workspace_size(1 << 24, 1090) > cap
    rc = lib.dlb_sort_by_expert_static(first.data_ptr(), _C.DLB_I64, 1 << 24, 1090, None, None, None, None, None, None,
                                       None)
    assert rc == -2 and b"built-in" in lib.dlb_last_error_string()
