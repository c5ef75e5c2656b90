"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares,
the registry behaves like the reference's, and operators refuse to run without a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "dlblas_b200.h")).read()
    return sorted(set(re.findall(r"\b(dlb_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    from dlblas_b200 import _C
    from dlblas_b200.build import build
    build()
    handle = ctypes.CDLL(_C.SO_PATH)
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/dlblas_b200.h but not exported"
        assert n in _C.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_C.SIGNATURES) == names
    assert _C.lib().dlb_version() >= 100


def test_argument_validation_without_gpu():
    """Size / dtype checks run before any CUDA call and report through the error string."""
    from dlblas_b200 import _C
    lib = _C.lib()
    assert lib.dlb_fp8_gemm(None, None, None, 1, 1, None, None, _C.DLB_BF16, 4, 128, 100, 0, None, None) == -1
    assert b"multiple of 128" in lib.dlb_last_error_string()
    assert lib.dlb_quant_fp8(None, _C.DLB_BF16, 4, 100, 100, 128, 0, 0.0, None, None, 1, 1, None, 1, None) == -1
    assert lib.dlb_sort_by_expert(None, _C.DLB_F32, 8, 4, None, None, None, None, None, None, None, 0, None) == -1
    assert lib.dlb_route_softmax_topk(None, _C.DLB_F32, 8, 2000, 2, 0, None, None, _C.DLB_I64, None) == -1
    with pytest.raises(AssertionError):
        _C.check(-1)
    assert lib.dlb_sort_by_expert_workspace_size(1 << 20, 256) > 0
    assert lib.dlb_topk_gating_workspace_size(4096, 64, 8) > 4096 * 64 * 4


def test_ops_refuse_cpu_tensors():
    from dlblas_b200.kernels.fp8_gemm import fp8_gemm
    from dlblas_b200.kernels.moe import quant_fp8
    a = torch.zeros(2, 128).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CUDA"):
        fp8_gemm(a, torch.zeros(128, 128).to(torch.float8_e4m3fn), torch.ones(2, 1), torch.ones(1, 1))
    with pytest.raises(RuntimeError, match="CUDA"):
        quant_fp8(torch.zeros(2, 128, dtype=torch.bfloat16), 128)


def test_registry_surface():
    import dlblas_b200
    from dlblas_b200.utils import (SymVar, Tensor, get_args_from_op_name, get_list_op_names, get_op, op_registry,
                                   register_dlblas_op)
    assert "topk_gating" in get_list_op_names()
    assert op_registry.get_op_count("topk_gating") == 2          # fp16 and fp32 registrations
    assert len(get_args_from_op_name("topk_gating")) == 2
    calls = []

    def impl(x, n):
        calls.append((x.shape, n))
        return x + n

    s = SymVar("s")
    register_dlblas_op("unit_add", None, (Tensor((s, s), dtype=torch.float32, device="cpu"), torch.SymInt), impl, None,
                       impl)
    x = torch.zeros(3, 3)
    op = get_op("unit_add", (x, 2))
    assert torch.equal(op(x, 2), x + 2) and calls
    assert op_registry.look_up_cache("unit_add", (x, 2)) is op          # second lookup is a cache hit
    assert op_registry.cache.gen_key("unit_add", (x, 2)) == "unit_add-0:f32_3x3-1:2"
    with pytest.raises(LookupError):
        get_op("unit_add", (torch.zeros(3, 4), 2))                       # symbol reused with different sizes
    with pytest.raises(LookupError):
        get_op("unit_add", (x.double(), 2))
    with pytest.raises(NameError):
        get_op("no_such_op", (x,))
    with pytest.raises(LookupError):
        # registered for cuda tensors only
        dlblas_b200.topk_gating(torch.zeros(4, 4), 2)


def test_install_as_dlblas_alias():
    import dlblas_b200
    dlblas_b200.install_as_dlblas()
    import dlblas
    from dlblas.kernels.fp8_gemm import fp8_gemm  # noqa: F401
    from dlblas.layers.moe.ep_moe import DlblasTritonFusedMoEBlockedF8Impl, build_deepep_moe  # noqa: F401
    from dlblas.layers.moe.kernels.fused_moe import _dlblas_get_sorted_idx  # noqa: F401
    assert dlblas.topk_gating is dlblas_b200.topk_gating
    impl = DlblasTritonFusedMoEBlockedF8Impl(top_k=2, num_experts=8, ep_size=2)
    assert impl.support_ep() and impl.ep_expert_list(2, 1) == [4, 5, 6, 7]


def test_disposible_tensor():
    from dlblas_b200.utils import DisposibleTensor
    d = DisposibleTensor(torch.zeros(2, 3))
    assert d.shape == (2, 3)
    d.dispose()
    assert d.is_disposed and d.shape == (2, 3) and d.dtype == torch.float32


def test_ctypes_signatures_have_the_header_arity():
    """Every binding passes exactly as many arguments as the header declares."""
    from dlblas_b200 import _C
    hdr = open(os.path.join(ROOT, "include", "dlblas_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    decls = re.findall(r"DLB_API\s+[\w\s\*]+?\b(dlb_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", hdr, flags=re.S)
    assert len(decls) == len(_C.SIGNATURES)
    for name, params in decls:
        params = params.strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(_C.SIGNATURES[name][1]), f"{name}: header has {n} parameters, binding {len(_C.SIGNATURES[name][1])}"


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure: nothing under the package (or the C sources) may refer to it."""
    pkg = os.path.join(ROOT, "dlblas_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), os.path.join(root, f)
                assert "moe_oracle" not in text, os.path.join(root, f)
