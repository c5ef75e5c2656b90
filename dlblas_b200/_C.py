"""ctypes binding of the C ABI in include/dlblas_b200.h.

The shared library is built in-tree by ``python -m dlblas_b200.build`` (or
``__graft_entry__.build()``).  There is no fallback: if the library is missing,
``lib()`` raises, and every operator of this package raises with it.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# DLBLAS_B200_LIB overrides the location of the shared library (e.g. an out-of-tree build)
SO_PATH = os.environ.get("DLBLAS_B200_LIB") or os.path.join(_HERE, "_dlblas_b200.so")

DLB_F32, DLB_BF16, DLB_F16, DLB_I32, DLB_I64 = 0, 1, 2, 3, 4
QUANT_RECIP_MUL, QUANT_DIV_EPS = 0, 1
EPI_STORE, EPI_SCATTER_WEIGHT, EPI_SWIGLU_QUANT = 0, 1, 2

_DTYPE_CODE = {
    torch.float32: DLB_F32, torch.bfloat16: DLB_BF16, torch.float16: DLB_F16,
    torch.int32: DLB_I32, torch.int64: DLB_I64,
}

c_i64, c_int, c_vp, c_sz, c_f = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float

# name -> (restype, argtypes); must list every symbol include/dlblas_b200.h declares
SIGNATURES = {
    "dlb_version": (c_int, []),
    "dlb_last_error_string": (ctypes.c_char_p, []),
    "dlb_launch_count": (c_i64, [c_int]),
    "dlb_set_wait_policy": (c_int, [ctypes.c_uint64, c_int]),
    "dlb_sort_by_expert_workspace_size": (c_sz, [c_i64, c_int]),
    "dlb_sort_by_expert": (c_int, [c_vp, c_int, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "dlb_sort_by_expert_static_capacity": (c_sz, []),
    "dlb_sort_by_expert_static": (c_int, [c_vp, c_int, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "dlb_moe_build_tiles": (c_int, [c_vp, c_vp, c_int, c_int, c_vp, c_int, c_vp]),
    "dlb_moe_build_tiles_masked": (c_int, [c_vp, c_int, c_int, c_vp, c_int, c_vp]),
    "dlb_quant_fp8": (c_int, [c_vp, c_int, c_i64, c_i64, c_i64, c_int, c_int, c_f, c_vp, c_vp, c_i64, c_i64, c_vp,
                              c_int, c_vp]),
    "dlb_permute_rows": (c_int, [c_vp, c_i64, c_vp, c_i64, c_i64, c_vp, c_int, c_vp, c_vp, c_vp]),
    "dlb_silu_and_mul": (c_int, [c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_i64, c_vp]),
    "dlb_silu_mul_quant": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_f, c_int, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "dlb_fp8_gemm": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_int, c_vp, c_vp]),
    "dlb_moe_grouped_gemm": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_int, c_i64, c_i64, c_vp, c_int, c_int, c_int, c_vp,
                                     c_int, c_i64, c_vp, c_int, c_f, c_vp, c_vp, c_vp, c_vp]),
    "dlb_moe_grouped_gemm_window": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_int, c_i64, c_i64, c_vp, c_int, c_int, c_int,
                                            c_vp, c_int, c_i64, c_vp, c_int, c_f, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64,
                                            c_int]),
    "dlb_ep_dest_ranks": (c_int, [c_vp, c_int, c_i64, c_int, c_int, c_int, c_vp, c_vp]),
    "dlb_moe_sum_topk": (c_int, [c_vp, c_int, c_i64, c_int, c_i64, c_vp, c_int, c_i64, c_i64, c_int, c_vp, c_vp]),
    "dlb_ep_gather": (c_int, [c_vp, c_int, c_i64, c_vp, c_vp, c_int, c_vp, c_i64, c_int, c_vp, c_vp]),
    "dlb_ep_scatter_workspace_size": (c_sz, [c_i64, c_int, c_int]),
    "dlb_ep_scatter": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_int, c_i64, c_int, c_vp, c_int, c_vp, c_vp, c_vp,
                               c_vp, c_i64, c_vp, c_vp, c_sz, c_vp]),
    "dlb_p2p_quant_push": (c_int, [c_vp, c_int, c_i64, c_i64, c_i64, c_int, c_f, c_vp, c_int, c_int, c_i64, c_vp, c_vp,
                                   c_vp, c_vp, c_int, c_vp, c_vp, c_vp]),
    "dlb_p2p_unpack_meta": (c_int, [c_vp, c_int, c_int, c_vp, c_int, c_i64, c_int, c_int, c_vp, c_vp, c_vp]),
    "dlb_p2p_sum_push": (c_int, [c_vp, c_int, c_vp, c_int, c_i64, c_vp, c_int, c_int, c_i64, c_vp, c_vp]),
    "dlb_p2p_sum_push_cols": (c_int, [c_vp, c_int, c_vp, c_int, c_i64, c_vp, c_int, c_int, c_i64, c_vp, c_vp, c_i64, c_i64,
                                      c_int]),
    "dlb_p2p_push_rows": (c_int, [c_vp, c_i64, c_vp, c_int, c_int, c_i64, c_vp, c_vp]),
    "dlb_p2p_push_rows_masked": (c_int, [c_vp, c_i64, c_vp, c_int, c_int, c_vp, c_vp, c_int, c_vp, c_vp]),
    "dlb_p2p_barrier": (c_int, [c_vp, c_int, c_int, c_vp, ctypes.c_uint64, c_vp, c_vp]),
    "dlb_p2p_ll_plan": (c_int, [c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_vp,
                                c_vp, c_vp, c_vp, c_vp]),
    "dlb_p2p_all_gather_small": (c_int, [c_vp, c_i64, c_int, c_int, c_vp, c_vp]),
    "dlb_p2p_ll_quant_push": (c_int, [c_vp, c_int, c_i64, c_i64, c_i64, c_int, c_f, c_vp, c_vp, c_int, c_int, c_vp, c_vp,
                                      c_vp]),
    "dlb_p2p_push_rows_indexed": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp, c_int, c_vp, c_vp]),
    "dlb_grouped_gemm_16bit": (c_int, [c_vp, c_vp, c_int, c_i64, c_int, c_i64, c_i64, c_vp, c_int, c_int, c_vp, c_i64,
                                       c_vp, c_vp]),
    "dlb_grouped_gemm_16bit_b_kn": (c_int, [c_vp, c_vp, c_int, c_i64, c_int, c_i64, c_i64, c_vp, c_int, c_int, c_vp,
                                            c_i64, c_vp, c_vp]),
    "dlb_k_grouped_gemm_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64, c_int, c_int]),
    "dlb_k_grouped_gemm_16bit": (c_int, [c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_int, c_int, c_vp, c_i64, c_vp,
                                         c_vp, c_vp]),
    "dlb_moe_build_tiles_rows": (c_int, [c_vp, c_vp, c_int, c_int, c_int, c_vp, c_int, c_vp]),
    "dlb_unpermute": (c_int, [c_vp, c_int, c_vp, c_vp, c_i64, c_int, c_i64, c_vp, c_vp]),
    "dlb_unpermute_bwd": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_i64, c_int, c_i64, c_vp, c_vp, c_vp]),
    "dlb_eplb_map_hash": (c_int, [c_vp, c_int, c_vp, c_vp, c_i64, c_int, c_int, c_int, ctypes.c_uint32, c_vp, c_vp]),
    "dlb_route_softmax_topk": (c_int, [c_vp, c_int, c_i64, c_int, c_int, c_int, c_vp, c_vp, c_int, c_vp]),
    "dlb_route_grouped_topk": (c_int, [c_vp, c_int, c_vp, c_i64, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp]),
    "dlb_topk_gating_workspace_size": (c_sz, [c_i64, c_int, c_int]),
    "dlb_topk_gating_bwd": (c_int, [c_vp, c_sz, c_int, c_i64, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "dlb_topk_gating": (c_int, [c_vp, c_int, c_i64, c_int, c_int, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]),
}

_lib = None
_lock = threading.Lock()


def lib():
    """The loaded extension; raises if it has not been built (no CPU or torch fallback)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(SO_PATH):
                    raise RuntimeError(
                        f"dlblas_b200: CUDA extension {SO_PATH} is missing; build it with "
                        "`python -m dlblas_b200.build` (needs nvcc with sm_100a support)")
                handle = ctypes.CDLL(SO_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(rc: int):
    """Maps a negative return code to the exception type the reference raises in that case:
    bad shapes / dtypes are `assert`s there, so DLB_ERR_INVALID becomes AssertionError."""
    if rc == 0:
        return
    msg = lib().dlb_last_error_string().decode("utf-8", "replace")
    if rc == -1:
        raise AssertionError(msg)
    raise RuntimeError(f"dlblas_b200 error {rc}: {msg}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise AssertionError(f"dlblas_b200: unsupported dtype {dt}") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("dlblas_b200 runs on CUDA tensors only (B200, sm_100a); there is no CPU path")


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the GEMM kernels set when a bounded wait gives up."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device=None):
    """Synchronises and raises if a kernel reported a timed-out barrier wait since the last check."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"dlblas_b200: a GEMM kernel gave up waiting on a barrier (status {v})")


def maybe_check_status(device=None):
    """The layers call this at the end of every forward.  With DLBLAS_CHECK_STATUS=1 it synchronises and raises
    if a bounded wait gave up during the call (at the price of one host synchronisation per layer); by default
    it does nothing and the caller is expected to run `check_status()` at a point of its own choosing."""
    if os.environ.get("DLBLAS_CHECK_STATUS", "0") == "1":
        check_status(device)


def set_wait_policy(limit_cycles: int = 0, withhold_loads: bool = False):
    """Limit of one barrier wait inside the GEMM kernels in SM clock cycles (0 = default, about 2 s);
    `withhold_loads` is the self-test switch of dlb_set_wait_policy."""
    check(lib().dlb_set_wait_policy(int(limit_cycles), 1 if withhold_loads else 0))


def launch_count(reset=False) -> int:
    return int(lib().dlb_launch_count(1 if reset else 0))
