"""`dlblas.kernels.permute` of the reference: token permutation for MoE training."""
from .moe_triton_kernels import (moe_permute_topk_bwd_op, moe_permute_topk_op_triton, moe_recover_topk_bwd_op_triton,  # noqa: F401
                                 moe_recover_topk_op_triton, permute, unpermute)
