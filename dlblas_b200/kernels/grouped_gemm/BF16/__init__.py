"""`dlblas.kernels.grouped_gemm.BF16` of the reference: grouped GEMMs on bf16 / fp16 operands."""
from . import utils  # noqa: F401
from .m_grouped_gemm import m_grouped_gemm  # noqa: F401
from .k_grouped_gemm import k_grouped_gemm  # noqa: F401
