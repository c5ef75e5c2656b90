"""`dlblas.kernels.grouped_gemm` of the reference."""
