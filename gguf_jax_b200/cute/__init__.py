"""Drop-in alias of the reference's optional ``gguf_jax.cute`` package
(src/gguf_jax/cute/__init__.py): the same nine names, served by the CUDA kernels."""
from ..kernels import (LOWBIT_TYPES, dequantize_q4_k, gemm_q4_k, matmul_iq4_xs, matmul_lowbit,
                       matmul_q4_k, matmul_q5_k, matmul_q6_k, register)

__all__ = [
    "LOWBIT_TYPES",
    "dequantize_q4_k",
    "gemm_q4_k",
    "matmul_iq4_xs",
    "matmul_lowbit",
    "matmul_q4_k",
    "matmul_q5_k",
    "matmul_q6_k",
    "register",
]
