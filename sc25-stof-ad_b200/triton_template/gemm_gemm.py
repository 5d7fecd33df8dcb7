"""`triton_template.gemm_gemm` of the reference (src/triton_template/gemm_gemm.py:158-174)."""
from stof_b200.fused import matmul_gelu_matmul as triton_matmul_batch  # noqa: F401
