"""`triton_template.gemm_add_layernorm` of the reference (src/triton_template/gemm_add_layernorm.py:126-144);
the module path is kept, the operator runs on the sm_100a GEMM + LayerNorm kernels."""
from stof_b200.fused import matmul_bias_layernorm as triton_matmul_bias_layernorm  # noqa: F401
