"""`triton_template.add_layernorm` of the reference (src/triton_template/add_layernorm.py:86-107)."""
from stof_b200.fused import batched_bias_layernorm as triton_batched_bias_layernorm  # noqa: F401
