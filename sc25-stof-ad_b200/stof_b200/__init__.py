"""stof_b200 -- host side of the B200 (sm_100a) kernels behind the STOF operator API.

PyTorch supplies device memory, streams and (for multi-GPU runs) process groups; every
computation of the two accelerated paths runs in the hand-written CUDA kernels of
`libstof_b200.so`, reached through its C ABI with ctypes.  There is no CPU or library
fallback: if the shared library is missing or a tensor is not on a CUDA device that can
be used, the call raises.
"""
from ._lib import StofError, lib, library_path  # noqa: F401
from .masks import (get_sparse_storage, SparseStorageRefresher, generate_causal_mask, generate_sliding_mask, generate_dilated_mask,  # noqa: F401
                    generate_longformer_mask, generate_bigbird_mask)
from .attention import block_attn_mask, block_attention, block_attention_host, HostAttentionPipeline  # noqa: F401
from .selector import GPUParams, BLOCK_WISE_CONFIGS, select_operator, select_block_size  # noqa: F401
from .rowwise import rowwise_attn_full, rowwise_attn_sliding, rowwise_attn_mask  # noqa: F401
from .fused import (gemm_bias, gemm_bias_gelu, gemm_bias_relu, gemm_bias_act, gemm_bias_residual, gemm_bias_residual_layernorm, gemm_bias_residual_then_layernorm, bias_residual_layernorm,  # noqa: F401
                    matmul_bias_layernorm, matmul_gelu_matmul, batched_bias_layernorm)
from .encoder import BertEncoder, EncoderWeights, T5Decoder, T5DecoderWeights, gpt2_stack, t5_encoder_stack  # noqa: F401
