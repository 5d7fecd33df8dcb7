"""`util.masks` of the reference (src/util/masks.py): mask generators and `get_sparse_storage`, the latter
computed by the CUDA compaction kernels."""
from functools import lru_cache

from stof_b200.masks import (generate_bigbird_mask, generate_causal_mask, generate_dilated_mask,  # noqa: F401
                             generate_longformer_mask, generate_sliding_mask, get_sparse_storage)


@lru_cache
def create_block_mask_cached(score_mod, B, H, M, N, device="cuda"):
    """FlexAttention block mask used by the reference's comparison baselines (src/util/masks.py:190-193)."""
    from torch.nn.attention.flex_attention import create_block_mask
    return create_block_mask(score_mod, B, H, M, N, device=device)


def flex_causal_mask(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx
