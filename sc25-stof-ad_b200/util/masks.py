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


# Score-mod predicates of the reference's FlexAttention comparison runs (src/util/masks.py:195-234).  They take index
# tensors (or ints) and return a boolean of the broadcast shape; the constants are the reference's.
_FLEX_WINDOW = 256


def _flex_window(q_idx, kv_idx):
    # one-sided: keys up to 256 positions behind the query, and every later key (the reference leaves the causal term out)
    return (q_idx - kv_idx) <= _FLEX_WINDOW


def _flex_global(q_idx, kv_idx):
    def in_bands(i):
        return (i < 32) | ((i >= 96) & (i < 128))
    return in_bands(q_idx) | in_bands(kv_idx)


def flex_sliding_window_mask(b, h, q_idx, kv_idx):
    return _flex_window(q_idx, kv_idx)


def flex_longformer_mask(b, h, q_idx, kv_idx):
    return _flex_window(q_idx, kv_idx) | _flex_global(q_idx, kv_idx)


def flex_bigbird_mask(b, h, q_idx, kv_idx):
    # the "random" part of the reference: query rows that are multiples of 3 (4) attend the keys with kv_idx / 5 == 0
    # (kv_idx / 7 == 0) under true division, i.e. key 0 only
    sprinkled = ((q_idx % 3 == 0) & (kv_idx / 5 == 0)) | ((q_idx % 4 == 0) & (kv_idx / 7 == 0))
    return _flex_window(q_idx, kv_idx) | _flex_global(q_idx, kv_idx) | sprinkled

