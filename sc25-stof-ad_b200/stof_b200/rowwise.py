"""Row-wise attention operators of the reference (`rowwise_attn_{full,sliding,mask}_op`,
src/ops/package_op.py:11-48), expressed on the block-masked tensor-core kernel.

The reference runs one warp per (query row, head) with scalar dot products
(src/ops/src/rowwise_attn_full_cuda.cu:20-136, rowwise_attn_sliding_cuda.cu:14-71,
rowwise_attn_mask_cuda.cu:31-86).  Here the key set of each variant is written as a 0/1 mask, compacted
once into a block index by the CUDA compaction (cached per shape and parameters, or per caller mask), and the attention
itself runs in `stof_block_attn`, which writes the merged-head (batch, S, heads*64) layout directly
through its output strides.  All heads are computed (the reference's sliding and mask launchers skip
the trailing heads when the head count is not a multiple of 3).  A row that admits no key at all is
undefined in the reference (it divides 0 by 0); here it yields zeros or, inside partially listed blocks, the
average over that row's masked keys.
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from . import _lib
from .attention import block_attention
from .masks import get_sparse_storage

_INDEX_CACHE = OrderedDict()
_INDEX_CACHE_MAX = 32


def _block_size(seq_len: int, element_granular: bool = True) -> int:
    """Index granularity: element-granular key sets (bands, causal edges, caller masks) run fastest with 32 x 32 blocks
    (fewer 16 x 16 groups need the mask add than with 64 x 64, as fast as 16 x 16 with a quarter of the index), block-aligned
    ones with the coarsest index (see `selector`)."""
    for b in ((32, 16) if element_granular else (64, 32, 16)):
        if seq_len % b == 0:
            return b
    raise _lib.StofError(f"row-wise attention: seq_len {seq_len} must be a multiple of 16")


def _cached_index(key, build_mask, element_granular=True, keep_alive=None):
    """Block index for a key set, built once per key.  `keep_alive` is stored with the entry: a key that names a caller's
    tensor by address and version stays valid for as long as that tensor cannot be freed."""
    hit = _INDEX_CACHE.get(key)
    if hit is not None:
        _INDEX_CACHE.move_to_end(key)
        return hit[0]
    mask = build_mask()
    blk = _block_size(mask.shape[-1], element_granular)
    idx = (blk,) + tuple(get_sparse_storage(mask, blk, blk)[1:])
    _INDEX_CACHE[key] = (idx, keep_alive)
    while len(_INDEX_CACHE) > _INDEX_CACHE_MAX:
        _INDEX_CACHE.popitem(last=False)
    return idx


def _run(q, k, v, index, result=None):
    _lib.require_cuda(q, k, v)
    B, H, S, D = q.shape
    if result is None:
        result = torch.empty(B, S, H * D, dtype=q.dtype, device=q.device)
    elif tuple(result.shape) != (B, S, H * D) or not result.is_contiguous():
        raise _lib.StofError("row-wise attention: result must be a contiguous (batch, S, heads*64) tensor")
    blk = index[0]
    out_view = result.view(B, S, H, D).permute(0, 2, 1, 3)              # (B,H,S,D) view of the merged-head buffer
    block_attention(q, k, v, out_view, *index[1:], blk, blk)
    return result


def _key_range_mask(seq_len, device, lower_exclusive, causal):
    """0/1 fp16 (1,S,S): col > row - lower_exclusive (None = no lower bound) and col <= (row if causal else S-1)."""
    i = torch.arange(seq_len, device=device)[:, None]
    j = torch.arange(seq_len, device=device)[None, :]
    allowed = torch.ones(seq_len, seq_len, dtype=torch.bool, device=device)
    if lower_exclusive is not None:
        allowed &= j > i - lower_exclusive
    if causal:
        allowed &= j <= i
    return allowed.to(torch.float16).unsqueeze(0)


def rowwise_attn_full(q, k, v, is_causal=False, result=None):
    """softmax(QK^T / sqrt(64)) V over all keys, or keys <= row when causal; merged-head output."""
    S = q.shape[2]
    key = ("full", S, bool(is_causal), str(q.device))
    index = _cached_index(key, lambda: _key_range_mask(S, q.device, None, bool(is_causal)), element_granular=bool(is_causal))
    return _run(q, k, v, index, result)


def rowwise_attn_sliding(q, k, v, is_causal, bandwidth, result=None):
    """Keys with row - bandwidth < col <= (row if causal else S-1) (src/ops/src/rowwise_attn_sliding_cuda.cu:37,44)."""
    S = q.shape[2]
    key = ("sliding", S, bool(is_causal), int(bandwidth), str(q.device))
    index = _cached_index(key, lambda: _key_range_mask(S, q.device, int(bandwidth), bool(is_causal)))
    return _run(q, k, v, index, result)


def rowwise_attn_mask(q, k, v, is_causal, row_mask, result=None):
    """Keys with row_mask[row, col] > 0 and col <= (row if causal else S-1) (src/ops/src/rowwise_attn_mask_cuda.cu:55-58).
    `row_mask` is a dense (S, S) tensor.  Its block index is cached under the tensor's address and version counter (the
    entry keeps the tensor alive), so a loop that passes the same mask pays for the compaction once; an in-place change
    of the mask bumps the version and rebuilds the index."""
    S = q.shape[2]

    def build():
        allowed = row_mask.reshape(S, S) > 0
        if is_causal:
            allowed = allowed & torch.ones(S, S, dtype=torch.bool, device=allowed.device).tril()
        return allowed.to(device=q.device, dtype=torch.float16).unsqueeze(0)

    key = ("mask", S, bool(is_causal), row_mask.data_ptr(), row_mask._version, tuple(row_mask.shape), tuple(row_mask.stride()),
           str(row_mask.dtype), str(row_mask.device), str(q.device))
    index = _cached_index(key, build, keep_alive=row_mask)
    return _run(q, k, v, index, result)
