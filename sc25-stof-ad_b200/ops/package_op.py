"""Operator API of the reference (src/ops/package_op.py), backed by the sm_100a kernels.

The row-wise operators return a new merged-head (batch, S, heads*64) tensor.
`block_attn_mask_op(q, k, v, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps)` keeps the reference's contract: forward only,
positional arguments, and the returned tensor IS `q`, overwritten with the attention output
(src/ops/package_op.py:50-68).  Where the reference silently leaves a non-contiguous `q` untouched, this
version raises.
"""
import torch
from torch.autograd import Function

from stof_b200.attention import block_attn_mask as _block_attn_mask_forward
from stof_b200 import rowwise as _rowwise

__all__ = ['rowwise_attn_full_op', 'rowwise_attn_sliding_op', 'rowwise_attn_mask_op', 'block_attn_mask_op']


# result.shape = {batch_size, seq_len, head_num * head_size}, as in the reference (src/ops/package_op.py:10-48)
class RowWise_Attn_Full(Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal=False):
        result = _rowwise.rowwise_attn_full(q.contiguous(), k.contiguous(), v.contiguous(), is_causal)
        ctx.mark_non_differentiable(result)
        return result


class RowWise_Attn_Sliding(Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal, bandwidth):
        result = _rowwise.rowwise_attn_sliding(q.contiguous(), k.contiguous(), v.contiguous(), is_causal, bandwidth)
        ctx.mark_non_differentiable(result)
        return result


class RowWise_Attn_Mask(Function):
    @staticmethod
    def forward(ctx, q, k, v, is_causal, row_mask):
        result = _rowwise.rowwise_attn_mask(q.contiguous(), k.contiguous(), v.contiguous(), is_causal, row_mask.contiguous())
        ctx.mark_non_differentiable(result)
        return result


class Block_Attn_Mask(Function):
    @staticmethod
    def forward(ctx, q, k, v,
                full_row_ptr, full_col_idx,
                part_row_ptr, part_col_idx, part_block_mask,
                load_row_ptr, load_col_idx,
                BLOCK_M, BLOCK_N, num_warps):
        _block_attn_mask_forward(q, k, v,
                                 full_row_ptr.contiguous(), full_col_idx.contiguous(),
                                 part_row_ptr.contiguous(), part_col_idx.contiguous(), part_block_mask,
                                 load_row_ptr.contiguous(), load_col_idx.contiguous(),
                                 BLOCK_M, BLOCK_N, num_warps)
        ctx.mark_non_differentiable(q)
        return q


rowwise_attn_full_op = RowWise_Attn_Full.apply
rowwise_attn_sliding_op = RowWise_Attn_Sliding.apply
rowwise_attn_mask_op = RowWise_Attn_Mask.apply
block_attn_mask_op = Block_Attn_Mask.apply
