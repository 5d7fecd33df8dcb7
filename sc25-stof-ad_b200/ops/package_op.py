"""Operator API of the reference (src/ops/package_op.py), backed by the sm_100a kernels.

`block_attn_mask_op(q, k, v, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps)` keeps the reference's contract: forward only,
positional arguments, and the returned tensor IS `q`, overwritten with the attention output
(src/ops/package_op.py:50-68).  Where the reference silently leaves a non-contiguous `q` untouched, this
version raises.
"""
import torch
from torch.autograd import Function

from stof_b200.attention import block_attn_mask as _block_attn_mask_forward

__all__ = ['block_attn_mask_op']


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


block_attn_mask_op = Block_Attn_Mask.apply
