"""Drop-in for the reference's extension module `rowwise_attn_mask` (src/ops/src/rowwise_attn_mask.cpp):
`forward(q, k, v, is_causal, result, row_mask)`."""
from stof_b200.rowwise import rowwise_attn_mask as _impl


def forward(q, k, v, is_causal, result, row_mask):
    return _impl(q, k, v, is_causal, row_mask, result)
