"""Drop-in for the reference's extension module `rowwise_attn_sliding` (src/ops/src/rowwise_attn_sliding.cpp):
`forward(q, k, v, is_causal, result, band_width)`."""
from stof_b200.rowwise import rowwise_attn_sliding as _impl


def forward(q, k, v, is_causal, result, band_width):
    return _impl(q, k, v, is_causal, band_width, result)
