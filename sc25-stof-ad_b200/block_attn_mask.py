"""Drop-in for the reference's compiled extension module `block_attn_mask`
(src/ops/src/block_attn_mask.cpp:52-56): `forward(...)` overwrites `q` with the output."""
from stof_b200.attention import block_attn_mask as forward  # noqa: F401
