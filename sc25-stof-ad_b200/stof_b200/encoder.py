"""Post-LN BERT encoder forward built from the fused operators
(reference loop: src/benchmk_end2end.py:31-88, QKV projection as in src/model-candidate/1-BERT-large.py:17-18)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from . import _lib
from .attention import block_attention
from .fused import bias_residual_layernorm, gemm_bias, gemm_bias_gelu, gemm_bias_residual
from .masks import get_sparse_storage


@dataclass
class EncoderWeights:
    """One layer: Wqkv (hid,3hid), bqkv, Wo (hid,hid), bo, g1, b1, W1 (hid,ffn), bi1, W2 (ffn,hid), bi2, g2, b2."""
    Wqkv: torch.Tensor
    bqkv: torch.Tensor
    Wo: torch.Tensor
    bo: torch.Tensor
    g1: torch.Tensor
    b1: torch.Tensor
    W1: torch.Tensor
    bi1: torch.Tensor
    W2: torch.Tensor
    bi2: torch.Tensor
    g2: torch.Tensor
    b2: torch.Tensor

    @staticmethod
    def from_dict(p: dict, device) -> "EncoderWeights":
        return EncoderWeights(**{k: p[k].to(device=device, dtype=torch.float16).contiguous() for k in
                                 ("Wqkv", "bqkv", "Wo", "bo", "g1", "b1", "W1", "bi1", "W2", "bi2", "g2", "b2")})


class BertEncoder:
    """Forward-only encoder.  Per layer six kernel launches:
    QKV GEMM+bias -> block-masked attention reading Q/K/V straight out of the fused QKV activation and
    writing merged heads -> out-proj GEMM+bias+residual -> LayerNorm -> FFN1 GEMM+bias+GELU ->
    FFN2 GEMM+bias+residual -> LayerNorm.  The block index is built once per mask."""

    def __init__(self, layers: List[EncoderWeights], head_num: int, eps: float = 1e-12, gelu: str = "erf",
                 block_m: int = 64, block_n: int = 64):
        self.layers = layers
        self.head_num = head_num
        self.eps = eps
        self.gelu = gelu
        self.block_m, self.block_n = block_m, block_n
        self._index = None
        self._bufs = {}

    def set_mask(self, mask: torch.Tensor):
        """mask: (1 or B, S, S) 0/1; only mask[0] defines the block index, as in the reference."""
        self._index = get_sparse_storage(mask, self.block_m, self.block_n)[1:]
        return self._index

    def set_index(self, index):
        """index: (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask, load_row_ptr, load_col_idx)."""
        self._index = tuple(index)

    def _buf(self, name, shape, device):
        key = (name, tuple(shape), str(device))
        if key not in self._bufs:
            self._bufs[key] = torch.empty(shape, dtype=torch.float16, device=device)
        return self._bufs[key]

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        if self._index is None:
            raise _lib.StofError("BertEncoder: call set_mask() or set_index() first")
        B, S, hid = hidden.shape
        H = self.head_num
        D = hid // H
        dev = hidden.device
        frp, fci, prp, pci, pbm, lrp, lci = self._index
        x = hidden
        qkv = self._buf("qkv", (B, S, 3 * hid), dev)
        ctx = self._buf("ctx", (B, S, hid), dev)
        ffn = self.layers[0].W1.shape[1]
        inter = self._buf("inter", (B, S, ffn), dev)
        y_bufs = [self._buf("y0", (B, S, hid), dev), self._buf("y1", (B, S, hid), dev), self._buf("y2", (B, S, hid), dev)]
        yi = 0
        for w in self.layers:
            gemm_bias(x, w.Wqkv, w.bqkv, out=qkv)
            q5 = qkv.view(B, S, 3, H, D)
            q = q5[:, :, 0].permute(0, 2, 1, 3)
            k = q5[:, :, 1].permute(0, 2, 1, 3)
            v = q5[:, :, 2].permute(0, 2, 1, 3)
            o = ctx.view(B, S, H, D).permute(0, 2, 1, 3)
            block_attention(q, k, v, o, frp, fci, prp, pci, pbm, lrp, lci, self.block_m, self.block_n)
            y = y_bufs[yi]; yi = (yi + 1) % 3
            gemm_bias_residual(ctx, w.Wo, w.bo, x, out=y)
            bias_residual_layernorm(y, None, None, w.g1, w.b1, self.eps, out=y)
            gemm_bias_gelu(y, w.W1, w.bi1, self.gelu, out=inter)
            z = y_bufs[yi]; yi = (yi + 1) % 3
            gemm_bias_residual(inter, w.W2, w.bi2, y, out=z)
            bias_residual_layernorm(z, None, None, w.g2, w.b2, self.eps, out=z)
            x = z
        return x

    __call__ = forward
