"""Post-LN transformer forward passes built from the fused operators: the BERT encoder (reference loop:
src/benchmk_end2end.py:31-88, QKV projection as in src/model-candidate/1-BERT-large.py:17-18), its GPT-2 and T5-encoder
variants (same loop with the tanh GELU, :93-147, or ReLU, :152-208) and the T5 decoder layer (:230-316)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from . import _lib
from .attention import block_attention
from .fused import bias_residual_layernorm, gemm_bias, gemm_bias_act, gemm_bias_residual, gemm_bias_residual_layernorm
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
    """Forward-only encoder.  Per layer five kernel launches:
    QKV GEMM+bias -> block-masked attention reading Q/K/V straight out of the fused QKV activation and
    writing merged heads -> out-proj GEMM+bias+residual+LayerNorm -> FFN1 GEMM+bias+GELU ->
    FFN2 GEMM+bias+residual+LayerNorm (seven with `fuse_layernorm=False`: the two LayerNorms as kernels of their
    own after GEMMs with the bias + residual epilogue).  The block index is built once per mask.
    The tensor `forward` returns is one of the encoder's own buffers: it holds the result until the next forward
    pass (or graph replay) of this encoder; clone it to keep it longer."""

    def __init__(self, layers: List[EncoderWeights], head_num: int, eps: float = 1e-12, gelu: str = "erf",
                 block_m: int = 64, block_n: int = 64, fuse_layernorm: bool = True):
        """`gelu` names the feed-forward activation: "erf" (BERT), "tanh" (GPT-2 `new_gelu`) or "relu" (T5)."""
        self.fuse_layernorm = bool(fuse_layernorm)
        if gelu not in ("erf", "tanh", "relu"):
            raise _lib.StofError(f"encoder: unknown activation {gelu!r}")
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
        # three hidden-state buffers in rotation: while a GEMM writes one, the previous one is still its residual input and the
        # one before that may be the caller's view of the last result
        y_bufs = [self._buf("y0", (B, S, hid), dev), self._buf("y1", (B, S, hid), dev), self._buf("y2", (B, S, hid), dev)]
        assert len(y_bufs) >= 3
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
            if self.fuse_layernorm:
                gemm_bias_residual_layernorm(ctx, w.Wo, w.bo, x, w.g1, w.b1, self.eps, out=y)
            else:
                gemm_bias_residual(ctx, w.Wo, w.bo, x, out=y)
                bias_residual_layernorm(y, None, None, w.g1, w.b1, self.eps, out=y)
            gemm_bias_act(y, w.W1, w.bi1, self.gelu, out=inter)
            z = y_bufs[yi]; yi = (yi + 1) % 3
            if self.fuse_layernorm:
                gemm_bias_residual_layernorm(inter, w.W2, w.bi2, y, w.g2, w.b2, self.eps, out=z)
            else:
                gemm_bias_residual(inter, w.W2, w.bi2, y, out=z)
                bias_residual_layernorm(z, None, None, w.g2, w.b2, self.eps, out=z)
            x = z
        return x

    __call__ = forward

    def capture(self, hidden: torch.Tensor):
        """Records one forward pass on `hidden` (a tensor the caller keeps and refills in place) into a CUDA graph and returns
        `replay() -> output tensor` (the output buffer is reused by every replay).  Two eager passes run first so that every
        buffer, the attention plan and its balanced schedule exist: a captured pass allocates nothing and reads nothing back.
        All launches of a pass then cost one graph launch on the host."""
        if not hidden.is_cuda:
            raise _lib.StofError("capture: hidden must live on the GPU")
        dev = hidden.device
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self.forward(hidden)
            self.forward(hidden)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.forward(hidden)

        def replay():
            graph.replay()
            return out
        replay.graph = graph
        return replay


def gpt2_stack(layers: List[EncoderWeights], head_num: int, eps: float = 1e-5, block_m: int = 64, block_n: int = 64) -> BertEncoder:
    """The reference's GPT-2 loop (src/benchmk_end2end.py:93-147): the same post-LN layer with the tanh-form GELU;
    the caller sets a causal mask."""
    return BertEncoder(layers, head_num, eps, "tanh", block_m, block_n)


def t5_encoder_stack(layers: List[EncoderWeights], head_num: int, eps: float = 1e-5, block_m: int = 64, block_n: int = 64) -> BertEncoder:
    """The encoder half of the reference's T5 loop (src/benchmk_end2end.py:152-208): the same layer with ReLU."""
    return BertEncoder(layers, head_num, eps, "relu", block_m, block_n)


@dataclass
class T5DecoderWeights:
    """One decoder layer: two attention sublayers (suffix _a, _c: Wqkv, bqkv, Wo, bo, g, b) and the feed-forward
    (W1, bi1, W2, bi2, g2, b2)."""
    Wqkv_a: torch.Tensor
    bqkv_a: torch.Tensor
    Wo_a: torch.Tensor
    bo_a: torch.Tensor
    g_a: torch.Tensor
    b_a: torch.Tensor
    Wqkv_c: torch.Tensor
    bqkv_c: torch.Tensor
    Wo_c: torch.Tensor
    bo_c: torch.Tensor
    g_c: torch.Tensor
    b_c: torch.Tensor
    W1: torch.Tensor
    bi1: torch.Tensor
    W2: torch.Tensor
    bi2: torch.Tensor
    g2: torch.Tensor
    b2: torch.Tensor

    @staticmethod
    def from_dict(p: dict, device) -> "T5DecoderWeights":
        names = [f.name for f in T5DecoderWeights.__dataclass_fields__.values()]
        return T5DecoderWeights(**{k: p[k].to(device=device, dtype=torch.float16).contiguous() for k in names})


class T5Decoder(BertEncoder):
    """Decoder layers of the reference's T5 loop (src/benchmk_end2end.py:230-316): masked self-attention, a second
    attention sublayer on the decoder state, and the ReLU feed-forward, each followed by residual + LayerNorm.  Per layer
    seven kernel launches (two QKV GEMMs, two attentions, two out-projections and the second FFN GEMM with the residual + LayerNorm
    epilogue, the first FFN GEMM with ReLU)."""

    def __init__(self, layers: List[T5DecoderWeights], head_num: int, eps: float = 1e-5, block_m: int = 64, block_n: int = 64):
        super().__init__(layers, head_num, eps, "relu", block_m, block_n)

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        if self._index is None:
            raise _lib.StofError("T5Decoder: call set_mask() or set_index() first")
        B, S, hid = hidden.shape
        H = self.head_num
        D = hid // H
        dev = hidden.device
        frp, fci, prp, pci, pbm, lrp, lci = self._index
        qkv = self._buf("qkv", (B, S, 3 * hid), dev)
        ctx = self._buf("ctx", (B, S, hid), dev)
        inter = self._buf("inter", (B, S, self.layers[0].W1.shape[1]), dev)
        ys = [self._buf(f"y{i}", (B, S, hid), dev) for i in range(4)]
        yi = 0

        def attention_sublayer(x, Wqkv, bqkv, Wo, bo, g, b, out):
            gemm_bias(x, Wqkv, bqkv, out=qkv)
            q5 = qkv.view(B, S, 3, H, D)
            q, k, v = (q5[:, :, i].permute(0, 2, 1, 3) for i in range(3))
            block_attention(q, k, v, ctx.view(B, S, H, D).permute(0, 2, 1, 3), frp, fci, prp, pci, pbm, lrp, lci, self.block_m, self.block_n)
            gemm_bias_residual_layernorm(ctx, Wo, bo, x, g, b, self.eps, out=out)
            return out

        x = hidden
        for w in self.layers:
            y = attention_sublayer(x, w.Wqkv_a, w.bqkv_a, w.Wo_a, w.bo_a, w.g_a, w.b_a, ys[yi]); yi = (yi + 1) % 4
            y2 = attention_sublayer(y, w.Wqkv_c, w.bqkv_c, w.Wo_c, w.bo_c, w.g_c, w.b_c, ys[yi]); yi = (yi + 1) % 4
            gemm_bias_act(y2, w.W1, w.bi1, "relu", out=inter)
            z = ys[yi]; yi = (yi + 1) % 4
            gemm_bias_residual_layernorm(inter, w.W2, w.bi2, y2, w.g2, w.b2, self.eps, out=z)
            x = z
        return x

    __call__ = forward
