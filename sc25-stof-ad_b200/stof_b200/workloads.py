"""Synthetic workloads with the shapes, seeds and mask recipes of the benchmark configurations.

The reference measures on random tensors only; these are seeded stand-ins generated on the CPU
(device RNG streams differ between GPUs) and copied to the device.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def block_sliding(nb: int, w: int) -> torch.Tensor:
    i = torch.arange(nb)
    return ((i[:, None] - i[None, :]).abs() <= w).float()


def block_bigbird(nb: int, seed: int) -> torch.Tensor:
    """3 sliding + 2 global block rows/cols + 3 random blocks per row (`torch.randperm(nb)[:3]`, one CPU
    generator seeded `seed`, rows in order)."""
    bm = block_sliding(nb, 1)
    bm[:2, :] = 1
    bm[:, :2] = 1
    g = torch.Generator().manual_seed(seed)
    for r in range(nb):
        bm[r, torch.randperm(nb, generator=g)[:3]] = 1
    return bm


def block_longformer_dilated(nb: int) -> torch.Tensor:
    """Window of +-4 blocks taking every other block (+-256 tokens dilated by 2 at block 64) plus block
    row/col 0 (the first 64 tokens) global."""
    i = torch.arange(nb)
    d = i[:, None] - i[None, :]
    bm = ((d.abs() <= 4) & (d % 2 == 0)).float()
    bm[0, :] = 1
    bm[:, 0] = 1
    return bm


def expand_block_mask(bm: torch.Tensor, blk: int = 64, dtype=torch.float16) -> torch.Tensor:
    """(nb, nb) block matrix -> (1, S, S) element mask."""
    return torch.kron(bm, torch.ones(blk, blk)).to(dtype).unsqueeze(0)


@dataclass(frozen=True)
class AttentionConfig:
    name: str
    batch: int
    heads: int
    seq_len: int
    seed: int
    mask: str          # recipe name
    head_dim: int = 64
    block: int = 64


@dataclass(frozen=True)
class EncoderConfig:
    name: str
    batch: int
    seq_len: int
    hidden: int
    heads: int
    ffn: int
    layers: int
    seed: int
    mask: str
    eps: float = 1e-12
    block: int = 64


ATTENTION_CONFIGS = {
    "cfg1": AttentionConfig("mha_sliding_b1_h12_s256", 1, 12, 256, 0, "sliding1"),
    "cfg2": AttentionConfig("mha_bigbird_b16_h12_s2048", 16, 12, 2048, 1, "bigbird"),
    "cfg3": AttentionConfig("mha_longformer_dilated_b8_h16_s4096", 8, 16, 4096, 2, "longformer_dilated"),
}
ENCODER_CONFIGS = {
    "cfg4": EncoderConfig("bert_base_layer_b16_s1024", 16, 1024, 768, 12, 3072, 1, 3, "sliding2"),
    "cfg5": EncoderConfig("bert_large_24l_b64_s4096", 64, 4096, 1024, 16, 4096, 24, 4, "bigbird"),
}


def block_matrix(recipe: str, nb: int, seed: int) -> torch.Tensor:
    if recipe == "sliding1":
        return block_sliding(nb, 1)
    if recipe == "sliding2":
        return block_sliding(nb, 2)
    if recipe == "bigbird":
        return block_bigbird(nb, seed)
    if recipe == "longformer_dilated":
        return block_longformer_dilated(nb)
    raise KeyError(recipe)


def config_mask(cfg) -> torch.Tensor:
    """(1, S, S) fp16 element mask of a configuration (CPU tensor)."""
    return expand_block_mask(block_matrix(cfg.mask, cfg.seq_len // cfg.block, cfg.seed), cfg.block)


def attention_inputs(cfg: AttentionConfig, batch_slice=None):
    """q, k, v ~ N(0,1) drawn in fp32 from one CPU generator seeded cfg.seed (order q, k, v), cast to fp16.
    `batch_slice=(lo, hi)` returns only those batch entries of the same global draw."""
    g = torch.Generator().manual_seed(cfg.seed)
    shape = (cfg.batch, cfg.heads, cfg.seq_len, cfg.head_dim)
    out = []
    for _ in range(3):
        t = torch.randn(shape, generator=g).half()
        out.append(t if batch_slice is None else t[batch_slice[0]:batch_slice[1]].contiguous())
    return tuple(out)


def encoder_weights(cfg: EncoderConfig):
    """Per layer W ~ N(0, 0.02), biases 0, gamma 1, beta 0; one CPU generator seeded cfg.seed, draw order
    Wqkv, Wo, W1, W2 per layer (the constant terms consume no random numbers)."""
    g = torch.Generator().manual_seed(cfg.seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).half()

    layers = []
    for _ in range(cfg.layers):
        h, f = cfg.hidden, cfg.ffn
        layers.append({
            "Wqkv": w(h, 3 * h), "bqkv": torch.zeros(3 * h).half(), "Wo": w(h, h), "bo": torch.zeros(h).half(),
            "g1": torch.ones(h).half(), "b1": torch.zeros(h).half(), "W1": w(h, f), "bi1": torch.zeros(f).half(),
            "W2": w(f, h), "bi2": torch.zeros(h).half(), "g2": torch.ones(h).half(), "b2": torch.zeros(h).half()})
    return layers


def encoder_input(cfg: EncoderConfig, batch_slice=None, seed_offset: int = 1000):
    """Hidden states ~ N(0,1), fp16, from a CPU generator seeded cfg.seed + seed_offset; generated per
    sequence so that a batch slice costs only its own memory."""
    lo, hi = (0, cfg.batch) if batch_slice is None else batch_slice
    out = torch.empty(hi - lo, cfg.seq_len, cfg.hidden, dtype=torch.float16)
    for b in range(lo, hi):
        g = torch.Generator().manual_seed(cfg.seed + seed_offset + b)
        out[b - lo] = torch.randn(cfg.seq_len, cfg.hidden, generator=g).half()
    return out


def attention_flops(n_load_blocks: int, batch: int, heads: int, bm: int = 64, bn: int = 64, d: int = 64) -> float:
    """Effective FLOPs: 4*bm*bn*d per listed block (QK^T and PV), times batch*heads."""
    return float(batch) * heads * n_load_blocks * 4.0 * bm * bn * d


def encoder_flops(cfg: EncoderConfig, n_load_blocks: int, batch: int) -> float:
    tokens = batch * cfg.seq_len
    gemm = 2.0 * tokens * cfg.hidden * (3 * cfg.hidden + cfg.hidden + 2 * cfg.ffn)
    return cfg.layers * (gemm + attention_flops(n_load_blocks, batch, cfg.heads, cfg.block, cfg.block, cfg.hidden // cfg.heads))
