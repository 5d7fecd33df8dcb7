"""Oracle (test infrastructure): masked multi-head attention on CPU.

Restates the reference's PyTorch-native attention and the semantics of its
block-wise / row-wise kernels with plain CPU PyTorch.  Nothing in the shipped
CUDA path imports this file.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def torch_attn_std(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(Q K^T / sqrt(D) - 10000 (1 - mask)) V in the dtype of the inputs
    (src/correct_verify_attn.py:19-30).  q/k/v (B,H,S,D); mask (B or 1,S,S) of 0/1."""
    scores = torch.matmul(q, k.transpose(-2, -1))
    scores = scores / (q.shape[-1] ** .5)
    if mask is not None:
        scores = scores - 10000.0 * (1.0 - mask.unsqueeze(1))
    probs = torch.nn.functional.softmax(scores, dim=-1)
    return torch.matmul(probs, v)


def masked_attention_fp32(q, k, v, mask) -> torch.Tensor:
    """The same path evaluated in fp32 from (possibly fp16) inputs; the parity
    target for the CUDA kernel (tolerance 2e-3 max-abs)."""
    m = None if mask is None else torch.as_tensor(np.asarray(mask, dtype=np.float32)) if not torch.is_tensor(mask) else mask.float()
    return torch_attn_std(q.float(), k.float(), v.float(), m)


def block_attention_from_index(q, k, v, st, bm: int, bn: int, out_dtype=torch.float32) -> torch.Tensor:
    """Semantics of the reference block-wise kernel
    (src/ops/src/block_attn_mask_cuda.cu:3526-3799, e.g. the 4-warp n64 variant):
    for every row block only the column blocks listed in `load_col_idx` take part;
    a partial block adds its fp16 tile to the UNSCALED scores (:3680-3690) before
    the 1/sqrt(D) scale inside the softmax (:3695, :193).  Evaluated in fp32; a row
    block without any listed column yields zeros.  `st` is an oracle SparseStorage
    (or any object with the same fields as numpy arrays / tensors)."""
    q32, k32, v32 = q.float(), k.float(), v.float()
    B, H, S, D = q32.shape
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, H, S, D, dtype=torch.float32)
    frp, fci = np.asarray(st.full_row_ptr), np.asarray(st.full_col_idx)
    prp, pci = np.asarray(st.part_row_ptr), np.asarray(st.part_col_idx)
    pbm = torch.as_tensor(np.asarray(st.part_block_mask, dtype=np.float32))
    for r in range(S // bm):
        cols, adds = [], []
        for c in fci[frp[r]:frp[r + 1]]:
            cols.append(int(c)); adds.append(None)
        for p in range(prp[r], prp[r + 1]):
            cols.append(int(pci[p])); adds.append(pbm[p])
        if not cols:
            continue
        order = np.argsort(cols, kind="stable")
        qr = q32[:, :, r * bm:(r + 1) * bm]
        s_list = []
        for o in order:
            c = cols[o]
            s = torch.matmul(qr, k32[:, :, c * bn:(c + 1) * bn].transpose(-2, -1))
            if adds[o] is not None:
                s = s + adds[o]
            s_list.append(s * scale)
        s_all = torch.cat(s_list, dim=-1)
        p_all = torch.softmax(s_all, dim=-1)
        v_all = torch.cat([v32[:, :, cols[o] * bn:(cols[o] + 1) * bn] for o in order], dim=2)
        out[:, :, r * bm:(r + 1) * bm] = torch.matmul(p_all, v_all)
    return out.to(out_dtype)


def merge_heads(o: torch.Tensor) -> torch.Tensor:
    """(B,H,S,D) -> (B,S,H*D), the layout the row-wise operators return
    (src/ops/src/rowwise_attn_full_cuda.cu:42)."""
    B, H, S, D = o.shape
    return o.permute(0, 2, 1, 3).reshape(B, S, H * D)


def rowwise_full(q, k, v, is_causal: bool) -> torch.Tensor:
    """Dense or causal softmax(QK^T/sqrt(D))V in merged-head layout
    (src/ops/src/rowwise_attn_full_cuda.cu:20-136), fp32."""
    S = q.shape[2]
    mask = torch.tril(torch.ones(S, S)) if is_causal else torch.ones(S, S)
    return merge_heads(_softmax_where(q, k, v, mask.bool()))


def rowwise_sliding(q, k, v, is_causal: bool, band_width: int) -> torch.Tensor:
    """Keys with row-band_width < col <= (row if causal else S-1)
    (src/ops/src/rowwise_attn_sliding_cuda.cu:37,44), fp32, merged heads."""
    S = q.shape[2]
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    allowed = (j > i - band_width) & (j <= (i if is_causal else S - 1))
    return merge_heads(_softmax_where(q, k, v, allowed))


def rowwise_mask(q, k, v, is_causal: bool, row_mask) -> torch.Tensor:
    """Keys with row_mask[row, col] > 0 and col <= (row if causal else S-1)
    (src/ops/src/rowwise_attn_mask_cuda.cu:55-58), fp32, merged heads."""
    S = q.shape[2]
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    allowed = (torch.as_tensor(row_mask).float() > 0) & (j <= (i if is_causal else S - 1))
    return merge_heads(_softmax_where(q, k, v, allowed))


def _softmax_where(q, k, v, allowed: torch.Tensor) -> torch.Tensor:
    q32, k32, v32 = q.float(), k.float(), v.float()
    s = torch.matmul(q32, k32.transpose(-2, -1)) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)          # rows without any allowed key give zeros
    return torch.matmul(p, v32)


def attention_flops(load_blocks: int, bm: int, bn: int, d: int, batch_heads: int) -> float:
    """Effective FLOPs: 2*bm*bn*d for QK^T plus the same for PV per listed block."""
    return float(batch_heads) * load_blocks * 4.0 * bm * bn * d
