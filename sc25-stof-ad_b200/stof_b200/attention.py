"""Block-masked multi-head attention (host side of `stof_block_attn`)."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch

from . import _lib


_PLAN_CACHE = OrderedDict()
_PLAN_CACHE_MAX = 16


def attention_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, seq_len: int, block_m: int, block_n: int):
    """Kernel-side plan of a block index (`stof_block_attn_plan`), cached per index: the key holds the four
    index tensors themselves (their storage cannot be recycled while the entry lives) and their versions."""
    tensors = (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx)
    key = tuple((t.data_ptr(), t._version, t.numel()) for t in tensors) + (seq_len, block_m, block_n, str(full_row_ptr.device))
    hit = _PLAN_CACHE.get(key)
    if hit is not None:
        _PLAN_CACHE.move_to_end(key)
        return hit[0]
    dev = full_row_ptr.device
    L = _lib.lib()
    nbytes = int(L.stof_block_attn_plan_bytes(seq_len, block_m, block_n))
    with torch.cuda.device(dev):
        plan = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        rc = L.stof_block_attn_plan(_lib.ptr(full_row_ptr), _lib.ptr(full_col_idx), _lib.ptr(part_row_ptr), _lib.ptr(part_col_idx),
                                    seq_len, int(block_m), int(block_n), _lib.ptr(plan), nbytes, _lib.ptr(_lib.status_word(dev)),
                                    _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_block_attn_plan")
    _PLAN_CACHE[key] = (plan, tensors)
    while len(_PLAN_CACHE) > _PLAN_CACHE_MAX:
        _PLAN_CACHE.popitem(last=False)
    return plan


def block_attention(q, k, v, out, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                    load_row_ptr, load_col_idx, block_m: int, block_n: int, num_warps: int = 4, softmax_scale=None):
    """Runs the attention kernel on (B,H,S,64)-shaped *views*: q, k, v and out may be arbitrary
    strided views with a contiguous last dimension (for instance slices of a fused (B,S,3*hidden)
    QKV activation permuted to (B,H,S,64), or a merged-head (B,S,hidden) output viewed the same
    way), so no transposing copy is needed around the kernel.  `out` may be `q` itself.
    `load_row_ptr` / `load_col_idx` are accepted for signature compatibility (they are the merge of
    the full and partial lists, which is what the kernel's plan is built from)."""
    _lib.require_cuda(q, k, v, out, full_row_ptr, part_row_ptr)
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16 or out.dtype != torch.float16:
        raise _lib.StofError("block attention expects float16 q/k/v/out")
    B, H, S, D = q.shape
    if k.shape != q.shape or v.shape != q.shape or out.shape != q.shape:
        raise _lib.StofError("block attention: q, k, v and out must share one (B,H,S,D) shape")
    for t in (q, k, v, out):
        if t.stride(3) != 1:
            raise _lib.StofError("block attention: the head dimension must be contiguous")
    for t in (full_row_ptr, full_col_idx, part_row_ptr, part_col_idx):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise _lib.StofError("block attention: index tensors must be contiguous int32")
    if full_row_ptr.numel() != S // block_m + 1 or part_row_ptr.numel() != S // block_m + 1:
        raise _lib.StofError("block attention: row pointer arrays must have S / BLOCK_M + 1 entries")
    if part_block_mask is not None and (part_block_mask.dtype != torch.float16 or not part_block_mask.is_contiguous()):
        raise _lib.StofError("block attention: part_block_mask must be contiguous float16")
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else float(softmax_scale)   # src/ops/src/block_attn_mask.cpp:32
    dev = q.device
    L = _lib.lib()
    plan = attention_plan(full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, S, int(block_m), int(block_n))
    with torch.cuda.device(dev):
        st = _lib.status_word(dev)
        rc = L.stof_block_attn(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), B, H, S, D,
                               _lib.strides3(q.stride()[:3]), _lib.strides3(k.stride()[:3]),
                               _lib.strides3(v.stride()[:3]), _lib.strides3(out.stride()[:3]),
                               _lib.ptr(part_row_ptr), _lib.ptr(part_block_mask), _lib.ptr(plan),
                               int(block_m), int(block_n), int(num_warps), scale, _lib.ptr(st), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_block_attn")
    return out


def block_attn_mask(q, k, v, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                    load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps):
    """Semantics of the reference extension's `block_attn_mask.forward`
    (src/ops/src/block_attn_mask.cpp:17-49): overwrites `q` with the attention output."""
    if not q.is_contiguous():
        raise _lib.StofError("block_attn_mask: q must be contiguous (it is overwritten in place)")
    return block_attention(q, k.contiguous(), v.contiguous(), q, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx,
                           part_block_mask.contiguous(), load_row_ptr, load_col_idx, BLOCK_M, BLOCK_N, num_warps)
