"""Mask generators and the CUDA mask -> block-index compaction.

Mirrors the interface of the reference's `src/util/masks.py` (same names, argument meaning and
return tuple) for the functions on the accelerated path.
"""
from __future__ import annotations

import random

import torch

from . import _lib


# ------------------------------------------------------------------------------------------
# get_sparse_storage (reference: src/util/masks.py:125-184)
# ------------------------------------------------------------------------------------------
def get_sparse_storage(Mask: torch.Tensor, block_size_m: int, block_size_n: int):
    """Block-CSR index of `Mask[0]`, computed by the CUDA compaction kernels.

    Returns `(nnz, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
    load_row_ptr, load_col_idx)` exactly as the reference: int32 index tensors on the mask's
    device, fp16 partial tiles -10000*(1-m) (a single tile of ones when there is no partial
    block), `nnz` a 0-dim float tensor = 100 * count_nonzero(whole tensor) / S^2.
    A mask living on the CPU is copied to the current CUDA device and the results are copied
    back; the computation itself always runs on the GPU.
    """
    if Mask.dim() != 3 or Mask.shape[-1] != Mask.shape[-2]:
        raise _lib.StofError("get_sparse_storage expects a (batch, S, S) mask")
    if Mask.dtype not in (torch.float16, torch.float32):
        raise _lib.StofError(f"get_sparse_storage: mask dtype {Mask.dtype} unsupported (float16 or float32)")
    home = Mask.device
    m = Mask if Mask.is_cuda else Mask.cuda()
    m = m.contiguous()
    dev = m.device
    B, S = m.shape[0], m.shape[-1]
    bm, bn = int(block_size_m), int(block_size_n)
    L = _lib.lib()
    dt = _lib.STOF_DTYPE_F16 if m.dtype == torch.float16 else _lib.STOF_DTYPE_F32
    if S % bm or S % bn:
        raise _lib.StofError(f"get_sparse_storage: S={S} must be a multiple of the block sizes ({bm}, {bn})")
    nbm = S // bm
    with torch.cuda.device(dev):
        stream = _lib.current_stream_ptr(dev)
        ws_bytes = int(L.stof_mask_workspace_bytes(S, bm, bn))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        row_ptrs = torch.empty(3, nbm + 1, dtype=torch.int32, device=dev)
        counts = torch.empty(4, dtype=torch.int64, device=dev)
        _lib.check(L.stof_mask_classify(_lib.ptr(m), dt, B, S, bm, bn, _lib.ptr(row_ptrs[0]), _lib.ptr(row_ptrs[1]),
                                        _lib.ptr(row_ptrs[2]), _lib.ptr(counts), _lib.ptr(ws), ws_bytes, stream),
                   "stof_mask_classify")
        n_full, n_part, n_load, nnz_elems = counts.tolist()          # the one host read: output sizes depend on the data
        _lib.check_status(dev, "a kernel launched before this get_sparse_storage")   # the stream is drained here anyway
        full_col = torch.empty(n_full, dtype=torch.int32, device=dev)
        part_col = torch.empty(n_part, dtype=torch.int32, device=dev)
        load_col = torch.empty(n_load, dtype=torch.int32, device=dev)
        tiles = torch.empty(n_part, bm, bn, dtype=torch.float16, device=dev) if n_part else None
        _lib.check(L.stof_mask_fill(_lib.ptr(m), dt, S, bm, bn, _lib.ptr(row_ptrs[0]), _lib.ptr(row_ptrs[1]), _lib.ptr(row_ptrs[2]),
                                    _lib.ptr(full_col), _lib.ptr(part_col), _lib.ptr(load_col), _lib.ptr(tiles),
                                    _lib.ptr(ws), ws_bytes, stream), "stof_mask_fill")
        if tiles is None:
            tiles = torch.ones(1, bm, bn, dtype=torch.float16, device=dev)
        # same operation order as the reference: int64 count -> / S^2 -> * 100, in float32
        nnz = torch.tensor(nnz_elems, dtype=torch.int64, device=dev) / (S * S) * 100
    out = (nnz, row_ptrs[0], full_col, row_ptrs[1], part_col, tiles, row_ptrs[2], load_col)
    if home != dev:
        out = tuple(t.to(home) for t in out)
    return out


class SparseStorageRefresher:
    """Recomputes the block index of a mask whose NUMBER of full / partial / loaded blocks is already known (the same
    mask structure evaluated again, e.g. every step of a serving loop) into buffers allocated once, with one call of
    the bounded single-call compaction (`stof_mask_compact_static`): no workspace, no host read, nothing allocated.
    `refresh()` returns the same tuple as `get_sparse_storage` (views of the buffers).  The buffers are sized for the
    counts of the mask seen at construction; blocks beyond them are dropped on the device, never written out of bounds,
    and `check()` (a host read) raises when the counts of the last refresh differ.  Refreshes must not overlap on the
    GPU (they share the library's built-in scratch): keep them on one stream."""

    def __init__(self, Mask: torch.Tensor, block_size_m: int, block_size_n: int):
        if not Mask.is_cuda or Mask.dim() != 3 or not Mask.is_contiguous():
            raise _lib.StofError("SparseStorageRefresher expects a contiguous (batch, S, S) CUDA mask")
        first = get_sparse_storage(Mask, block_size_m, block_size_n)
        self.mask, self.bm, self.bn = Mask, int(block_size_m), int(block_size_n)
        dev, S = Mask.device, Mask.shape[-1]
        n_full, n_part, n_load = first[2].numel(), first[4].numel(), first[7].numel()
        self._sizes = (n_full, n_part, n_load)
        self._cap = max(n_load, 1)
        self._row_ptrs = torch.empty(3, S // self.bm + 1, dtype=torch.int32, device=dev)
        self._cols = torch.empty(3, self._cap, dtype=torch.int32, device=dev)
        self._tile_cap = max(n_part, 1)
        self._tiles = torch.ones(self._tile_cap, self.bm, self.bn, dtype=torch.float16, device=dev)
        self._counts = torch.empty(4, dtype=torch.int64, device=dev)
        self.out = (first[0], self._row_ptrs[0], self._cols[0][:n_full], self._row_ptrs[1], self._cols[1][:n_part],
                    self._tiles, self._row_ptrs[2], self._cols[2][:n_load])
        self.refresh()                                    # also the library's one-time scratch lookup, outside any capture

    def refresh(self):
        m, L = self.mask, _lib.lib()
        dt = _lib.STOF_DTYPE_F16 if m.dtype == torch.float16 else _lib.STOF_DTYPE_F32
        with torch.cuda.device(m.device):
            rc = L.stof_mask_compact_static(_lib.ptr(m), dt, m.shape[0], m.shape[-1], self.bm, self.bn,
                                            _lib.ptr(self._row_ptrs[0]), _lib.ptr(self._row_ptrs[1]), _lib.ptr(self._row_ptrs[2]),
                                            _lib.ptr(self._cols[0]), _lib.ptr(self._cols[1]), _lib.ptr(self._cols[2]), self._cap,
                                            _lib.ptr(self._tiles), self._tile_cap if self._sizes[1] else 0,
                                            _lib.ptr(self._counts), _lib.current_stream_ptr(m.device))
        _lib.check(rc, "stof_mask_compact_static")
        # the index was rewritten behind torch's back: plans cached for the old contents must not be found again
        from .attention import index_rewritten
        index_rewritten(self._row_ptrs[0], self._row_ptrs[1], self._row_ptrs[2], self._cols[0], self._cols[1], self._cols[2], self._tiles)
        return self.out

    def check(self):
        """Host-side check (synchronises): the refreshed mask had the block counts the buffers were sized for."""
        n_full, n_part, n_load, _ = self._counts.tolist()
        if (n_full, n_part, n_load) != self._sizes:
            raise _lib.StofError(f"mask structure changed: {n_full}/{n_part}/{n_load} full/partial/loaded blocks, buffers hold {self._sizes}")


# ------------------------------------------------------------------------------------------
# Generators (reference: src/util/masks.py:10-122), vectorised; same signatures and results.
# ------------------------------------------------------------------------------------------
def _band(seq_len, bandwidth, device):
    i = torch.arange(seq_len, device=device)
    return (i[:, None] - i[None, :]).abs() <= bandwidth


def _causal_quirk(mask):
    # the reference clears the strict upper triangle of the last batch entry only (src/util/masks.py:28-30)
    s = mask.shape[1]
    upper = torch.triu(torch.ones(s, s, dtype=torch.bool, device=mask.device), diagonal=1)
    mask[-1][upper] = 0


def generate_causal_mask(attr_mask):
    """Lower-triangular ones, float32, on the CPU like the reference (src/util/masks.py:10-14)."""
    s = attr_mask.shape[1]
    return torch.tril(torch.ones(s, s)).unsqueeze(0).repeat(attr_mask.shape[0], 1, 1)


def generate_sliding_mask(attr_mask, bandwidth=1, is_cauasl=False):
    """|i-j| <= bandwidth, dtype/device of `attr_mask` (src/util/masks.py:17-32)."""
    out = torch.zeros_like(attr_mask)
    out[:, _band(attr_mask.shape[1], bandwidth, attr_mask.device)] = 1
    if is_cauasl:
        _causal_quirk(out)
    return out


def generate_dilated_mask(attr_mask, bandwidth=1, dilation_rate=1, is_cauasl=False):
    """Every (dilation_rate+1)-th column from i-bandwidth-dilation_rate up to
    min(S, i+bandwidth+dilation_rate+1) (src/util/masks.py:35-52)."""
    s = attr_mask.shape[1]
    i = torch.arange(s, device=attr_mask.device)[:, None]
    j = torch.arange(s, device=attr_mask.device)[None, :]
    start = i - bandwidth - dilation_rate
    end = torch.clamp(i + bandwidth + dilation_rate + 1, max=s)
    hit = (j >= start) & (j < end) & (((j - start) % (dilation_rate + 1)) == 0)
    out = torch.zeros_like(attr_mask)
    out[:, hit] = 1
    if is_cauasl:
        _causal_quirk(out)
    return out


def generate_longformer_mask(attr_mask, globalwidth=1, bandwidth=1, is_cauasl=False):
    """Global rows/cols [0,g) and [S/2,S/2+g) plus the band (src/util/masks.py:55-81)."""
    s = attr_mask.shape[1]
    out = torch.zeros_like(attr_mask)
    out[:, :globalwidth, :] = 1
    out[:, :, :globalwidth] = 1
    s0, s1 = int(s / 2), int(s / 2 + globalwidth)
    out[:, s0:s1, :] = 1
    out[:, :, s0:s1] = 1
    out[:, _band(s, bandwidth, attr_mask.device)] = 1
    if is_cauasl:
        _causal_quirk(out)
    return out


def generate_bigbird_mask(attr_mask, globalwidth=1, bandwidth=1, fill_rate=0.2, is_cauasl=False):
    """Global + band + pseudo-random fill drawn with Python's `random` seeded 0 in 32x32 tiles
    along the diagonal, with the reference's inclusive randint(0, 32) (src/util/masks.py:86-122)."""
    b, s = attr_mask.shape[0], attr_mask.shape[1]
    out = torch.zeros_like(attr_mask)
    out[:, :globalwidth, :] = 1
    out[:, :, :globalwidth] = 1
    out[:, _band(s, bandwidth, attr_mask.device)] = 1
    num_ones = int(1024 * fill_rate)
    random.seed(0)
    bi, xs, ys = [], [], []
    for batch in range(b):
        for t in range(int(s / 32) - 1):
            sx = t * 32
            if t == 0:
                sy = sx + 32 * random.choice([1, 0])
            elif t == int(s / 32) - 2:
                sy = sx + 32 * random.choice([-1, 0])
            else:
                sy = sx + 32 * random.choice([-1, 0, 1])
            for _ in range(num_ones):
                bi.append(batch)
                xs.append(sx + random.randint(0, 32))
                ys.append(sy + random.randint(0, 32))
    if bi:
        dev = attr_mask.device
        out[torch.tensor(bi, device=dev), torch.tensor(xs, device=dev), torch.tensor(ys, device=dev)] = 1
    if is_cauasl:
        _causal_quirk(out)
    return out
