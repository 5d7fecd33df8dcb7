"""Oracle (test infrastructure): mask generators and mask -> block-index compaction.

Restates `src/util/masks.py` of the reference on CPU with numpy.  Nothing in the
shipped CUDA path imports this file.

Pinned bit-exactly against the reference's own functions by the fixtures under
`tests/golden/` (see `tests/golden/make_golden.py`).
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import numpy as np


# ----------------------------------------------------------------------------
# Mask generators (reference: src/util/masks.py:10-122).  All return float
# arrays of shape (B, S, S) holding 0/1, dtype as stated per function.
# ----------------------------------------------------------------------------

def _apply_reference_causal_quirk(mask: np.ndarray) -> None:
    """The reference zeroes the strict upper triangle of the LAST batch entry
    only (the loop reuses the stale `batch` variable, src/util/masks.py:28-30),
    and only for rows 0..S-2 (row S-1 has no strict upper part anyway)."""
    s = mask.shape[1]
    upper = np.triu(np.ones((s, s), dtype=bool), k=1)
    mask[-1][upper] = 0


def generate_causal_mask(batch: int, seq_len: int) -> np.ndarray:
    """Lower-triangular ones, float32 (src/util/masks.py:10-14)."""
    tri = np.tril(np.ones((seq_len, seq_len), dtype=np.float32))
    return np.broadcast_to(tri, (batch, seq_len, seq_len)).copy()


def generate_sliding_mask(batch: int, seq_len: int, bandwidth: int = 1, is_causal: bool = False,
                          dtype=np.float16) -> np.ndarray:
    """|i-j| <= bandwidth (src/util/masks.py:17-32)."""
    i = np.arange(seq_len)
    band = (np.abs(i[:, None] - i[None, :]) <= bandwidth).astype(dtype)
    out = np.broadcast_to(band, (batch, seq_len, seq_len)).copy()
    if is_causal:
        _apply_reference_causal_quirk(out)
    return out


def generate_dilated_mask(batch: int, seq_len: int, bandwidth: int = 1, dilation_rate: int = 1,
                          is_causal: bool = False, dtype=np.float16) -> np.ndarray:
    """Columns start, start+(r+1), ... < end with start = i-bandwidth-r,
    end = min(S, i+bandwidth+r+1), negative columns dropped
    (src/util/masks.py:35-52)."""
    step = dilation_rate + 1
    i = np.arange(seq_len)[:, None]
    j = np.arange(seq_len)[None, :]
    start = i - bandwidth - dilation_rate
    end = np.minimum(seq_len, i + bandwidth + dilation_rate + 1)
    hit = (j >= start) & (j < end) & (((j - start) % step) == 0)
    out = np.broadcast_to(hit.astype(dtype), (batch, seq_len, seq_len)).copy()
    if is_causal:
        _apply_reference_causal_quirk(out)
    return out


def generate_longformer_mask(batch: int, seq_len: int, globalwidth: int = 1, bandwidth: int = 1,
                             is_causal: bool = False, dtype=np.float16) -> np.ndarray:
    """Global rows/cols [0,g) and [S/2, S/2+g) plus a sliding band
    (src/util/masks.py:55-81)."""
    m = np.zeros((seq_len, seq_len), dtype=dtype)
    m[:globalwidth, :] = 1
    m[:, :globalwidth] = 1
    s0 = int(seq_len / 2)
    s1 = int(seq_len / 2 + globalwidth)
    m[s0:s1, :] = 1
    m[:, s0:s1] = 1
    i = np.arange(seq_len)
    m[np.abs(i[:, None] - i[None, :]) <= bandwidth] = 1
    out = np.broadcast_to(m, (batch, seq_len, seq_len)).copy()
    if is_causal:
        _apply_reference_causal_quirk(out)
    return out


def generate_bigbird_mask(batch: int, seq_len: int, globalwidth: int = 1, bandwidth: int = 1,
                          fill_rate: float = 0.2, is_causal: bool = False, dtype=np.float16) -> np.ndarray:
    """Global + band + pseudo-random fill drawn with Python's `random` seeded 0,
    in 32x32 tiles along the diagonal (src/util/masks.py:86-122).  `randint(0, 32)`
    is inclusive on both ends, so a tile touches 33 rows/cols, as in the reference."""
    out = np.zeros((batch, seq_len, seq_len), dtype=dtype)
    out[:, :globalwidth, :] = 1
    out[:, :, :globalwidth] = 1
    i = np.arange(seq_len)
    out[:, np.abs(i[:, None] - i[None, :]) <= bandwidth] = 1
    num_ones = int(1024 * fill_rate)
    random.seed(0)
    ntiles = int(seq_len / 32) - 1
    for b in range(batch):
        for t in range(ntiles):
            sx = t * 32
            if t == 0:
                sy = sx + 32 * random.choice([1, 0])
            elif t == int(seq_len / 32) - 2:
                sy = sx + 32 * random.choice([-1, 0])
            else:
                sy = sx + 32 * random.choice([-1, 0, 1])
            for _ in range(num_ones):
                rx = random.randint(0, 32)
                ry = random.randint(0, 32)
                out[b, sx + rx, sy + ry] = 1
    if is_causal:
        _apply_reference_causal_quirk(out)
    return out


# ----------------------------------------------------------------------------
# Block-aligned recipes used as the benchmark / parity configurations.  The
# recipe is the contract (the reference has no block-level generator); the
# element mask is the Kronecker expansion of the block matrix.
# ----------------------------------------------------------------------------

def block_sliding(nb: int, w: int) -> np.ndarray:
    i = np.arange(nb)
    return (np.abs(i[:, None] - i[None, :]) <= w).astype(np.float32)


def block_bigbird(nb: int, seed: int) -> np.ndarray:
    """3 sliding + 2 global + 3 random blocks per row; the random columns of row i
    are `torch.randperm(nb, generator=g)[:3]` drawn row after row from one CPU
    generator seeded `seed`."""
    import torch
    bm = block_sliding(nb, 1)
    bm[:2, :] = 1
    bm[:, :2] = 1
    g = torch.Generator().manual_seed(seed)
    for r in range(nb):
        cols = torch.randperm(nb, generator=g)[:3].numpy()
        bm[r, cols] = 1
    return bm


def block_longformer_dilated(nb: int) -> np.ndarray:
    """Window of +-4 blocks taking every other block, plus block row/col 0 global."""
    i = np.arange(nb)
    d = i[:, None] - i[None, :]
    bm = ((np.abs(d) <= 4) & (d % 2 == 0)).astype(np.float32)
    bm[0, :] = 1
    bm[:, 0] = 1
    return bm


def expand_block_mask(bm: np.ndarray, blk: int = 64, dtype=np.float16) -> np.ndarray:
    """(nb, nb) 0/1 block matrix -> (1, S, S) element mask."""
    return np.kron(bm, np.ones((blk, blk), dtype=np.float32)).astype(dtype)[None]


RECIPES = {
    # name: (block-matrix factory, S, B, H)
    "cfg1_sliding_S256": (lambda: block_sliding(4, 1), 256, 1, 12),
    "cfg2_bigbird_S2048_seed1": (lambda: block_bigbird(32, 1), 2048, 16, 12),
    "cfg3_longdil_S4096": (lambda: block_longformer_dilated(64), 4096, 8, 16),
    "cfg4_sliding2_S1024": (lambda: block_sliding(16, 2), 1024, 16, 12),
    "cfg5_bigbird_S4096_seed4": (lambda: block_bigbird(64, 4), 4096, 64, 16),
}


def recipe_block_matrix(name: str) -> np.ndarray:
    return RECIPES[name][0]()


def recipe_mask(name: str) -> np.ndarray:
    return expand_block_mask(recipe_block_matrix(name))


# ----------------------------------------------------------------------------
# Compaction (reference: src/util/masks.py:125-184)
# ----------------------------------------------------------------------------

@dataclass
class SparseStorage:
    nnz: float                  # 100 * count_nonzero(whole tensor) / S^2  (src/util/masks.py:136-137)
    full_row_ptr: np.ndarray    # int32 (S/bm + 1)
    full_col_idx: np.ndarray    # int32
    part_row_ptr: np.ndarray    # int32 (S/bm + 1)
    part_col_idx: np.ndarray    # int32
    part_block_mask: np.ndarray  # float16 (max(n_part,1), bm, bn); ones(1,bm,bn) when there is no partial block
    load_row_ptr: np.ndarray    # int32 (S/bm + 1)
    load_col_idx: np.ndarray    # int32

    def astuple(self):
        return (self.nnz, self.full_row_ptr, self.full_col_idx, self.part_row_ptr, self.part_col_idx,
                self.part_block_mask, self.load_row_ptr, self.load_col_idx)


def get_sparse_storage(mask: np.ndarray, bm: int, bn: int) -> SparseStorage:
    """Block-CSR index of `mask[0]` (src/util/masks.py:125-184).

    Blocks are scanned row-major.  A block whose elements all equal 1 is "full"
    (:149), one whose elements all equal 0 is dropped (:156), anything else is
    "partial" and carries the tile -10000 * (1 - block) in float16 (:160), whose
    masked-in entries are therefore -0.0.  `load_*` is the merge of both kinds
    in column order (:153,165).  Row pointers are running totals (:168-170).
    """
    assert mask.ndim == 3
    s = mask.shape[-1]
    assert mask.shape[-2] == s and s % bm == 0 and s % bn == 0
    nbm, nbn = s // bm, s // bn
    m0 = mask[0]
    tiles = m0.reshape(nbm, bm, nbn, bn).transpose(0, 2, 1, 3)       # (nbm, nbn, bm, bn)
    is_full = (tiles == 1).all(axis=(2, 3))
    is_zero = (tiles == 0).all(axis=(2, 3))
    is_part = ~is_full & ~is_zero
    is_load = is_full | is_part

    def csr(flag):
        ptr = np.zeros(nbm + 1, dtype=np.int32)
        ptr[1:] = np.cumsum(flag.sum(axis=1))
        col = np.nonzero(flag)[1].astype(np.int32)                    # row-major => ascending column inside a row
        return ptr, col

    full_row_ptr, full_col_idx = csr(is_full)
    part_row_ptr, part_col_idx = csr(is_part)
    load_row_ptr, load_col_idx = csr(is_load)
    if is_part.any():
        sel = tiles[is_part].astype(np.float16)                      # row-major order of the partial blocks
        part_block_mask = (np.float16(-10000.0) * (np.float16(1.0) - sel)).astype(np.float16)
    else:
        part_block_mask = np.ones((1, bm, bn), dtype=np.float16)
    nnz = float(np.float32(np.count_nonzero(mask)) / np.float32(s * s) * np.float32(100))
    return SparseStorage(nnz, full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, part_block_mask,
                         load_row_ptr, load_col_idx)


def index_sha256(st: SparseStorage) -> str:
    """sha256 over the little-endian int32 bytes of the six index arrays in the
    order full_row_ptr, full_col_idx, part_row_ptr, part_col_idx, load_row_ptr,
    load_col_idx."""
    import hashlib
    h = hashlib.sha256()
    for a in (st.full_row_ptr, st.full_col_idx, st.part_row_ptr, st.part_col_idx, st.load_row_ptr, st.load_col_idx):
        h.update(np.ascontiguousarray(a).astype("<i4").tobytes())
    return h.hexdigest()
