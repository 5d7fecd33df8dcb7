"""Operator selection for masked attention (host side).

The reference chooses, per mask, between its row-wise and its block-wise kernels and among 36 (num_warps, BLOCK_M,
BLOCK_N) variants of the latter with an analytic model of shared memory, occupancy and grid size
(`select_operator`, src/benchmk_attn_unified.py:100-163).  Here one tensor-core kernel serves every case: the row-wise
operators are expressed through it, its thread-block shape is fixed (128 x 64 tiles, four softmax warps) and BLOCK_M x
BLOCK_N only sets the granularity of the block index.  What is left to choose is that granularity, and the rule below is
re-derived from measurements on a B200 (masks of the reference generators at S = 1024 and 4096, every BLOCK_M x BLOCK_N in
{16, 32, 64, 128}^2):

* the kernel walks the 64-wide key tiles that hold at least one listed block, whatever the block size, so blocks up to
  64 x 64 give the same walk; 128-wide blocks widen it (up to 3x slower on Longformer / BigBird masks);
* partial blocks cost a mask add per 16 x 16 group; finer blocks turn most groups of a band's edge into "full" or
  "absent" ones: 32 x 32 was as fast as 16 x 16 and 3 - 15 % faster than 64 x 64 on element-granular masks, with a quarter
  of the index entries of 16 x 16;
* a mask without partial blocks (block-aligned masks) runs the same at every size: the coarsest index wins.
"""
from __future__ import annotations

import math

# every (BLOCK_M, BLOCK_N) the reference's block-wise launcher accepts (src/benchmk_attn_unified.py:54-96); the kernel here
# takes all of them, and any num_warps (ignored)
BLOCK_WISE_CONFIGS = [{"num_warps": w, "block_m": m, "block_n": n}
                      for w, shapes in ((1, [(16, 16), (32, 16), (64, 16), (16, 32), (32, 32), (64, 32), (16, 64), (32, 64), (64, 64), (16, 128), (32, 128)]),
                                        (2, [(32, 16), (64, 16), (16, 32), (32, 32), (64, 32), (16, 64), (32, 64), (64, 64), (16, 128), (32, 128)]),
                                        (4, [(64, 16), (32, 32), (64, 32), (16, 64), (32, 64), (64, 64), (16, 128), (32, 128)]),
                                        (8, [(64, 32), (32, 64), (64, 64), (16, 128), (32, 128)]),
                                        (16, [(64, 64), (32, 128)]))
                      for m, n in shapes]


class GPUParams:
    """Device figures the reference's model reads (src/benchmk_attn_unified.py:33-52), with the B200 added as the default."""

    def __init__(self, gpu_type: str = "B200"):
        table = {"B200": (148, 227 * 1024, 2048, 64, 126 * 1024 * 1024),
                 "A100": (108, 164 * 1024, 2048, 64, 40 * 1024 * 1024),
                 "4090": (128, 100 * 1024, 1536, 48, 72 * 1024 * 1024)}
        self.gpu_type = gpu_type if gpu_type in table else "4090"
        self.sm_count, self.sm_shared, self.max_threads_per_sm, self.max_warps_per_sm, self.l2_cache = table[self.gpu_type]
        self.tensor_core_count = self.sm_count * 4
        self.register_file_size = 256 * 1024
        self.max_blocks_per_sm = 32


def phase1_decision(load_row_ptr, seq_len: int) -> bool:
    """Block-wise or row-wise?  The reference compares the share of listed 16 x 16 blocks with 1 / log2(S / 16)^2
    (src/benchmk_attn_unified.py:100-110).  The row-wise operators here run on the same tensor-core kernel, so the answer
    is always block-wise; the two figures are still returned by `mask_density` for reports."""
    return True


def mask_density(load_row_ptr, seq_len: int):
    """(share of listed 16 x 16 blocks, the reference's threshold) for an index built with BLOCK_M = BLOCK_N = 16."""
    total = (seq_len // 16) ** 2
    loaded = int(load_row_ptr[-1])
    return loaded / total, 1.0 / (math.log2(seq_len / 16) ** 2)


def phase2_selection(configs, gpu, seq_len: int, batch_size: int, head_num: int, has_partial_blocks: bool = True):
    """Index granularity for the B200 kernel among `configs`: 64 x 64 when the mask has no partial blocks at that size,
    else 32 x 32; num_warps 4 (the kernel's softmax warps; the value is not used by the launch).  Falls back to the
    admissible entry closest to the wish when `configs` lacks it.  `gpu`, `seq_len`, `batch_size` and `head_num` are
    accepted for the reference's signature; the measured ranking did not depend on them."""
    want = 32 if has_partial_blocks else 64
    ok = [c for c in configs if c["block_m"] <= 64 and c["block_n"] <= 64] or list(configs)
    if not ok:
        return None
    return min(ok, key=lambda c: (abs(c["block_m"] - want) + abs(c["block_n"] - want), abs(c["num_warps"] - 4)))


def select_operator(gpu_params, load_row_ptr, batch_size: int, seq_len: int, head_num: int, has_partial_blocks: bool = True) -> str:
    """Same result format as the reference ("block-wise warp{w}m{m}n{n}" or "row-wise",
    src/benchmk_attn_unified.py:157-163); never "row-wise" here."""
    best = phase2_selection(BLOCK_WISE_CONFIGS, gpu_params, seq_len, batch_size, head_num, has_partial_blocks)
    return f"block-wise warp{best['num_warps']}m{best['block_m']}n{best['block_n']}"


def select_block_size(mask) -> int:
    """BLOCK_M = BLOCK_N for `get_sparse_storage` on this mask (a CUDA tensor (B, S, S)): 64 if the mask has no partial
    64 x 64 block, else 32.  Costs one compaction (tens of microseconds) and a read of its counts."""
    from .masks import get_sparse_storage
    seq_len = mask.shape[-1]
    if seq_len % 64 != 0:
        return 32 if seq_len % 32 == 0 else 16
    part_row_ptr = get_sparse_storage(mask, 64, 64)[3]
    return 64 if int(part_row_ptr[-1].item()) == 0 else 32
