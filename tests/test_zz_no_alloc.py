"""The allocation-free compaction entry point against the two-phase one, through the C ABI.

Collected last on purpose (file name), so that a run that stops at the first failure has already been
through every other test.  It must also pass alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import masks as om

pytestmark = pytest.mark.gpu


def _static_call(mask_t, bm, bn, col_cap, part_cap):
    """Calls stof_mask_compact_static with caller-made buffers; returns the raw buffers and the counts."""
    from stof_b200 import _lib
    L = _lib.lib()
    dev = mask_t.device
    B, S = mask_t.shape[0], mask_t.shape[-1]
    nbm = S // bm
    row_ptrs = torch.full((3, nbm + 1), -7, dtype=torch.int32, device=dev)
    cols = torch.full((3, max(col_cap, 1)), -7, dtype=torch.int32, device=dev)
    tiles = torch.full((max(part_cap, 1), bm, bn), 3.0, dtype=torch.float16, device=dev)
    counts = torch.full((4,), -1, dtype=torch.int64, device=dev)
    dt = _lib.STOF_DTYPE_F16 if mask_t.dtype == torch.float16 else _lib.STOF_DTYPE_F32
    rc = L.stof_mask_compact_static(_lib.ptr(mask_t), dt, B, S, bm, bn, _lib.ptr(row_ptrs[0]), _lib.ptr(row_ptrs[1]), _lib.ptr(row_ptrs[2]),
                                    _lib.ptr(cols[0]), _lib.ptr(cols[1]), _lib.ptr(cols[2]), col_cap, _lib.ptr(tiles), part_cap,
                                    _lib.ptr(counts), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_mask_compact_static")
    torch.cuda.synchronize()
    return row_ptrs, cols, tiles, counts.tolist()


def _check_against_oracle(mask_np, bm, bn, row_ptrs, cols, tiles, counts):
    """The same buffers against the CPU restatement of the reference's get_sparse_storage, bit for bit."""
    st = om.get_sparse_storage(mask_np, bm, bn)
    n_full, n_part, n_load, nnz_elems = counts
    assert (n_full, n_part, n_load) == (st.full_col_idx.size, st.part_col_idx.size, st.load_col_idx.size)
    assert nnz_elems == int(np.count_nonzero(mask_np))
    for i, want in enumerate((st.full_row_ptr, st.part_row_ptr, st.load_row_ptr)):
        assert np.array_equal(row_ptrs[i].cpu().numpy(), want)
    for i, (n, want) in enumerate(((n_full, st.full_col_idx), (n_part, st.part_col_idx), (n_load, st.load_col_idx))):
        assert np.array_equal(cols[i, :n].cpu().numpy(), want)
    if n_part:
        assert np.array_equal(tiles[:n_part].cpu().numpy().view(np.uint16), st.part_block_mask.view(np.uint16))


def _check_against_two_phase(mask_np, bm, bn):
    import stof_b200
    mask_t = torch.from_numpy(mask_np).cuda()
    nnz, frp, fci, prp, pci, pbm, lrp, lci = stof_b200.get_sparse_storage(mask_t, bm, bn)       # existing entry points
    S = mask_np.shape[-1]
    cap = (S // bm) * (S // bn)
    row_ptrs, cols, tiles, (n_full, n_part, n_load, nnz_elems) = _static_call(mask_t, bm, bn, cap, cap)
    assert (n_full, n_part, n_load) == (fci.numel(), pci.numel(), lci.numel())
    assert nnz_elems == int(np.count_nonzero(mask_np))
    assert torch.equal(row_ptrs[0], frp) and torch.equal(row_ptrs[1], prp) and torch.equal(row_ptrs[2], lrp)
    assert torch.equal(cols[0, :n_full], fci) and torch.equal(cols[1, :n_part], pci) and torch.equal(cols[2, :n_load], lci)
    if n_part:
        assert torch.equal(tiles[:n_part].view(torch.int16), pbm.view(torch.int16))           # bit-exact, like the index
    assert torch.all(cols[0, n_full:] == -7) and torch.all(cols[2, n_load:] == -7)             # nothing written past the counts
    _check_against_oracle(mask_np, bm, bn, row_ptrs, cols, tiles, (n_full, n_part, n_load, nnz_elems))


def test_static_compaction_equals_two_phase_on_consecutive_calls():
    a = om.generate_causal_mask(1, 512).astype(np.float16)                  # full + partial + empty tiles
    b = om.recipe_mask("cfg2_bigbird_S2048_seed1")                          # the benchmark mask: all listed tiles full
    c = om.generate_sliding_mask(2, 256, 37, False, np.float32)             # fp32, batch 2, every listed tile partial
    # back-to-back calls share the built-in scratch: each must still match, whatever the previous one left behind
    _check_against_two_phase(a, 32, 32)
    _check_against_two_phase(b, 64, 64)
    _check_against_two_phase(a, 32, 32)
    _check_against_two_phase(c, 64, 16)
    _check_against_two_phase(c, 64, 16)


def test_static_compaction_allocates_no_device_memory():
    """What the entry point exists for: once a device has seen its first call, a call leaves the amount of free device
    memory exactly as it found it.  The buffers are made before the measurement; the call itself goes straight to the
    C ABI, so nothing of torch's caching allocator is involved either."""
    from stof_b200 import _lib
    L = _lib.lib()
    mask_np = om.generate_causal_mask(1, 512).astype(np.float16)
    mask_t = torch.from_numpy(mask_np).cuda()
    bm = bn = 32
    cap = (512 // bm) * (512 // bn)
    _static_call(mask_t, bm, bn, cap, cap)                                   # first call on this device: the one-time set-up
    dev = mask_t.device
    row_ptrs = torch.empty(3, 512 // bm + 1, dtype=torch.int32, device=dev)
    cols = torch.empty(3, cap, dtype=torch.int32, device=dev)
    tiles = torch.empty(cap, bm, bn, dtype=torch.float16, device=dev)
    counts = torch.empty(4, dtype=torch.int64, device=dev)
    stream = _lib.current_stream_ptr(dev)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    reserved_before = torch.cuda.memory_reserved(dev)
    for _ in range(2):
        rc = L.stof_mask_compact_static(_lib.ptr(mask_t), _lib.STOF_DTYPE_F16, 1, 512, bm, bn, _lib.ptr(row_ptrs[0]), _lib.ptr(row_ptrs[1]),
                                        _lib.ptr(row_ptrs[2]), _lib.ptr(cols[0]), _lib.ptr(cols[1]), _lib.ptr(cols[2]), cap, _lib.ptr(tiles),
                                        cap, _lib.ptr(counts), stream)
        assert rc == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before and torch.cuda.memory_reserved(dev) == reserved_before
    _check_against_oracle(mask_np, bm, bn, row_ptrs, cols, tiles, counts.tolist())


def test_static_compaction_respects_capacities_and_limits():
    from stof_b200 import _lib
    L = _lib.lib()
    mask_np = om.generate_causal_mask(1, 256).astype(np.float16)
    mask_t = torch.from_numpy(mask_np).cuda()
    st = om.get_sparse_storage(mask_np, 32, 32)
    row_ptrs, cols, tiles, counts = _static_call(mask_t, 32, 32, 5, 2)       # deliberately too small
    assert counts[:3] == [st.full_col_idx.size, st.part_col_idx.size, st.load_col_idx.size]   # the counts tell what was needed
    assert np.array_equal(cols[0, :5].cpu().numpy(), st.full_col_idx[:5])
    assert np.array_equal(tiles[:2].cpu().numpy().view(np.uint16), st.part_block_mask[:2].view(np.uint16))
    # beyond the built-in scratch: a clear error instead of a launch
    one = ctypes.c_void_p(256)
    rc = L.stof_mask_compact_static(one, 0, 1, 32768, 16, 16, one, one, one, one, one, one, 1, None, 0, one, None)
    assert rc == -4 and b"built-in scratch" in L.stof_last_error()
