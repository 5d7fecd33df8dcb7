"""CUDA mask -> block-index compaction against the oracle and the reference-generated fixtures (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import masks as om
from _cases import build_mask, golden_arrays, golden_meta

pytestmark = pytest.mark.gpu
META = golden_meta()


def _run(mask_np, bm, bn):
    import stof_b200
    out = stof_b200.get_sparse_storage(torch.from_numpy(mask_np).cuda(), bm, bn)
    torch.cuda.synchronize()
    return out


def _compare(got, st):
    nnz, frp, fci, prp, pci, pbm, lrp, lci = got
    for name, g, w in (("full_row_ptr", frp, st.full_row_ptr), ("full_col_idx", fci, st.full_col_idx),
                       ("part_row_ptr", prp, st.part_row_ptr), ("part_col_idx", pci, st.part_col_idx),
                       ("load_row_ptr", lrp, st.load_row_ptr), ("load_col_idx", lci, st.load_col_idx)):
        assert g.dtype == torch.int32 and g.is_cuda, name
        assert np.array_equal(g.cpu().numpy(), w), name
    assert pbm.dtype == torch.float16 and tuple(pbm.shape) == st.part_block_mask.shape
    got_u16, want_u16 = pbm.cpu().numpy().view(np.uint16), st.part_block_mask.view(np.uint16)
    nan = np.isnan(st.part_block_mask)
    assert np.array_equal(np.isnan(pbm.cpu().numpy()), nan)            # NaN payload bits are not part of the contract
    assert np.array_equal(got_u16[~nan], want_u16[~nan]), "partial tiles (bit pattern, incl. -0.0)"
    assert nnz.dim() == 0 and np.float32(nnz.item()).tobytes() == np.float32(st.nnz).tobytes()


@pytest.mark.parametrize("name", sorted(META))
def test_compaction_matches_reference_fixture(name):
    meta, arrs = META[name], golden_arrays()
    mask = build_mask(meta["how"], meta["mask_dtype"])
    got = _run(mask, meta["bm"], meta["bn"])
    _compare(got, om.get_sparse_storage(mask, meta["bm"], meta["bn"]))
    for key, t in (("frp", got[1]), ("fci", got[2]), ("prp", got[3]), ("pci", got[4]), ("lrp", got[6]), ("lci", got[7])):
        assert np.array_equal(t.cpu().numpy(), arrs[f"{name}/{key}"]), key      # the reference's own output


@pytest.mark.parametrize("bm,bn", [(16, 16), (16, 128), (32, 64), (64, 16), (128, 32), (128, 128), (64, 8), (8, 64), (256, 256)])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_compaction_random_masks_every_block_shape(bm, bn, dtype):
    rng = np.random.default_rng(bm * 1000 + bn)
    S = 512
    nbm, nbn = S // bm, S // bn
    kind = rng.integers(0, 3, size=(nbm, nbn))                         # 0 empty, 1 full, 2 partial
    mask = np.kron((kind == 1).astype(np.float32), np.ones((bm, bn), np.float32))
    noise = (rng.random((S, S)) < 0.5).astype(np.float32)
    part = np.kron((kind == 2).astype(np.float32), np.ones((bm, bn), np.float32)).astype(bool)
    mask[part] = noise[part]
    mask = np.broadcast_to(mask, (2, S, S)).astype(dtype).copy()
    mask[1, :7, :9] = 1                                                # batch 1 only feeds the non-zero count
    _compare(_run(mask, bm, bn), om.get_sparse_storage(mask, bm, bn))


def test_compaction_edge_masks():
    S = 256
    for mask in (np.zeros((1, S, S), np.float16), np.ones((1, S, S), np.float16)):
        _compare(_run(mask, 64, 64), om.get_sparse_storage(mask, 64, 64))
    m = np.ones((1, S, S), np.float16)
    m[0, 0, 0] = np.float16(-0.0)          # negative zero is zero: one partial block
    m[0, 200, 100] = np.float16(np.nan)    # NaN is neither 0 nor 1: partial, counts as non-zero
    _compare(_run(m, 64, 64), om.get_sparse_storage(m, 64, 64))
    tiny = np.tril(np.ones((1, 16, 16), np.float32))
    _compare(_run(tiny, 16, 16), om.get_sparse_storage(tiny, 16, 16))


def test_compaction_full_size_properties():
    """S = 4096 (the largest configuration): structural invariants of the index, plus equality with the oracle."""
    mask = om.recipe_mask("cfg5_bigbird_S4096_seed4")
    got = _run(mask, 64, 64)
    nnz, frp, fci, prp, pci, pbm, lrp, lci = [t.cpu() for t in got]
    assert int(lrp[-1]) == 608 and int(prp[-1]) == 0 and torch.equal(frp, lrp) and torch.equal(fci, lci)
    for r in range(64):
        cols = lci[lrp[r]:lrp[r + 1]]
        assert torch.all(cols[1:] > cols[:-1])                          # strictly ascending inside a row
    _compare(got, om.get_sparse_storage(mask, 64, 64))
    # idempotence: rebuilding the element mask from the index and compacting again gives the same index
    rebuilt = np.zeros((64, 64), np.float32)
    for r in range(64):
        rebuilt[r, lci[lrp[r]:lrp[r + 1]].numpy()] = 1
    again = _run(om.expand_block_mask(rebuilt), 64, 64)
    assert torch.equal(again[7].cpu(), lci) and torch.equal(again[6].cpu(), lrp)


def test_cpu_resident_mask_round_trips_through_the_gpu():
    import stof_b200
    mask = torch.from_numpy(om.generate_causal_mask(1, 128))
    out = stof_b200.get_sparse_storage(mask, 32, 32)
    assert all(not t.is_cuda for t in out)
    _compare(tuple(t.cuda() if i else t for i, t in enumerate(out)), om.get_sparse_storage(mask.numpy(), 32, 32))


@pytest.mark.gpu
def test_refresher_reuses_buffers_and_detects_structure_change():
    """`SparseStorageRefresher` recomputes the index without a host read; same mask -> identical tensors, a mask with
    other block counts -> `check()` raises."""
    import stof_b200
    S = 512
    m1 = torch.from_numpy(om.generate_sliding_mask(1, S, 70, False, np.float16)).cuda()
    want = stof_b200.get_sparse_storage(m1, 64, 64)
    ref = stof_b200.SparseStorageRefresher(m1, 64, 64)
    got = ref.refresh()
    ref.check()
    for a, b in zip(got[1:], want[1:]):
        assert torch.equal(a, b)
    m1.copy_(torch.from_numpy(om.generate_causal_mask(1, S).astype(np.float16)).cuda())      # other structure, same buffer
    ref.refresh()
    with pytest.raises(stof_b200.StofError):
        ref.check()
