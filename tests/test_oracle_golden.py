"""The CPU oracle against fixtures produced by the reference's own functions."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import attention as oa
from oracle import fused as of
from oracle import masks as om
from _cases import GOLDEN, build_mask, golden_arrays, golden_meta

META = golden_meta()


@pytest.mark.parametrize("name", sorted(META))
def test_generators_and_compaction_match_reference(name):
    meta, arrs = META[name], golden_arrays()
    mask = build_mask(meta["how"], meta["mask_dtype"])
    # the generator itself is pinned through the sha of the reference's mask bytes
    assert hashlib.sha256(np.ascontiguousarray(mask).tobytes()).hexdigest() == meta["mask_sha256"]
    st = om.get_sparse_storage(mask, meta["bm"], meta["bn"])
    for key, got in (("frp", st.full_row_ptr), ("fci", st.full_col_idx), ("prp", st.part_row_ptr),
                     ("pci", st.part_col_idx), ("lrp", st.load_row_ptr), ("lci", st.load_col_idx)):
        want = arrs[f"{name}/{key}"]
        assert got.dtype == np.int32 and np.array_equal(got, want), key
    assert om.index_sha256(st) == meta["index_sha256"]
    assert list(st.part_block_mask.shape) == meta["pbm_shape"]
    got_u16 = st.part_block_mask.view(np.uint16)
    assert hashlib.sha256(np.ascontiguousarray(got_u16).tobytes()).hexdigest() == meta["pbm_sha256"]
    if f"{name}/pbm_u16" in arrs:
        assert np.array_equal(got_u16, arrs[f"{name}/pbm_u16"])
    assert np.float32(st.nnz).tobytes().hex() == meta["nnz_f32_hex"]


def test_known_answer_cfg1():
    st = om.get_sparse_storage(om.recipe_mask("cfg1_sliding_S256"), 64, 64)
    assert st.full_row_ptr.tolist() == [0, 2, 5, 8, 10] == st.load_row_ptr.tolist()
    assert st.full_col_idx.tolist() == [0, 1, 0, 1, 2, 1, 2, 3, 2, 3] == st.load_col_idx.tolist()
    assert st.part_row_ptr.tolist() == [0, 0, 0, 0, 0] and st.part_col_idx.size == 0
    assert np.array_equal(st.part_block_mask, np.ones((1, 64, 64), np.float16))


def test_recipe_hash_prefixes():
    want = {"cfg1_sliding_S256": "db1c49c515fa6317", "cfg2_bigbird_S2048_seed1": "bca28eef803e8c97",
            "cfg3_longdil_S4096": "1e90d193002604cd", "cfg4_sliding2_S1024": "208c1623a676858b",
            "cfg5_bigbird_S4096_seed4": "e6cfa39f0fc3a19f"}
    for name, prefix in want.items():
        st = om.get_sparse_storage(om.recipe_mask(name), 64, 64)
        assert om.index_sha256(st).startswith(prefix), name


def test_masked_zero_is_negative_zero():
    st = om.get_sparse_storage(om.generate_causal_mask(1, 64), 32, 32)
    u = st.part_block_mask.view(np.uint16)
    assert set(np.unique(u).tolist()) == {0x8000, 0xF0E2}     # -0.0 and -10000.0


def _attn_fixture():
    z = np.load(os.path.join(GOLDEN, "attention.npz"))
    q, k, v = (torch.from_numpy(z[n]) for n in ("q16", "k16", "v16"))
    return z, q, k, v


def test_attention_oracle_matches_reference_function():
    z, q, k, v = _attn_fixture()
    S = q.shape[2]
    causal = om.generate_causal_mask(1, S)
    sliding = om.expand_block_mask(om.block_sliding(4, 1), 64, np.float32)
    banded = om.generate_sliding_mask(1, S, 32, False, np.float32)
    for key, mask in (("o_causal_f32", causal), ("o_sliding_block_f32", sliding), ("o_banded32_f32", banded), ("o_nomask_f32", None)):
        got = oa.masked_attention_fp32(q, k, v, None if mask is None else torch.from_numpy(mask))
        assert torch.allclose(got, torch.from_numpy(z[key]), atol=2e-6, rtol=0), key


def test_block_index_semantics_equal_dense_masked_path():
    """Softmax over the listed blocks (+ partial tiles) equals the dense -10000 path."""
    z, q, k, v = _attn_fixture()
    S = q.shape[2]
    for mask, bm, bn, key in ((om.generate_causal_mask(1, S), 32, 32, "o_causal_f32"),
                              (om.generate_causal_mask(1, S), 16, 64, "o_causal_f32"),
                              (om.generate_sliding_mask(1, S, 32, False, np.float32), 64, 64, "o_banded32_f32"),
                              (om.expand_block_mask(om.block_sliding(4, 1), 64, np.float32), 64, 64, "o_sliding_block_f32")):
        st = om.get_sparse_storage(mask, bm, bn)
        got = oa.block_attention_from_index(q, k, v, st, bm, bn)
        assert (got - torch.from_numpy(z[key])).abs().max().item() < 1e-5, key


def test_reference_fp16_path_is_within_tolerance_of_fp32_oracle():
    z, q, k, v = _attn_fixture()
    d = (torch.from_numpy(z["o_causal_f16"]).float() - torch.from_numpy(z["o_causal_f32"])).abs().max().item()
    assert d < 4e-3     # the reference's own fp16 path sits at ~1e-3 from fp32


def test_bert_layer_oracle_matches_reference_function():
    z = np.load(os.path.join(GOLDEN, "bert_layer.npz"))
    params = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("p_")}
    hidden = torch.from_numpy(z["hidden16"])
    B, S, _ = hidden.shape
    mask = torch.tril(torch.ones(S, S)).unsqueeze(0).repeat(B, 1, 1)
    got = of.bert_layer(hidden, params, mask, head_num=2, eps=1e-5)
    assert torch.allclose(got, torch.from_numpy(z["out_f32"]), atol=2e-5, rtol=0)


def test_make_bert_params_is_seed_stable():
    z = np.load(os.path.join(GOLDEN, "bert_layer.npz"))
    p = of.make_bert_params(128, 256, 1, seed=3, random_affine=True)[0]
    for k, v in p.items():
        assert np.array_equal(v.numpy(), z["p_" + k]), k


def test_rowwise_oracles_agree_with_dense_path():
    z, q, k, v = _attn_fixture()
    S = q.shape[2]
    want = oa.merge_heads(torch.from_numpy(z["o_causal_f32"]))
    assert torch.allclose(oa.rowwise_full(q, k, v, True), want, atol=1e-5)
    band = 17
    i = np.arange(S)
    allowed = ((i[None, :] > i[:, None] - band) & (i[None, :] <= i[:, None])).astype(np.float32)
    want = oa.merge_heads(oa.masked_attention_fp32(q, k, v, torch.from_numpy(allowed)[None]))
    assert torch.allclose(oa.rowwise_sliding(q, k, v, True, band), want, atol=1e-5)
    assert torch.allclose(oa.rowwise_mask(q, k, v, False, allowed), want, atol=1e-5)
