"""CPU-side checks: the C-ABI library loads and exports what the header declares, argument validation
answers without a GPU, and the host-side generators reproduce the reference's masks."""
import ctypes
import hashlib
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("stof_build", os.path.join(ROOT, "sc25-stof-ad_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    path = mod.build_library()
    from stof_b200 import _lib
    return _lib.lib(), path


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "stof_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(stof_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    L, path = built_lib
    names = declared_symbols()
    assert len(names) >= 8
    raw = ctypes.CDLL(path)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/stof_b200.h but not exported"
    assert L.stof_version() >= 100


def test_binding_table_matches_header(built_lib):
    from stof_b200 import _lib
    assert sorted(_lib.EXPORTS) == declared_symbols()


def test_argument_validation_needs_no_gpu(built_lib):
    L, _ = built_lib
    from stof_b200 import _lib
    s3 = _lib.strides3((64, 64, 64))
    one = ctypes.c_void_p(16)
    rc = L.stof_block_attn(one, one, one, one, 1, 1, 64, 32, s3, s3, s3, s3, one, None, one, 64, 64, 4, 0.125, None, None)
    assert rc == -1 and b"head_dim" in L.stof_last_error()
    rc = L.stof_block_attn(one, one, one, one, 1, 1, 100, 64, s3, s3, s3, s3, one, None, one, 64, 64, 4, 0.125, None, None)
    assert rc == -1 and b"multiple" in L.stof_last_error()
    rc = L.stof_block_attn(one, one, one, one, 1, 1, 96, 64, s3, s3, s3, s3, one, None, one, 48, 48, 4, 0.125, None, None)
    assert rc == -1 and b"BLOCK_M" in L.stof_last_error()
    rc = L.stof_block_attn_plan(one, one, one, one, 128, 64, 64, one, 8, None, None)
    assert rc == -3 and b"plan buffer" in L.stof_last_error()
    rc = L.stof_block_attn_plan(one, one, one, one, 65536, 16, 16, one, 1 << 30, None, None)
    assert rc == -4 and b"block table" in L.stof_last_error()
    assert L.stof_block_attn_plan_bytes(2048, 64, 64) > 16 * 32 * 66
    rc = L.stof_mask_classify(one, 0, 1, 100, 64, 64, one, one, one, one, one, 1 << 20, None)
    assert rc == -1
    rc = L.stof_mask_classify(one, 0, 1, 128, 64, 64, one, one, one, one, one, 8, None)
    assert rc == -3 and b"workspace" in L.stof_last_error()
    rc = L.stof_gemm_bias_act(one, 60, one, 64, None, None, 0, one, 64, 8, 64, 60, 0, None, None)
    assert rc == -1
    rc = L.stof_bias_residual_layernorm(one, 16384, None, None, 0, None, None, 1e-5, one, 16384, 4, 16384, None, None)
    assert rc == -4 and b"8192" in L.stof_last_error()
    assert L.stof_mask_workspace_bytes(4096, 64, 64) == 16 + 64 * 64


def test_ops_refuse_cpu_tensors(built_lib):
    import stof_b200
    x = torch.zeros(2, 8, dtype=torch.float16)
    with pytest.raises(stof_b200.StofError):
        stof_b200.bias_residual_layernorm(x)
    with pytest.raises(stof_b200.StofError):
        stof_b200.gemm_bias(x, torch.zeros(8, 8, dtype=torch.float16))


def test_host_generators_match_reference_masks():
    from _cases import golden_meta
    import stof_b200.masks as hm
    meta = golden_meta()

    def sha(t):
        return hashlib.sha256(np.ascontiguousarray(t.numpy()).tobytes()).hexdigest()

    z = lambda b, s: torch.zeros(b, s, s, dtype=torch.float16)
    assert sha(hm.generate_sliding_mask(z(1, 256), bandwidth=32)) == meta["sliding_bw32_S256_b64"]["mask_sha256"]
    assert sha(hm.generate_causal_mask(z(1, 256))) == meta["causal_S256_b32"]["mask_sha256"]
    assert sha(hm.generate_bigbird_mask(z(1, 512), globalwidth=32, bandwidth=32, fill_rate=0.2)) == meta["bigbird_S512_b32"]["mask_sha256"]
    assert sha(hm.generate_bigbird_mask(z(1, 512), globalwidth=1, bandwidth=1, fill_rate=0.2)) == meta["bigbird_S512_b64"]["mask_sha256"]
    assert sha(hm.generate_longformer_mask(z(1, 512), globalwidth=16, bandwidth=48)) == meta["longformer_S512_b64"]["mask_sha256"]
    assert sha(hm.generate_dilated_mask(z(1, 256), bandwidth=8, dilation_rate=1)) == meta["dilated_S256_b16"]["mask_sha256"]
    assert sha(hm.generate_sliding_mask(z(2, 128), bandwidth=20, is_cauasl=True)) == meta["sliding_causal_B2_S128_b32"]["mask_sha256"]


def test_drop_in_module_names_import():
    import ops.package_op as po
    import util.masks as um
    import util.utils as uu
    import triton_template.gemm_add_layernorm as t1
    import triton_template.gemm_gemm as t2
    import triton_template.add_layernorm as t3
    import block_attn_mask as ext
    import rowwise_attn_full as r1, rowwise_attn_sliding as r2, rowwise_attn_mask as r3
    assert callable(po.block_attn_mask_op) and callable(ext.forward)
    assert all(callable(f) for f in (po.rowwise_attn_full_op, po.rowwise_attn_sliding_op, po.rowwise_attn_mask_op, r1.forward, r2.forward, r3.forward))
    assert callable(um.get_sparse_storage) and callable(um.generate_bigbird_mask)
    assert callable(uu.transpose_for_scores) and callable(uu.time_stamp_cudasync)
    assert callable(t1.triton_matmul_bias_layernorm) and callable(t2.triton_matmul_batch) and callable(t3.triton_batched_bias_layernorm)
    x = torch.arange(2 * 4 * 6.0).view(2, 4, 6)
    assert uu.transpose_for_scores(x, 2, 3).shape == (2, 2, 4, 3)


def test_workload_recipes_equal_the_oracle_recipes():
    from oracle import masks as om
    from stof_b200 import workloads as wl
    pairs = {"cfg1": "cfg1_sliding_S256", "cfg2": "cfg2_bigbird_S2048_seed1", "cfg3": "cfg3_longdil_S4096"}
    for key, oname in pairs.items():
        assert np.array_equal(wl.config_mask(wl.ATTENTION_CONFIGS[key]).numpy(), om.recipe_mask(oname)), key
    for key, oname in {"cfg4": "cfg4_sliding2_S1024", "cfg5": "cfg5_bigbird_S4096_seed4"}.items():
        assert np.array_equal(wl.config_mask(wl.ENCODER_CONFIGS[key]).numpy(), om.recipe_mask(oname)), key
    q, k, v = wl.attention_inputs(wl.ATTENTION_CONFIGS["cfg1"])
    g = torch.Generator().manual_seed(0)
    assert torch.equal(q, torch.randn(1, 12, 256, 64, generator=g).half())
    assert wl.attention_flops(286, 16, 12) == pytest.approx(5.758e10, rel=1e-3)


def test_lpt_schedule_table():
    """Host-side deal of the attention work items: every item exactly once, offsets monotone, and a better balance than
    dealing the sorted items round-robin."""
    from stof_b200.attention import lpt_schedule, _SCHED_OVERHEAD_STEPS
    counts = [32, 6, 7, 9, 12, 12, 0, 11, 9, 10, 13, 8, 9, 12, 10, 11]
    bh, blocks = 48, 40
    table, g = lpt_schedule(counts, bh, blocks)
    t = table.tolist()
    assert g == blocks and t[0] == blocks and t[1] == 0 and t[1 + blocks] == len(counts) * bh
    offs, ids = t[1:2 + blocks], t[2 + blocks:]
    assert all(a <= b for a, b in zip(offs, offs[1:]))
    assert sorted(ids) == list(range(len(counts) * bh))
    cost = lambda i: (counts[i % len(counts)] + _SCHED_OVERHEAD_STEPS) if counts[i % len(counts)] else 0.25
    loads = [sum(cost(i) for i in ids[offs[b]:offs[b + 1]]) for b in range(blocks)]
    order = sorted(range(len(counts)), key=lambda q: -counts[q])
    rr = [0.0] * blocks
    for n, i in enumerate(q + len(counts) * h for q in order for h in range(bh)):
        rr[n % blocks] += cost(i)
    assert max(loads) <= max(rr) and max(loads) <= 1.06 * sum(loads) / blocks
    few, g2 = lpt_schedule([3, 2], 1, 40)                     # fewer items than blocks: one block per item
    assert g2 == 2 and few.tolist()[0] == 2


def test_util_helpers_of_the_reference_scripts(tmp_path):
    """`util.masks.flex_*_mask`, `util.utils.{transpose_for_scores1, read_config_file, get_best_config}`: the helper names the
    reference's benchmark scripts import, with the reference's behaviour (score-mod predicates with its constants; tuning-log
    parser)."""
    import torch
    from util import masks as um, utils as uu
    q = torch.arange(400)[:, None]
    k = torch.arange(400)[None, :]
    w = um.flex_sliding_window_mask(0, 0, q, k)
    assert bool(w[300, 44]) and not bool(w[300, 43]) and bool(w[0, 399])              # q - kv <= 256, one-sided
    lf = um.flex_longformer_mask(0, 0, q, k)
    assert bool(lf[390, 100]) and bool(lf[100, 390 - 390]) and not bool(lf[390, 64]) and bool(lf[20, 399])
    bb = um.flex_bigbird_mask(0, 0, q, k)
    assert bool(bb[399, 0]) and not bool(bb[397, 64]) and torch.equal(bb, lf)      # its extra keys (key 0) are global already
    assert um.flex_causal_mask(0, 0, 5, 5) and not um.flex_causal_mask(0, 0, 4, 5)
    x = torch.arange(2 * 3 * 768, dtype=torch.float32).reshape(2, 3, 768)
    assert uu.transpose_for_scores1(x).shape == (2, 12, 3, 64) and torch.equal(uu.transpose_for_scores1(x)[1, 2, 1], x[1, 1, 128:192])
    log = tmp_path / "tuning.txt"
    log.write_text("num_warp4 | m64n64 | bs:16 | seq:2048 | 0.52 ms/iter | Speedup/FA2: 1.93\nheader line\n"
                   "num_warp8 | m128n64 | bs:16 | seq:2048 | 0.61 ms/iter | Speedup/FA2: 1.6\n"
                   "num_warp2 | m32n32 | bs:1 | seq:256 | 0.02 ms/iter | Speedup/FA2: 3.1\n")
    table = uu.read_config_file(str(log))
    assert table == {16: {2048: [(64, 64, 4), (128, 64, 8)]}, 1: {256: [(32, 32, 2)]}}
    assert uu.get_best_config(table, 16, 2048) == (64, 64, 4)
    with pytest.raises(ValueError):
        uu.get_best_config(table, 2, 2048)


def test_pair_halves_host_logic():
    """`pair_halves` on block indices given as plain lists: a dilated window pairs halves r and r + 2 (their key-tile lists
    agree: fewer loads), rows with long and short lists in turn are paired long with long (fewer steps), every half lands
    in exactly one item (an odd count leaves one alone), and a plain sliding window, whose neighbours already agree, is
    left to the default pairing."""
    import numpy as np
    from stof_b200.attention import pair_halves

    def index(blocks):
        ptr, col = [0], []
        for r in range(blocks.shape[0]):
            col += np.nonzero(blocks[r])[0].tolist()
            ptr.append(len(col))
        return ptr, col

    for nb in (64, 17):
        i = np.arange(nb)
        d = i[:, None] - i[None, :]
        dil = (np.abs(d) <= 4) & (d % 2 == 0)
        ptr, col = index(dil)
        pairs, before, after = pair_halves(ptr, col, [0] * (nb + 1), [], nb * 64, 64, 64)
        assert pairs is not None and after < 0.9 * before
        assert sum(1 for p in pairs if p[1] >= 0 and (p[1] - p[0]) % 2 == 0) >= len(pairs) - 3      # r with r + 2, but for the ends
        flat = [h for p in pairs for h in p if h >= 0]
        assert sorted(flat) == list(range(nb)) and len(pairs) == (nb + 1) // 2
        assert sum(1 for p in pairs if p[1] < 0) == nb % 2
        assert all(p[0] >= 0 and (p[1] < 0 or p[0] < p[1]) for p in pairs)
        # the same index as partial blocks of 16 x 32
        ptr16, col16 = index(np.kron(dil, np.ones((4, 2), bool)))
        pairs16, b16, a16 = pair_halves([0] * (4 * nb + 1), [], ptr16, col16, nb * 64, 16, 32)
        assert (b16, a16) == (before, after) and pairs16 == pairs
        slide = np.abs(d) <= 1
        ptr, col = index(slide)
        assert pair_halves(ptr, col, [0] * (nb + 1), [], nb * 64, 64, 64)[0] is None
    # even rows list eight tiles, odd rows two: an item takes as many steps as its longer half, so like goes with like
    nb = 32
    uneven = np.zeros((nb, nb), bool)
    for r in range(nb):
        uneven[r, [(r + 3 * c) % nb for c in range(8 if r % 2 == 0 else 2)]] = True
    ptr, col = index(uneven)
    pairs, before, after = pair_halves(ptr, col, [0] * (nb + 1), [], nb * 64, 64, 64)
    assert pairs is not None and after < 0.75 * before
    assert all(a % 2 == b % 2 for a, b in pairs)


def test_plan_cache_key_follows_in_place_rewrites():
    """The plan cache identifies a block index by its tensors' storage, version and length; a rewrite through the C ABI moves
    none of them, so `index_rewritten` advances a generation that is part of the key (the refresher calls it)."""
    from stof_b200 import attention as A
    idx = tuple(torch.zeros(n, dtype=torch.int32) for n in (5, 7, 5, 3))
    k0 = A._plan_key(idx, 256, 64, 64)
    assert A._plan_key(idx, 256, 64, 64) == k0
    A.index_rewritten(idx[1], None)
    k1 = A._plan_key(idx, 256, 64, 64)
    assert k1 != k0 and k1[0] == k0[0] and k1[1] != k0[1]
    idx[0].add_(1)                                       # a write torch does see moves the version counter
    assert A._plan_key(idx, 256, 64, 64) != k1
    assert A._plan_key(idx, 256, 32, 64) != A._plan_key(idx, 256, 64, 64)


def test_operator_selector_host_logic():
    """The selector keeps the reference's interface (src/benchmk_attn_unified.py:100-163) and result format; on this
    kernel it never answers "row-wise" and picks the index granularity from whether partial blocks exist."""
    from stof_b200 import selector as sel
    assert len(sel.BLOCK_WISE_CONFIGS) == 36 and {"num_warps": 16, "block_m": 32, "block_n": 128} in sel.BLOCK_WISE_CONFIGS
    gpu = sel.GPUParams()
    assert (gpu.gpu_type, gpu.sm_count, gpu.sm_shared) == ("B200", 148, 227 * 1024)
    assert sel.GPUParams("A100").sm_count == 108 and sel.GPUParams("other").sm_count == 128
    load_row_ptr = [0, 3, 7, 12]
    assert sel.select_operator(gpu, load_row_ptr, 8, 4096, 12) == "block-wise warp4m32n32"
    assert sel.select_operator(gpu, load_row_ptr, 8, 4096, 12, has_partial_blocks=False) == "block-wise warp4m64n64"
    assert sel.phase1_decision(load_row_ptr, 4096) is True
    rho, tau = sel.mask_density(load_row_ptr, 4096)
    assert abs(rho - 12 / 65536) < 1e-12 and abs(tau - 1 / 64) < 1e-12
    only_wide = [c for c in sel.BLOCK_WISE_CONFIGS if c["block_n"] == 128]
    assert sel.phase2_selection(only_wide, gpu, 4096, 8, 12)["block_m"] == 32
    assert sel.phase2_selection([], gpu, 4096, 8, 12) is None


def test_host_pipeline_chunking():
    """Chunk sizes of the host-buffer pipeline: they cover the batch in order, none exceeds the staging size, and the tail is
    tapered so that little work follows the last inbound copy."""
    from stof_b200.attention import tapered_chunks
    assert tapered_chunks(16, 4, 0) == [4, 4, 4, 4]
    assert tapered_chunks(16, 4, 2) == [4, 4, 4, 2, 1, 1]
    assert tapered_chunks(7, 3, 1) == [3, 3, 1]
    assert tapered_chunks(1, 4, 2) == [1]
    assert tapered_chunks(0, 4, 2) == []
    for batch in range(1, 20):
        for chunk in (1, 2, 5):
            sizes = tapered_chunks(batch, chunk, 2)
            assert sum(sizes) == batch and max(sizes) <= chunk and min(sizes) >= 1
