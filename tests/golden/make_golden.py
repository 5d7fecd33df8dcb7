"""Generate the golden fixtures in this directory by running the REFERENCE's own
Python functions on CPU.

Usage (only where the reference tree is available):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `src/util/masks.py` unchanged (with an empty stand-in
for matplotlib, which that file imports only for plotting) and executes the bodies
of `torch_attn_std` (src/correct_verify_attn.py:19-30) and `bert_fwd_std`
(src/benchmk_end2end.py:31-88) extracted from their scripts with `ast` (the
scripts themselves import compiled CUDA extensions at top level and cannot be
imported).  Outputs: sparse_storage.npz, generators.json, attention.npz,
bert_layer.npz.  The tests never need the reference tree, only these files.
"""
from __future__ import annotations

import ast
import hashlib
import json
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def load_reference(ref_root: str):
    mp = types.ModuleType("matplotlib")
    pp = types.ModuleType("matplotlib.pyplot")
    mp.pyplot = pp
    sys.modules.setdefault("matplotlib", mp)
    sys.modules.setdefault("matplotlib.pyplot", pp)
    sys.dont_write_bytecode = True
    src = os.path.join(ref_root, "src")
    sys.path.insert(0, src)
    import util.masks as ref_masks  # noqa
    return src, ref_masks


def extract_function(path: str, name: str, glb: dict):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), glb)
            return glb[name]
    raise KeyError(name)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# ---------------------------------------------------------------- mask cases
def mask_cases(ref_masks):
    """name -> (mask tensor, bm, bn, how to rebuild it with the oracle generators)."""
    from oracle import masks as om
    cases = {}
    for name in om.RECIPES:
        cases[name] = (torch.from_numpy(om.recipe_mask(name)), 64, 64, {"recipe": name})
    z16 = lambda b, s: torch.zeros(b, s, s, dtype=torch.float16)
    cases["sliding_bw32_S256_b64"] = (ref_masks.generate_sliding_mask(z16(1, 256), bandwidth=32), 64, 64,
                                      {"gen": "sliding", "B": 1, "S": 256, "bandwidth": 32})
    cases["causal_S256_b32"] = (ref_masks.generate_causal_mask(z16(1, 256)), 32, 32,
                                {"gen": "causal", "B": 1, "S": 256})
    cases["causal_S256_m16n64"] = (ref_masks.generate_causal_mask(z16(2, 256)), 16, 64,
                                   {"gen": "causal", "B": 2, "S": 256})
    cases["causal_S512_m128n128"] = (ref_masks.generate_causal_mask(z16(1, 512)), 128, 128,
                                     {"gen": "causal", "B": 1, "S": 512})
    cases["bigbird_S512_b32"] = (ref_masks.generate_bigbird_mask(z16(1, 512), globalwidth=32, bandwidth=32, fill_rate=0.2), 32, 32,
                                 {"gen": "bigbird", "B": 1, "S": 512, "globalwidth": 32, "bandwidth": 32, "fill_rate": 0.2})
    cases["bigbird_S512_b64"] = (ref_masks.generate_bigbird_mask(z16(1, 512), globalwidth=1, bandwidth=1, fill_rate=0.2), 64, 64,
                                 {"gen": "bigbird", "B": 1, "S": 512, "globalwidth": 1, "bandwidth": 1, "fill_rate": 0.2})
    cases["longformer_S512_b64"] = (ref_masks.generate_longformer_mask(z16(1, 512), globalwidth=16, bandwidth=48), 64, 64,
                                    {"gen": "longformer", "B": 1, "S": 512, "globalwidth": 16, "bandwidth": 48})
    cases["dilated_S256_b16"] = (ref_masks.generate_dilated_mask(z16(1, 256), bandwidth=8, dilation_rate=1), 16, 16,
                                 {"gen": "dilated", "B": 1, "S": 256, "bandwidth": 8, "dilation_rate": 1})
    cases["sliding_causal_B2_S128_b32"] = (ref_masks.generate_sliding_mask(z16(2, 128), bandwidth=20, is_cauasl=True), 32, 32,
                                           {"gen": "sliding", "B": 2, "S": 128, "bandwidth": 20, "is_causal": True})
    frac = ref_masks.generate_sliding_mask(z16(1, 128), bandwidth=40).clone()
    frac[0, 5, 7] = 0.5
    frac[0, 100, 90] = 2.0
    cases["fractional_S128_b64"] = (frac, 64, 64, {"gen": "sliding", "B": 1, "S": 128, "bandwidth": 40,
                                                   "poke": [[5, 7, 0.5], [100, 90, 2.0]]})
    empty_rows = ref_masks.generate_sliding_mask(z16(1, 256), bandwidth=10).clone()
    empty_rows[0, 64:128, :] = 0
    cases["empty_rowblock_S256_b64"] = (empty_rows, 64, 64, {"gen": "sliding", "B": 1, "S": 256, "bandwidth": 10,
                                                             "zero_rows": [64, 128]})
    return cases


def make_sparse_storage(ref_masks, out_dir):
    arrays, meta = {}, {}
    for name, (mask, bm, bn, how) in mask_cases(ref_masks).items():
        nnz, frp, fci, prp, pci, pbm, lrp, lci = ref_masks.get_sparse_storage(mask, bm, bn)
        for key, t in (("frp", frp), ("fci", fci), ("prp", prp), ("pci", pci), ("lrp", lrp), ("lci", lci)):
            arrays[f"{name}/{key}"] = t.numpy().astype(np.int32)
        pbm_u16 = pbm.numpy().view(np.uint16)
        if pbm_u16.size <= 64 * 1024:
            arrays[f"{name}/pbm_u16"] = pbm_u16
        h = hashlib.sha256()
        for t in (frp, fci, prp, pci, lrp, lci):
            h.update(t.numpy().astype("<i4").tobytes())
        meta[name] = {"bm": bm, "bn": bn, "how": how, "nnz": float(nnz), "nnz_f32_hex": np.float32(float(nnz)).tobytes().hex(),
                      "index_sha256": h.hexdigest(), "pbm_shape": list(pbm.shape), "pbm_sha256": sha(pbm_u16),
                      "mask_sha256": sha(mask.numpy()), "mask_dtype": str(mask.dtype).replace("torch.", "")}
    np.savez_compressed(os.path.join(out_dir, "sparse_storage.npz"), **arrays)
    json.dump(meta, open(os.path.join(out_dir, "sparse_storage.json"), "w"), indent=1, sort_keys=True)


# ---------------------------------------------------------------- attention
def make_attention(src, ref_masks, out_dir):
    fn = extract_function(os.path.join(src, "correct_verify_attn.py"), "torch_attn_std", {"torch": torch})
    g = torch.Generator().manual_seed(0)
    B, H, S, D = 1, 2, 256, 64
    q32 = torch.randn(B, H, S, D, generator=g)
    k32 = torch.randn(B, H, S, D, generator=g)
    v32 = torch.randn(B, H, S, D, generator=g)
    from oracle import masks as om
    causal = ref_masks.generate_causal_mask(torch.zeros(B, S, S))
    sliding = torch.from_numpy(om.expand_block_mask(om.block_sliding(4, 1), 64, np.float32))
    banded = ref_masks.generate_sliding_mask(torch.zeros(B, S, S), bandwidth=32)
    out = {"q16": q32.half().numpy(), "k16": k32.half().numpy(), "v16": v32.half().numpy()}
    q, k, v = q32.half().float(), k32.half().float(), v32.half().float()
    out["o_causal_f32"] = fn(q, k, v, causal).numpy()
    out["o_sliding_block_f32"] = fn(q, k, v, sliding).numpy()
    out["o_banded32_f32"] = fn(q, k, v, banded).numpy()
    out["o_nomask_f32"] = fn(q, k, v, None).numpy()
    out["o_causal_f16"] = fn(q32.half(), k32.half(), v32.half(), causal.half()).numpy()
    np.savez_compressed(os.path.join(out_dir, "attention.npz"), **out)


# ---------------------------------------------------------------- BERT layer
def make_bert_layer(src, out_dir):
    import torch.nn.functional as F
    from oracle import fused as of
    B, S, hid, heads, ffn = 2, 128, 128, 2, 256
    g = torch.Generator().manual_seed(3)
    hidden = torch.randn(B, S, hid, generator=g).half()
    params = of.make_bert_params(hid, ffn, 1, seed=3, random_affine=True)[0]
    mask = torch.tril(torch.ones(S, S)).unsqueeze(0).repeat(B, 1, 1)
    p32 = {k_: v_.float() for k_, v_ in params.items()}
    x = hidden.float()
    glb = {
        "torch": torch, "F": F, "math": math,
        "input_from_tensor": x, "layer_num": 1, "head_num": heads, "head_size": hid // heads, "hidden_dim": hid,
        "attention_type": "torch_attention",
        "qkv_kernel": [torch.matmul(x, p32["Wqkv"])], "qkv_bias": [p32["bqkv"]],
        "attr_output_kernel": [p32["Wo"]], "attr_output_bias": [p32["bo"]],
        "attr_output_layernorm_gamma": [p32["g1"]], "attr_output_layernorm_beta": [p32["b1"]],
        "inter_kernel": [p32["W1"]], "inter_bias": [p32["bi1"]],
        "output_kernel": [p32["W2"]], "output_bias": [p32["bi2"]],
        "output_layernorm_gamma": [p32["g2"]], "output_layernorm_beta": [p32["b2"]],
        "transformer_output": [None],
    }
    sys.path.insert(0, src)
    from util.utils import transpose_for_scores
    glb["transpose_for_scores"] = transpose_for_scores
    fn = extract_function(os.path.join(src, "benchmk_end2end.py"), "bert_fwd_std", glb)
    fn(mask)
    out = {"hidden16": hidden.numpy(), "out_f32": glb["transformer_output"][0].numpy()}
    for k_, v_ in params.items():
        out["p_" + k_] = v_.numpy()
    np.savez_compressed(os.path.join(out_dir, "bert_layer.npz"), **out)


if __name__ == "__main__":
    ref_root = sys.argv[1]
    src, ref_masks = load_reference(ref_root)
    make_sparse_storage(ref_masks, HERE)
    make_attention(src, ref_masks, HERE)
    make_bert_layer(src, HERE)
    print("golden fixtures written to", HERE)
