"""Shared helpers for the tests: golden fixtures and mask reconstruction."""
import json
import os

import numpy as np

from oracle import masks as om

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_meta():
    return json.load(open(os.path.join(GOLDEN, "sparse_storage.json")))


def golden_arrays():
    return np.load(os.path.join(GOLDEN, "sparse_storage.npz"))


def build_mask(how: dict, dtype_name: str) -> np.ndarray:
    """Rebuild the mask of a golden case with the oracle's generators."""
    dt = {"float16": np.float16, "float32": np.float32}[dtype_name]
    if "recipe" in how:
        return om.recipe_mask(how["recipe"]).astype(dt)
    gen, B, S = how["gen"], how["B"], how["S"]
    if gen == "causal":
        m = om.generate_causal_mask(B, S).astype(dt)
    elif gen == "sliding":
        m = om.generate_sliding_mask(B, S, how["bandwidth"], how.get("is_causal", False), dt)
    elif gen == "dilated":
        m = om.generate_dilated_mask(B, S, how["bandwidth"], how["dilation_rate"], how.get("is_causal", False), dt)
    elif gen == "longformer":
        m = om.generate_longformer_mask(B, S, how["globalwidth"], how["bandwidth"], how.get("is_causal", False), dt)
    elif gen == "bigbird":
        m = om.generate_bigbird_mask(B, S, how["globalwidth"], how["bandwidth"], how["fill_rate"], how.get("is_causal", False), dt)
    else:
        raise KeyError(gen)
    for r, c, val in how.get("poke", []):
        m[0, r, c] = val
    if "zero_rows" in how:
        a, b = how["zero_rows"]
        m[0, a:b, :] = 0
    return m
