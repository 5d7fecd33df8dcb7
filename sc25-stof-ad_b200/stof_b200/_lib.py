"""ctypes binding of libstof_b200.so (declarations follow include/stof_b200.h)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# STOF_B200_LIBRARY selects another build of the same library (for instance a debug build)
_LIB_PATH = os.environ.get("STOF_B200_LIBRARY") or os.path.join(_HERE, "libstof_b200.so")

STOF_DTYPE_F16, STOF_DTYPE_F32 = 0, 1
EPI_BIAS, EPI_BIAS_GELU_ERF, EPI_BIAS_GELU_TANH, EPI_BIAS_RESIDUAL, EPI_BIAS_RELU = 0, 1, 2, 3, 4

EXPORTS = ("stof_version", "stof_last_error", "stof_mask_workspace_bytes", "stof_mask_classify", "stof_mask_fill", "stof_mask_compact_static",
           "stof_block_attn_plan_bytes", "stof_block_attn_plan", "stof_block_attn_plan_paired", "stof_block_attn", "stof_block_attn_scheduled", "stof_gemm_bias_act", "stof_gemm_bias_residual_layernorm", "stof_bias_residual_layernorm")


class StofError(RuntimeError):
    pass


def library_path() -> str:
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the shared library once.  Raises StofError when it has not been built
    (run `python sc25-stof-ad_b200/build.py`); nothing else can stand in for it."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise StofError(f"{_LIB_PATH} is missing: build it with `python sc25-stof-ad_b200/build.py` "
                        "(there is no fallback path)")
    L = ctypes.CDLL(_LIB_PATH)
    vp, i32, i64, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_size_t
    i64x3 = ctypes.POINTER(ctypes.c_longlong)
    L.stof_version.restype = i32
    L.stof_last_error.restype = ctypes.c_char_p
    L.stof_mask_workspace_bytes.restype = sz
    L.stof_mask_workspace_bytes.argtypes = [i32, i32, i32]
    L.stof_mask_classify.restype = i32
    L.stof_mask_classify.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, sz, vp]
    L.stof_mask_fill.restype = i32
    L.stof_mask_fill.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    L.stof_mask_compact_static.restype = i32
    L.stof_mask_compact_static.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, i64, vp, i64, vp, vp]
    L.stof_block_attn_plan_bytes.restype = sz
    L.stof_block_attn_plan_bytes.argtypes = [i32, i32, i32]
    L.stof_block_attn_plan.restype = i32
    L.stof_block_attn_plan.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, sz, vp, vp]
    L.stof_block_attn_plan_paired.restype = i32
    L.stof_block_attn_plan_paired.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp, sz, vp, vp]
    L.stof_block_attn.restype = i32
    L.stof_block_attn.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i64x3, i64x3, i64x3, i64x3,
                                  vp, vp, vp, i32, i32, i32, f32, vp, vp]
    L.stof_block_attn_scheduled.restype = i32
    L.stof_block_attn_scheduled.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i64x3, i64x3, i64x3, i64x3,
                                            vp, vp, vp, i32, i32, i32, f32, vp, i32, vp, vp]
    L.stof_gemm_bias_act.restype = i32
    L.stof_gemm_bias_act.argtypes = [vp, i64, vp, i64, vp, vp, i64, vp, i64, i32, i32, i32, i32, vp, vp]
    L.stof_gemm_bias_residual_layernorm.restype = i32
    L.stof_gemm_bias_residual_layernorm.argtypes = [vp, i64, vp, i64, vp, vp, i64, vp, vp, f32, vp, i64, i32, i32, i32, vp, vp]
    L.stof_bias_residual_layernorm.restype = i32
    L.stof_bias_residual_layernorm.argtypes = [vp, i64, vp, vp, i64, vp, vp, f32, vp, i64, i32, i32, vp, vp]
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().stof_last_error().decode("utf-8", "replace")
        raise StofError(f"{what} failed (code {rc}): {msg}")


def strides3(vals):
    return (ctypes.c_longlong * 3)(*[int(v) for v in vals])


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream_ptr(device):
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise StofError("stof_b200 operators need CUDA tensors (there is no CPU fallback)")


_status = {}


def status_word(device):
    """Per-device int32 the kernels report bounded-wait failures through."""
    import torch
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


def check_status(device, what: str) -> None:
    """Synchronising read of the status word; raises if a kernel reported a failure."""
    st = status_word(device)
    v = int(st.item())
    if v != 0:
        st.zero_()
        code, bar = v & 0xFF, v >> 8
        raise StofError(f"{what}: kernel reported status {code} (1 = bounded wait ran out, 2 = bad block index), barrier id {bar}")
