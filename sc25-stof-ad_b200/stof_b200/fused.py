"""Fused GEMM / LayerNorm operators (host side of `stof_gemm_bias_act` and
`stof_bias_residual_layernorm`)."""
from __future__ import annotations

import torch

from . import _lib


def _as_rows(t: torch.Tensor):
    """(…, C) tensor -> (rows, C) view with a contiguous last dim, without copying when possible."""
    if t.stride(-1) != 1:
        t = t.contiguous()
    t2 = t.reshape(-1, t.shape[-1])          # a view whenever the leading dims are collapsible
    return t2


def _gemm(a, w, bias, epilogue, residual=None, out=None):
    _lib.require_cuda(a, w, bias, residual, out)
    if a.dtype != torch.float16 or w.dtype != torch.float16:
        raise _lib.StofError("gemm: float16 operands expected")
    if w.dim() != 2:
        raise _lib.StofError("gemm: weight must be (K, N)")
    a2 = _as_rows(a)
    if w.stride(1) != 1:
        w = w.contiguous()
    M, K = a2.shape
    K2, N = w.shape
    if K != K2:
        raise _lib.StofError(f"gemm: inner dimensions differ ({K} vs {K2})")
    if bias is not None:
        bias = bias.reshape(-1)
        if bias.numel() != N or bias.dtype != torch.float16:
            raise _lib.StofError("gemm: bias must be a float16 vector of length N")
        bias = bias.contiguous()
    out_shape = tuple(a.shape[:-1]) + (N,)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.float16, device=a.device)
    elif out.dtype != torch.float16 or out.numel() != M * N or out.shape[-1] != N:
        raise _lib.StofError(f"gemm: out must be float16 of shape {out_shape}")       # the kernel stores M rows of N whatever out holds
    c2 = out.reshape(-1, N)
    if c2.data_ptr() != out.data_ptr() or c2.stride(1) != 1:
        raise _lib.StofError("gemm: output must be viewable as contiguous rows")
    r2, ldr = None, 0
    if residual is not None:
        r2 = _as_rows(residual)
        if r2.shape != (M, N) or r2.dtype != torch.float16:
            raise _lib.StofError("gemm: residual must be float16 of the output's shape")
        ldr = r2.stride(0)
    dev = a.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        st = _lib.status_word(dev)
        rc = L.stof_gemm_bias_act(_lib.ptr(a2), a2.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(bias), _lib.ptr(r2), ldr,
                                  _lib.ptr(c2), c2.stride(0), M, N, K, epilogue, _lib.ptr(st), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_gemm_bias_act")
    return out


def gemm_bias(a, w, bias=None, out=None):
    """a (..., K) @ w (K, N) + bias (N) -> (..., N) fp16 (fp32 accumulation)."""
    return _gemm(a, w, bias, _lib.EPI_BIAS, out=out)


def gemm_bias_gelu(a, w, bias=None, mode: str = "erf", out=None):
    """GEMM + bias + GELU in one kernel; mode "erf" (F.gelu, src/benchmk_end2end.py:81) or
    "tanh" (src/triton_template/gemm_gemm.py:146-150)."""
    if mode not in ("erf", "tanh"):
        raise _lib.StofError(f"gemm_bias_gelu: unknown mode {mode!r}")
    return _gemm(a, w, bias, _lib.EPI_BIAS_GELU_ERF if mode == "erf" else _lib.EPI_BIAS_GELU_TANH, out=out)


def gemm_bias_relu(a, w, bias=None, out=None):
    """GEMM + bias + ReLU in one kernel (the FFN activation of the T5 loops, src/benchmk_end2end.py:203,313)."""
    return _gemm(a, w, bias, _lib.EPI_BIAS_RELU, out=out)


def gemm_bias_act(a, w, bias=None, activation: str = "gelu_erf", out=None):
    """GEMM + bias + activation by name: "gelu_erf" (BERT), "gelu_tanh" (GPT-2 `new_gelu`), "relu" (T5), "none"."""
    epi = {"gelu_erf": _lib.EPI_BIAS_GELU_ERF, "erf": _lib.EPI_BIAS_GELU_ERF, "gelu_tanh": _lib.EPI_BIAS_GELU_TANH,
           "tanh": _lib.EPI_BIAS_GELU_TANH, "relu": _lib.EPI_BIAS_RELU, "none": _lib.EPI_BIAS}.get(activation)
    if epi is None:
        raise _lib.StofError(f"gemm_bias_act: unknown activation {activation!r}")
    return _gemm(a, w, bias, epi, out=out)


def gemm_bias_residual(a, w, bias, residual, out=None):
    """GEMM + bias + residual add in one kernel."""
    return _gemm(a, w, bias, _lib.EPI_BIAS_RESIDUAL, residual=residual, out=out)


def bias_residual_layernorm(x, bias=None, residual=None, gamma=None, beta=None, eps: float = 1e-5, out=None):
    """y = LayerNorm(x + bias + residual) * gamma + beta over the last dimension, one pass over HBM."""
    _lib.require_cuda(x, bias, residual, gamma, beta, out)
    if x.dtype != torch.float16:
        raise _lib.StofError("layernorm: float16 input expected")
    x2 = _as_rows(x)
    rows, hidden = x2.shape
    r2, ldr = None, 0
    if residual is not None:
        r2 = _as_rows(residual)
        if r2.shape != x2.shape or r2.dtype != torch.float16:
            raise _lib.StofError("layernorm: residual must be float16 of the input's shape")
        ldr = r2.stride(0)
    vecs = []
    for v in (bias, gamma, beta):
        if v is not None:
            v = v.reshape(-1).contiguous()
            if v.numel() != hidden or v.dtype != torch.float16:
                raise _lib.StofError("layernorm: bias/gamma/beta must be float16 vectors of length hidden")
        vecs.append(v)
    if out is None:
        out = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    elif out.dtype != torch.float16 or out.numel() != rows * hidden or out.shape[-1] != hidden:
        raise _lib.StofError(f"layernorm: out must be float16 of shape {tuple(x.shape)}")
    y2 = out.reshape(-1, hidden)
    if y2.data_ptr() != out.data_ptr() or y2.stride(1) != 1:
        raise _lib.StofError("layernorm: output must be viewable as contiguous rows")
    dev = x.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        rc = L.stof_bias_residual_layernorm(_lib.ptr(x2), x2.stride(0), _lib.ptr(vecs[0]), _lib.ptr(r2), ldr, _lib.ptr(vecs[1]),
                                            _lib.ptr(vecs[2]), float(eps), _lib.ptr(y2), y2.stride(0), rows, hidden,
                                            _lib.ptr(_lib.status_word(dev)), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_bias_residual_layernorm")
    return out


def gemm_bias_residual_layernorm(a, w, bias, residual, gamma, beta, eps: float, out=None):
    """LayerNorm(a @ w + bias + residual) * gamma + beta (src/benchmk_end2end.py:73-76, 83-86; the statistics inside the GEMM
    kernel as in src/triton_template/gemm_add_layernorm.py:77-123): for N a multiple of 256 up to 1024 and K <= 2048 ONE tcgen05
    kernel whose epilogue takes the row statistics across a cluster of thread blocks (`stof_gemm_bias_residual_layernorm`); other
    shapes run the GEMM with the bias + residual epilogue and the LayerNorm kernel in place, behind the same entry point.
    bias, residual, gamma, beta may be None."""
    _lib.require_cuda(a, w, bias, residual, gamma, beta, out)
    if a.dtype != torch.float16 or w.dtype != torch.float16 or w.dim() != 2:
        raise _lib.StofError("gemm+layernorm: float16 operands and a (K, N) weight expected")
    a2 = _as_rows(a)
    if w.stride(1) != 1:
        w = w.contiguous()
    M, K = a2.shape
    K2, N = w.shape
    if K != K2:
        raise _lib.StofError(f"gemm+layernorm: inner dimensions differ ({K} vs {K2})")
    vecs = []
    for v in (bias, gamma, beta):
        if v is not None:
            v = v.reshape(-1).contiguous()
            if v.numel() != N or v.dtype != torch.float16:
                raise _lib.StofError("gemm+layernorm: bias/gamma/beta must be float16 vectors of length N")
        vecs.append(v)
    out_shape = tuple(a.shape[:-1]) + (N,)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.float16, device=a.device)
    elif out.dtype != torch.float16 or out.numel() != M * N or out.shape[-1] != N:
        raise _lib.StofError(f"gemm+layernorm: out must be float16 of shape {out_shape}")
    c2 = out.reshape(-1, N)
    if c2.data_ptr() != out.data_ptr() or c2.stride(1) != 1:
        raise _lib.StofError("gemm+layernorm: output must be viewable as contiguous rows")
    r2, ldr = None, 0
    if residual is not None:
        r2 = _as_rows(residual)
        if r2.shape != (M, N) or r2.dtype != torch.float16:
            raise _lib.StofError("gemm+layernorm: residual must be float16 of the output's shape")
        ldr = r2.stride(0)
    dev = a.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        rc = L.stof_gemm_bias_residual_layernorm(_lib.ptr(a2), a2.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(vecs[0]), _lib.ptr(r2), ldr,
                                                 _lib.ptr(vecs[1]), _lib.ptr(vecs[2]), float(eps), _lib.ptr(c2), c2.stride(0), M, N, K,
                                                 _lib.ptr(_lib.status_word(dev)), _lib.current_stream_ptr(dev))
    _lib.check(rc, "stof_gemm_bias_residual_layernorm")
    return out


def gemm_bias_residual_then_layernorm(a, w, bias, residual, gamma, beta, eps: float, out=None):
    """The same result from two kernels: tcgen05 GEMM with the bias + residual epilogue (fp16 out), then the one-pass LayerNorm
    kernel in place.  Kept for comparison with the fused form (it rounds the GEMM output to fp16 before the statistics)."""
    x = gemm_bias_residual(a, w, bias, residual, out=out) if residual is not None else gemm_bias(a, w, bias, out=out)
    return bias_residual_layernorm(x, None, None, gamma, beta, eps, out=x)


# ------------------------------------------------------------------------------------------
# Operators with the signatures of the reference's Triton templates
# ------------------------------------------------------------------------------------------
def matmul_bias_layernorm(A, B, bias, eps: float = 1e-5):
    """`triton_matmul_bias_layernorm(A, B, bias, eps)` (src/triton_template/gemm_add_layernorm.py:126-144):
    C[b] = normalise_rows(A[b] @ B[b] + bias[:N]), no gamma/beta.  A (batch,M,K), B (batch,K,N);
    a batch-expanded weight (stride 0) runs as one GEMM over batch*M rows."""
    batch, M, K = A.shape
    _, Kb, N = B.shape
    if K != Kb:
        raise _lib.StofError(f"matmul_bias_layernorm: K mismatch ({K} vs {Kb})")
    bvec = bias.reshape(-1)[:N].contiguous()
    C = torch.empty(batch, M, N, dtype=A.dtype, device=A.device)
    if B.stride(0) == 0 or batch == 1:
        gemm_bias_residual_layernorm(A, B[0], bvec, None, None, None, eps, out=C)
    else:
        for b in range(batch):
            gemm_bias_residual_layernorm(A[b], B[b], bvec, None, None, None, eps, out=C[b])
    return C


def matmul_gelu_matmul(a, b, d, bias):
    """`triton_matmul_batch(a, b, d, bias)` (src/triton_template/gemm_gemm.py:158-174):
    gelu_tanh(a @ b + bias[:N]) @ d with the intermediate rounded to fp16.  a (batch,M,K), b (K,N), d (N,H).
    Two back-to-back tcgen05 GEMMs; the (batch*M, N) intermediate stays in L2 for typical FFN sizes."""
    N = b.shape[-1]
    t = gemm_bias_gelu(a, b, bias.reshape(-1)[:N].contiguous(), mode="tanh")
    return gemm_bias(t, d, None)


def batched_bias_layernorm(x, bias, weight, bias_ln, eps: float = 1e-5):
    """`triton_batched_bias_layernorm(x, bias, weight, bias_ln, eps)`
    (src/triton_template/add_layernorm.py:86-107): LN(x + bias) * weight + bias_ln."""
    return bias_residual_layernorm(x, bias, None, weight, bias_ln, eps)
