"""Oracle (test infrastructure): the fused GEMM / LayerNorm operators and the BERT
encoder layer, restated with CPU PyTorch in fp32.  Nothing in the shipped CUDA
path imports this file.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """tanh-form GELU as the reference's fused kernel evaluates it
    (src/triton_template/gemm_gemm.py:146-150)."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def gemm_bias(a, w, bias) -> torch.Tensor:
    """a (..., K) @ w (K, N) + bias (N) in fp32 (src/benchmk_end2end.py:73,80,83)."""
    return torch.matmul(a.float(), w.float()) + bias.float()


def gemm_bias_gelu(a, w, bias, mode: str = "erf") -> torch.Tensor:
    """GEMM + bias followed by GELU: erf form as `F.gelu` (src/benchmk_end2end.py:80-81)
    or tanh form (src/triton_template/gemm_gemm.py:146-150)."""
    x = gemm_bias(a, w, bias)
    return F.gelu(x) if mode == "erf" else gelu_tanh(x)


def gemm_bias_residual_layernorm(a, w, bias, residual, gamma, beta, eps: float) -> torch.Tensor:
    """LayerNorm(a @ w + bias + residual) * gamma + beta over the last dim
    (src/benchmk_end2end.py:73-76, 83-86)."""
    x = gemm_bias(a, w, bias) + residual.float()
    return F.layer_norm(x, (x.shape[-1],), gamma.float(), beta.float(), eps)


def matmul_bias_layernorm(A, B, bias, eps: float = 1e-5) -> torch.Tensor:
    """Semantics of `triton_matmul_bias_layernorm`: C[b] = normalise_rows(A[b] @ B[b] + bias[:N])
    without gamma/beta, biased variance (src/triton_template/gemm_add_layernorm.py:77-144)."""
    n = B.shape[-1]
    x = torch.matmul(A.float(), B.float()) + bias.reshape(-1)[:n].float()
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps)


def matmul_gelu_matmul(a, b, d, bias) -> torch.Tensor:
    """Semantics of `triton_matmul_batch`: gelu_tanh(a @ b + bias) rounded to fp16, then @ d
    (src/triton_template/gemm_gemm.py:99-174).  a (B,M,K), b (K,N), d (N,H), bias (N)."""
    t = gelu_tanh(torch.matmul(a.float(), b.float()) + bias.reshape(-1)[: b.shape[-1]].float())
    return torch.matmul(t.half().float(), d.float())


def bias_layernorm(x, bias, weight, bias_ln, eps: float = 1e-5) -> torch.Tensor:
    """Semantics of `triton_batched_bias_layernorm`: LN(x + bias) * weight + bias_ln
    (src/triton_template/add_layernorm.py:19-107)."""
    y = x.float() + bias.float()
    return F.layer_norm(y, (y.shape[-1],), weight.float(), bias_ln.float(), eps)


def bert_layer(hidden, params: dict, mask, head_num: int, eps: float = 1e-5, qkv_from_gemm: bool = True,
               gelu_mode: str = "erf") -> torch.Tensor:
    """One post-LN BERT layer (src/benchmk_end2end.py:31-88) in fp32, with the QKV
    projection `hidden @ Wqkv + bqkv` in front as in src/model-candidate/1-BERT-large.py:17-18.

    params: Wqkv (hid,3hid), bqkv, Wo (hid,hid), bo, g1, b1, W1 (hid,ffn), bi1, W2 (ffn,hid), bi2, g2, b2.
    mask: (1 or B, S, S) 0/1.  Attention is the reference's torch-native branch (:44-52).
    With qkv_from_gemm=False `params['qkv']` holds the ready (B,S,3hid) activation that the
    reference script itself uses in place of the GEMM (:37)."""
    x = hidden.float()
    B, S, hid = x.shape
    hs = hid // head_num
    if qkv_from_gemm:
        qkv = torch.matmul(x, params["Wqkv"].float()) + params["bqkv"].float()
    else:
        qkv = params["qkv"].float() + params["bqkv"].float()
    q, k, v = qkv.chunk(3, dim=-1)

    def heads(t):
        return t.reshape(B, S, head_num, hs).permute(0, 2, 1, 3)

    q, k, v = heads(q), heads(k), heads(v)
    scores = torch.matmul(q, k.transpose(-2, -1)) / (hs ** .5)
    scores = scores - 10000.0 * (1.0 - torch.as_tensor(mask).float().unsqueeze(1))
    h = torch.matmul(F.softmax(scores, dim=-1), v)
    h = h.permute(0, 2, 1, 3).reshape(B, S, hid)
    y = torch.matmul(h, params["Wo"].float()) + params["bo"].float() + x
    y = F.layer_norm(y, (hid,), params["g1"].float(), params["b1"].float(), eps)
    z = torch.matmul(y, params["W1"].float()) + params["bi1"].float()
    z = _activation(z, gelu_mode)
    z = torch.matmul(z, params["W2"].float()) + params["bi2"].float() + y
    return F.layer_norm(z, (hid,), params["g2"].float(), params["b2"].float(), eps)


def _activation(z: torch.Tensor, mode: str) -> torch.Tensor:
    """FFN activation of the three model loops: "erf" = F.gelu (BERT, src/benchmk_end2end.py:81), "tanh" = `new_gelu`
    (GPT-2, :142), "relu" = F.relu (T5, :203 and :313)."""
    if mode == "erf":
        return F.gelu(z)
    if mode == "tanh":
        return gelu_tanh(z)
    if mode == "relu":
        return F.relu(z)
    raise ValueError(mode)


def _attention_fp32(x, Wqkv, bqkv, mask, head_num: int) -> torch.Tensor:
    """QKV projection + the reference's torch-native attention branch (src/benchmk_end2end.py:44-52), merged heads."""
    B, S, hid = x.shape
    hs = hid // head_num
    qkv = torch.matmul(x, Wqkv.float()) + bqkv.float()
    q, k, v = (t.reshape(B, S, head_num, hs).permute(0, 2, 1, 3) for t in qkv.chunk(3, dim=-1))
    scores = torch.matmul(q, k.transpose(-2, -1)) / (hs ** .5)
    scores = scores - 10000.0 * (1.0 - torch.as_tensor(mask).float().unsqueeze(1))
    return torch.matmul(F.softmax(scores, dim=-1), v).permute(0, 2, 1, 3).reshape(B, S, hid)


def t5_decoder_layer(hidden, params: dict, mask, head_num: int, eps: float = 1e-5) -> torch.Tensor:
    """One decoder layer of the reference's T5 loop (src/benchmk_end2end.py:230-316) in fp32: masked self-attention,
    out-projection + residual + LayerNorm, a second attention sublayer whose Q, K and V all come from the decoder state
    (the loop projects `decoder_hidden_states` with `qkv_kernel_3`, :263-268), out-projection + residual + LayerNorm,
    and the ReLU feed-forward + residual + LayerNorm.  The first sublayer's QKV is projected from the layer input here
    (the script feeds a ready activation in place of that GEMM, :232).

    params: Wqkv_a, bqkv_a, Wo_a, bo_a, g_a, b_a (first attention), Wqkv_c, bqkv_c, Wo_c, bo_c, g_c, b_c (second),
    W1, bi1, W2, bi2, g2, b2 (feed-forward)."""
    x = hidden.float()
    hid = x.shape[-1]
    f = lambda k: params[k].float()
    h = _attention_fp32(x, params["Wqkv_a"], params["bqkv_a"], mask, head_num)
    y = F.layer_norm(torch.matmul(h, f("Wo_a")) + f("bo_a") + x, (hid,), f("g_a"), f("b_a"), eps)
    h = _attention_fp32(y, params["Wqkv_c"], params["bqkv_c"], mask, head_num)
    y2 = F.layer_norm(torch.matmul(h, f("Wo_c")) + f("bo_c") + y, (hid,), f("g_c"), f("b_c"), eps)
    z = F.relu(torch.matmul(y2, f("W1")) + f("bi1"))
    z = torch.matmul(z, f("W2")) + f("bi2") + y2
    return F.layer_norm(z, (hid,), f("g2"), f("b2"), eps)


def make_t5_decoder_params(hidden: int, ffn: int, seed: int, dtype=torch.float16):
    """Seeded CPU weights of one decoder layer: W ~ N(0, 0.02), biases and affine terms uniform(-0.4, 0.4) around 0 / 1
    (src/benchmk_end2end.py:453-454).  Draw order = the order of the `params` list in `t5_decoder_layer`."""
    g = torch.Generator().manual_seed(seed)
    w = lambda *shape: (torch.randn(*shape, generator=g) * 0.02).to(dtype)
    u = lambda n, base: (base + (torch.rand(n, generator=g) * 0.8 - 0.4) * 0.25).to(dtype)
    p = {}
    for tag in ("a", "c"):
        p["Wqkv_" + tag] = w(hidden, 3 * hidden); p["bqkv_" + tag] = u(3 * hidden, 0.0)
        p["Wo_" + tag] = w(hidden, hidden); p["bo_" + tag] = u(hidden, 0.0)
        p["g_" + tag] = u(hidden, 1.0); p["b_" + tag] = u(hidden, 0.0)
    p["W1"] = w(hidden, ffn); p["bi1"] = u(ffn, 0.0); p["W2"] = w(ffn, hidden); p["bi2"] = u(hidden, 0.0)
    p["g2"] = u(hidden, 1.0); p["b2"] = u(hidden, 0.0)
    return p


def make_bert_params(hidden: int, ffn: int, layers: int, seed: int, dtype=torch.float16, random_affine: bool = False):
    """Seeded CPU weights: W ~ N(0, 0.02), biases 0, gamma 1, beta 0 (BERT init).  Draw order
    per layer: Wqkv, bqkv, Wo, bo, g1, b1, W1, bi1, W2, bi2, g2, b2 (biases and affine terms
    consume no random numbers unless `random_affine`, which draws them uniform(-0.4, 0.4)
    like src/benchmk_end2end.py:453-454)."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(dtype)

    def aff(n, base):
        if random_affine:
            return (torch.rand(n, generator=g) * 0.8 - 0.4 + base).to(dtype)
        return torch.full((n,), float(base)).to(dtype)

    out = []
    for _ in range(layers):
        p = {}
        p["Wqkv"] = w(hidden, 3 * hidden); p["bqkv"] = aff(3 * hidden, 0)
        p["Wo"] = w(hidden, hidden); p["bo"] = aff(hidden, 0)
        p["g1"] = aff(hidden, 1); p["b1"] = aff(hidden, 0)
        p["W1"] = w(hidden, ffn); p["bi1"] = aff(ffn, 0)
        p["W2"] = w(ffn, hidden); p["bi2"] = aff(hidden, 0)
        p["g2"] = aff(hidden, 1); p["b2"] = aff(hidden, 0)
        out.append(p)
    return out


def encoder_forward(hidden, layers_params, mask, head_num: int, eps: float, gelu_mode: str = "erf",
                    round_fp16_between_layers: bool = True) -> torch.Tensor:
    """Stack of `bert_layer`.  Activations are rounded to fp16 between layers when
    `round_fp16_between_layers` (the storage type of the reference path)."""
    x = hidden
    for p in layers_params:
        x = bert_layer(x, p, mask, head_num, eps, True, gelu_mode)
        if round_fp16_between_layers:
            x = x.half()
    return x.float()


def encoder_gemm_flops(tokens: int, hidden: int, ffn: int) -> float:
    """2*T*hidden*(3*hidden + hidden + ffn + ffn) per layer."""
    return 2.0 * tokens * hidden * (3 * hidden + hidden + 2 * ffn)
