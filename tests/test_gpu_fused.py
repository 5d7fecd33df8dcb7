"""tcgen05 GEMM epilogues, LayerNorm and the encoder layer against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import fused as of
from oracle import masks as om
from _cases import GOLDEN

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).half()


def _err(a, b):
    return (a.float().cpu() - b).abs().max().item()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 128), (300, 264, 200), (1000, 768, 768), (64, 3072, 768), (2048, 1024, 4096), (1, 8, 8)])
def test_gemm_bias_matches_oracle(m, n, k):
    import stof_b200
    a, w, b = _rand((m, k), 1), _rand((k, n), 2, 0.05), _rand((n,), 3)
    got = stof_b200.gemm_bias(a.cuda(), w.cuda(), b.cuda())
    torch.cuda.synchronize()
    want = of.gemm_bias(a, w, b)
    # fp32 accumulation, one fp16 rounding of the result: half an ulp of the largest magnitude plus summation noise
    tol = 2e-3 * max(1.0, want.abs().max().item())
    assert _err(got, want) <= tol


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 512, 200), (1000, 768, 768), (2048, 1024, 1024), (37 * 256 + 129, 1024, 72),
                                   (49 * 128 * 2 + 5, 768, 64), (513, 1024, 2048), (513, 1024, 4096), (300, 264, 200), (256, 1280, 128)])
def test_gemm_with_layernorm_epilogue(m, n, k):
    """LayerNorm(a @ w + bias + residual) * gamma + beta: for n in {256, 512, 768, 1024} one kernel whose thread blocks exchange
    row statistics across a cluster (1, 2, 3, 4 blocks; one and several row blocks per cluster; ragged last row block; K not a
    multiple of the stage), for other n and for K > 2048 the two-kernel path behind the same entry point.  Random gamma / beta, and the operands
    left out one by one.  Against the fp32 oracle and, loosely, against the two-kernel path."""
    import stof_b200
    a, w, b, r = _rand((m, k), 31), _rand((k, n), 32, 0.1), _rand((n,), 33), _rand((m, n), 34)
    gam, bet = (_rand((n,), 35, 0.3).float() + 1).half(), _rand((n,), 36, 0.3)
    ad, wd, bd, rd, gd, btd = (t.cuda() for t in (a, w, b, r, gam, bet))
    want = of.gemm_bias_residual_layernorm(a, w, b, r, gam, bet, 1e-12)
    tol = 2e-3 * max(1.0, want.abs().max().item())
    got = stof_b200.gemm_bias_residual_layernorm(ad, wd, bd, rd, gd, btd, 1e-12)
    torch.cuda.synchronize()
    from stof_b200 import _lib
    _lib.check_status(got.device, "gemm + layernorm")
    assert _err(got, want) <= tol
    two = stof_b200.gemm_bias_residual_then_layernorm(ad, wd, bd, rd, gd, btd, 1e-12)
    assert _err(two, want) <= 2 * tol and (got.float() - two.float()).abs().max().item() <= 3 * tol
    # operands left out: no residual, no affine, no bias
    zero_r, one_g, zero_b = torch.zeros_like(r), torch.ones_like(gam), torch.zeros_like(bet)
    got = stof_b200.gemm_bias_residual_layernorm(ad, wd, bd, None, gd, btd, 1e-5)
    assert _err(got, of.gemm_bias_residual_layernorm(a, w, b, zero_r, gam, bet, 1e-5)) <= tol
    got = stof_b200.gemm_bias_residual_layernorm(ad, wd, None, rd, None, None, 1e-5)
    assert _err(got, of.gemm_bias_residual_layernorm(a, w, torch.zeros_like(b), r, one_g, zero_b, 1e-5)) <= tol
    # in place over the residual, as the encoder never does but the signature allows for a caller that owns both
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    assert stof_b200.gemm_bias_residual_layernorm(ad, wd, bd, rd, gd, btd, 1e-12, out=out).data_ptr() == out.data_ptr()
    assert _err(out, want) <= tol


def test_layernorm_epilogue_rows_with_a_large_common_offset():
    """Rows whose mean is far larger than their spread: the row statistics are merged from per-thread means and centred sums of
    squares, so nothing is lost to cancellation."""
    import stof_b200
    if os.environ.get("STOF_B200_GEMM_LN", "").startswith("s"):
        pytest.skip("the two-kernel path rounds the GEMM output to fp16 before the statistics; this case is about the fused one")
    m, n, k = 256, 1024, 64
    a, w = _rand((m, k), 41, 0.1), _rand((k, n), 42, 0.1)
    r = (_rand((m, n), 43, 0.5).float() + 60.0).half()
    got = stof_b200.gemm_bias_residual_layernorm(a.cuda(), w.cuda(), None, r.cuda(), None, None, 1e-12)
    torch.cuda.synchronize()
    want = of.gemm_bias_residual_layernorm(a, w, torch.zeros(n).half(), r, torch.ones(n).half(), torch.zeros(n).half(), 1e-12)
    assert _err(got, want) <= 4e-3


@pytest.mark.parametrize("mode", ["erf", "tanh"])
def test_gemm_bias_gelu(mode):
    import stof_b200
    a, w, b = _rand((512, 256), 4), _rand((256, 1024), 5, 0.1), _rand((1024,), 6)
    got = stof_b200.gemm_bias_gelu(a.cuda(), w.cuda(), b.cuda(), mode)
    torch.cuda.synchronize()
    want = of.gemm_bias_gelu(a, w, b, mode)
    assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("m,n,k", [(4096, 2560, 136), (4136, 2568, 72), (37 * 256 + 129, 1024, 64)])
def test_large_gemm_on_block_pairs_every_epilogue(m, n, k):
    """Shapes with at least two 256 x 256 tiles per pair of SMs run on the two-block (cta_group::2) kernel: every epilogue,
    ragged edges in both directions (a last tile whose second block has no rows at all, or only one), a K that is not a
    multiple of the 64-wide stage, and a GELU check against erf on values across the polynomial's whole range."""
    import stof_b200
    a, w, b, r = _rand((m, k), 11), _rand((k, n), 12, 0.1), _rand((n,), 13), _rand((m, n), 14)
    ad, wd, bd, rd = a.cuda(), w.cuda(), b.cuda(), r.cuda()
    base = of.gemm_bias(a, w, b)
    tol = 2e-3 * max(1.0, base.abs().max().item())
    assert _err(stof_b200.gemm_bias(ad, wd, bd), base) <= tol
    assert _err(stof_b200.gemm_bias_residual(ad, wd, bd, rd), base + r.float()) <= 2 * tol
    assert _err(stof_b200.gemm_bias_relu(ad, wd, bd), torch.relu(base)) <= tol
    for mode in ("erf", "tanh"):
        assert _err(stof_b200.gemm_bias_gelu(ad, wd, bd, mode), of.gemm_bias_gelu(a, w, b, mode)) <= tol
    wide = _rand((m, k), 15, 4.0)                                          # pre-activations well beyond +-4.5
    want = of.gemm_bias_gelu(wide, w, b, "erf")
    assert _err(stof_b200.gemm_bias_gelu(wide.cuda(), wd, bd, "erf"), want) <= 2e-3 * max(1.0, want.abs().max().item())
    torch.cuda.synchronize()
    from stof_b200 import _lib
    _lib.check_status(torch.device("cuda:0"), "pair gemm")


def test_gemm_bias_residual_and_3d_inputs():
    import stof_b200
    a, w, b, r = _rand((4, 96, 128), 7), _rand((128, 256), 8, 0.1), _rand((256,), 9), _rand((4, 96, 256), 10)
    got = stof_b200.gemm_bias_residual(a.cuda(), w.cuda(), b.cuda(), r.cuda())
    torch.cuda.synchronize()
    want = of.gemm_bias(a, w, b) + r.float()
    assert got.shape == (4, 96, 256) and _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("hidden", [64, 256, 768, 1024, 1536, 4096])
def test_layernorm_with_bias_and_residual(hidden):
    import stof_b200
    x, bias, res = _rand((37, hidden), 11), _rand((hidden,), 12), _rand((37, hidden), 13)
    gamma, beta = _rand((hidden,), 14, 0.3) + 1, _rand((hidden,), 15, 0.3)
    for eps in (1e-5, 1e-12):
        got = stof_b200.bias_residual_layernorm(x.cuda(), bias.cuda(), res.cuda(), gamma.cuda(), beta.cuda(), eps)
        torch.cuda.synchronize()
        want = torch.nn.functional.layer_norm(x.float() + bias.float() + res.float(), (hidden,), gamma.float(), beta.float(), eps)
        assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())
    got = stof_b200.bias_residual_layernorm(x.cuda())
    want = torch.nn.functional.layer_norm(x.float(), (hidden,), None, None, 1e-5)
    assert _err(got, want) <= 3e-3


def test_reference_fused_operator_signatures():
    from triton_template.add_layernorm import triton_batched_bias_layernorm
    from triton_template.gemm_add_layernorm import triton_matmul_bias_layernorm
    from triton_template.gemm_gemm import triton_matmul_batch
    B, M, K, N = 2, 128, 256, 512
    A, W, bias = _rand((B, M, K), 20), _rand((K, N), 21, 0.1), _rand((N,), 22)
    got = triton_matmul_bias_layernorm(A.cuda(), W.cuda().unsqueeze(0).expand(B, -1, -1), bias.cuda())
    want = of.matmul_bias_layernorm(A, W.unsqueeze(0).expand(B, -1, -1), bias)
    assert _err(got, want) <= 4e-3
    Wb = _rand((B, K, N), 23, 0.1)
    got = triton_matmul_bias_layernorm(A.cuda(), Wb.cuda(), bias.cuda(), 1e-6)
    assert _err(got, of.matmul_bias_layernorm(A, Wb, bias, 1e-6)) <= 4e-3
    d = _rand((N, K), 24, 0.05)
    got = triton_matmul_batch(A.cuda(), W.cuda(), d.cuda(), bias.cuda())
    want = of.matmul_gelu_matmul(A, W, d, bias)
    assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())
    x, w, b = _rand((B, M, N), 25), _rand((N,), 26), _rand((N,), 27)
    got = triton_batched_bias_layernorm(x.cuda(), bias.cuda(), w.cuda(), b.cuda())
    assert _err(got, of.bias_layernorm(x, bias, w, b)) <= 4e-3


def test_encoder_layer_against_reference_function_fixture():
    """One BERT layer on the inputs of the fixture produced by the reference's bert_fwd_std (eps 1e-5, causal mask)."""
    import stof_b200
    z = np.load(os.path.join(GOLDEN, "bert_layer.npz"))
    params = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("p_")}
    hidden = torch.from_numpy(z["hidden16"])
    B, S, hid = hidden.shape
    enc = stof_b200.BertEncoder([stof_b200.EncoderWeights.from_dict(params, "cuda")], head_num=2, eps=1e-5, block_m=32, block_n=32)
    enc.set_mask(torch.tril(torch.ones(1, S, S)).cuda())
    got = enc(hidden.cuda())
    torch.cuda.synchronize()
    # post-LN outputs are O(1..4); tolerance = the task's 2e-3 scaled by the output magnitude (fp16 ulp grows with it)
    want = torch.from_numpy(z["out_f32"])
    assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())


def test_encoder_config4_shape_one_layer_slice():
    """BERT-base layer (hidden 768, 12 heads, FFN 3072, eps 1e-12, sliding +-2 blocks) on 2 sequences of 1024."""
    import stof_b200
    B, S, hid, heads, ffn = 2, 1024, 768, 12, 3072
    params = of.make_bert_params(hid, ffn, 1, seed=3)
    g = torch.Generator().manual_seed(3)
    hidden = torch.randn(B, S, hid, generator=g).half()
    mask = om.recipe_mask("cfg4_sliding2_S1024")
    enc = stof_b200.BertEncoder([stof_b200.EncoderWeights.from_dict(params[0], "cuda")], head_num=heads, eps=1e-12)
    enc.set_mask(torch.from_numpy(mask).cuda())
    got = enc(hidden.cuda())
    torch.cuda.synchronize()
    want = of.bert_layer(hidden, params[0], torch.from_numpy(mask.astype(np.float32)), heads, eps=1e-12)
    assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())


def test_two_layer_encoder_random_affine():
    """Two stacked layers with random gamma/beta/biases, BigBird-style block mask with a partial (causal) variant."""
    import stof_b200
    B, S, hid, heads, ffn = 2, 256, 256, 4, 512
    params = of.make_bert_params(hid, ffn, 2, seed=9, random_affine=True)
    g = torch.Generator().manual_seed(9)
    hidden = torch.randn(B, S, hid, generator=g).half()
    mask = om.generate_sliding_mask(1, S, 70, False, np.float16)
    enc = stof_b200.BertEncoder([stof_b200.EncoderWeights.from_dict(p, "cuda") for p in params], head_num=heads, eps=1e-12)
    enc.set_mask(torch.from_numpy(mask).cuda())
    got = enc(hidden.cuda()).clone()
    torch.cuda.synchronize()
    want = of.encoder_forward(hidden, params, torch.from_numpy(mask.astype(np.float32)), heads, 1e-12)
    assert _err(got, want) <= 3e-3 * max(1.0, want.abs().max().item())     # two layers of fp16 storage
    # deterministic, buffers reused (the second use of the block index may re-pair its halves, which changes the order of the
    # attention's partial sums and with it the last bit; from then on every pass is bit-identical)
    again = enc(hidden.cuda()).clone()
    assert _err(again, want) <= 3e-3 * max(1.0, want.abs().max().item())
    assert torch.equal(enc(hidden.cuda()), again)


def test_gemm_bias_relu():
    import stof_b200
    a, w, b = _rand((300, 200), 5), _rand((200, 264), 6, 0.1), _rand((264,), 7)
    got = stof_b200.gemm_bias_relu(a.cuda(), w.cuda(), b.cuda())
    want = torch.relu(of.gemm_bias(a, w, b))
    assert _err(got, want) <= 2e-3 * max(1.0, want.abs().max().item())
    assert (got >= 0).all()


@pytest.mark.parametrize("activation", ["tanh", "relu"])
def test_gpt2_and_t5_encoder_layers(activation):
    """The GPT-2 loop (tanh GELU, causal mask) and the T5 encoder loop (ReLU) are the BERT layer with another activation."""
    import stof_b200
    B, S, hid, heads, ffn = 2, 256, 256, 4, 1024
    params = of.make_bert_params(hid, ffn, 2, seed=21, random_affine=True)
    hidden = _rand((B, S, hid), 22)
    mask = om.generate_causal_mask(1, S).astype(np.float16) if activation == "tanh" else om.generate_sliding_mask(1, S, 40, False, np.float16)
    make = stof_b200.gpt2_stack if activation == "tanh" else stof_b200.t5_encoder_stack
    model = make([stof_b200.EncoderWeights.from_dict(p, "cuda") for p in params], heads, 1e-5, 32, 32)
    model.set_mask(torch.from_numpy(mask).cuda())
    got = model(hidden.cuda())
    torch.cuda.synchronize()
    want = of.encoder_forward(hidden, params, torch.from_numpy(mask.astype(np.float32)), heads, 1e-5, activation)
    assert _err(got, want) <= 3e-3 * max(1.0, want.abs().max().item())


def test_t5_decoder_layer():
    """Two attention sublayers + ReLU feed-forward (the decoder loop of the reference's T5 forward) on a causal mask."""
    import stof_b200
    B, S, hid, heads, ffn = 2, 256, 256, 4, 512
    params = of.make_t5_decoder_params(hid, ffn, seed=31)
    hidden = _rand((B, S, hid), 32)
    mask = om.generate_causal_mask(1, S).astype(np.float16)
    dec = stof_b200.T5Decoder([stof_b200.T5DecoderWeights.from_dict(params, "cuda")], heads, 1e-5, 32, 32)
    dec.set_mask(torch.from_numpy(mask).cuda())
    got = dec(hidden.cuda())
    torch.cuda.synchronize()
    want = of.t5_decoder_layer(hidden, params, torch.from_numpy(mask.astype(np.float32)), heads, 1e-5)
    assert _err(got, want) <= 3e-3 * max(1.0, want.abs().max().item())


def test_encoder_config5_shapes_batch_independence():
    """BERT-large shapes of configuration 5 (hidden 1024, 16 heads, FFN 4096, S = 4096, BigBird block mask, eps 1e-12) at
    full sequence length: three layers on four sequences; every sequence is an independent shard, so running two of them
    alone gives bit-identical rows (the property the multi-GPU batch sharding rests on), the result is finite and a second
    run reproduces it; the first layer of one sequence is compared with the fp32 oracle on a sample of rows."""
    import stof_b200
    B, S, hid, heads, ffn = 4, 4096, 1024, 16, 4096
    params = of.make_bert_params(hid, ffn, 3, seed=4)
    g = torch.Generator().manual_seed(4)
    hidden = torch.randn(B, S, hid, generator=g).half()
    mask = om.recipe_mask("cfg5_bigbird_S4096_seed4")
    layers = [stof_b200.EncoderWeights.from_dict(p, "cuda") for p in params]
    enc = stof_b200.BertEncoder(layers, head_num=heads, eps=1e-12)
    enc.set_mask(torch.from_numpy(mask).cuda())
    full = enc(hidden.cuda()).clone()
    torch.cuda.synchronize()
    assert torch.isfinite(full.float()).all()
    assert torch.equal(enc(hidden.cuda()), full)
    part = stof_b200.BertEncoder(layers, head_num=heads, eps=1e-12)
    part.set_mask(torch.from_numpy(mask).cuda())
    assert torch.equal(part(hidden[1:3].cuda()), full[1:3])
    # one layer, one sequence against the oracle (dense fp32 attention of a 4096 x 4096 score matrix per head on the CPU)
    one = stof_b200.BertEncoder(layers[:1], head_num=heads, eps=1e-12)
    one.set_mask(torch.from_numpy(mask).cuda())
    got = one(hidden[:1].cuda())
    torch.cuda.synchronize()
    want = of.bert_layer(hidden[:1], params[0], torch.from_numpy(mask.astype(np.float32)), heads, eps=1e-12)
    rows = torch.arange(0, S, 37)
    assert _err(got[:, rows], want[:, rows]) <= 2e-3 * max(1.0, want.abs().max().item())


def test_encoder_forward_captured_in_a_cuda_graph():
    """`BertEncoder.capture`: a replayed graph of the forward pass gives the eager result, also after the input buffer has
    been refilled in place."""
    import stof_b200
    B, S, hid, heads, ffn = 2, 512, 256, 4, 1024
    params = of.make_bert_params(hid, ffn, 2, seed=41, random_affine=True)
    enc = stof_b200.BertEncoder([stof_b200.EncoderWeights.from_dict(p, "cuda") for p in params], head_num=heads, eps=1e-12)
    enc.set_mask(torch.from_numpy(om.generate_sliding_mask(1, S, 100, False, np.float16)).cuda())
    x = _rand((B, S, hid), 42).cuda()
    enc(x)                                              # first pass: the block index is planned, and re-planned at its second use
    eager = enc(x).clone()
    replay = enc.capture(x)
    assert torch.equal(replay(), eager)
    x2 = _rand((B, S, hid), 43).cuda()
    want2 = enc(x2).clone()
    x.copy_(x2)
    assert torch.equal(replay(), want2)
    from stof_b200 import _lib
    _lib.check_status(x.device, "graph replay")
