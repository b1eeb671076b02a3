"""The single track on the GPU: pair-bias pass, dense-layer kernel, attention with pair bias, single transition and
the full PairformerLayerV1 / PairformerModule, against the oracle and the fixtures made from the reference modules."""

import math

import pytest
import torch
import torch.nn.functional as F

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200 import _lib, ops
from bionemo_inference_runtime_b200.layers.attention_pair_bias import fold_linear
from oracle import triangle_oracle as orc
from tests.helpers import golden_single_attention_weights, golden_single_transition_weights, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(rtol=2e-2, atol=2e-2)  # bf16 tolerance of the hot path


def _ok():
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def _attention_layer(w: orc.PairBiasAttentionWeights):
    layer = b200.AttentionPairBias(layer_idx=0, c_s=384, c_z=128, num_heads=16, dtype=torch.bfloat16, bias_proj=True,
                                   inf=1e9, initial_norm=w.norm_s_w is not None, out_bias=w.b_o is not None)
    sd = {"in_proj.weight": w.w_in, "in_proj.bias": w.b_in, "proj_z.0.weight": w.norm_z_w, "proj_z.0.bias": w.norm_z_b,
          "proj_z.1.weight": w.w_z, "proj_o.weight": w.w_o}
    if w.norm_s_w is not None:
        sd.update({"norm_s.weight": w.norm_s_w, "norm_s.bias": w.norm_s_b})
    if w.b_o is not None:
        sd["proj_o.bias"] = w.b_o
    layer.load_state_dict(sd, strict=True)
    return layer.to(DEV)


def _transition_layer(w: orc.TransitionWeights):
    layer = b200.Transition(384, 1536, dtype=torch.bfloat16)
    layer.load_state_dict({"norm.weight": w.ln_w, "norm.bias": w.ln_b, "fused_fc2_fc1.weight": w.w1, "fc3.weight": w.w2},
                          strict=True)
    return layer.to(DEV)


@pytest.mark.parametrize("B,Q,K,heads", [(1, 40, 40, 16), (2, 130, 130, 16), (1, 257, 263, 16), (1, 64, 72, 4)])
def test_pair_bias_pass_matches_layer_norm_projection_and_padding(B, Q, K, heads):
    g = torch.Generator().manual_seed(Q + K)
    z = torch.randn(B, Q, K, 128, generator=g).bfloat16().to(DEV)
    gamma, beta = (1 + 0.2 * torch.randn(128, generator=g)).to(DEV), (0.2 * torch.randn(128, generator=g)).to(DEV)
    w_z = (torch.randn(heads, 128, generator=g) * 0.05).to(DEV)
    scale = math.sqrt(24)
    bias = ops.pair_bias(z, ops.pack_pair_bias_weights(gamma, beta, w_z, scale), heads)
    _ok()
    assert tuple(bias.shape) == (B, heads, Q, ops.pad8(K))
    want = scale * F.linear(F.layer_norm(z.float(), (128,), gamma, beta), w_z).movedim(-1, 1)
    torch.testing.assert_close(bias[..., :K].float(), want, rtol=2e-2, atol=3e-2)
    assert not bias[..., K:].any()  # the key padding is written as zero


@pytest.mark.parametrize("rows,K,N", [(40, 384, 384), (300, 1536, 384), (129, 384, 3072)])
def test_dense_layer_kernel_row_and_swiglu_forms(rows, K, N):
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(2, rows, K, generator=g) + 0.3).bfloat16().to(DEV)
    w, b = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(DEV), torch.randn(N, generator=g).to(DEV)
    gamma, beta = (1 + 0.2 * torch.randn(K, generator=g)).to(DEV), (0.2 * torch.randn(K, generator=g)).to(DEV)
    res = torch.randn(2, rows, N, generator=g).bfloat16().to(DEV)
    # plain projection with bias and residual
    wq, sc = fold_linear(w, b, None, None)
    got = ops.linear(x, wq, sc, ops.LINEAR_ROWS, B=2, rows=rows, residual=res)
    _ok()
    torch.testing.assert_close(got.float(), F.linear(x.float(), wq.float(), b) + res.float(), **TOL)
    # LayerNorm folded in, statistics from the row-statistics kernel
    wq, sc = fold_linear(w, b, gamma, beta)
    stats = ops.row_stats(x)
    got = ops.linear(x, wq, sc, ops.LINEAR_ROWS, B=2, rows=rows, stats=stats)
    _ok()
    want = F.linear(F.layer_norm(x.float(), (K,), gamma, beta), w, b)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=4e-2)
    mean, var = x.float().mean(-1), x.float().var(-1, unbiased=False)
    torch.testing.assert_close(stats.view(2, rows, 2)[..., 0], torch.rsqrt(var + 1e-5), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(stats.view(2, rows, 2)[..., 1], -mean * torch.rsqrt(var + 1e-5), rtol=1e-4, atol=1e-5)
    # SwiGLU form: groups of 16 values followed by their 16 gates
    got = ops.linear(x, wq, sc, ops.LINEAR_SWIGLU, B=2, rows=rows, stats=stats)
    _ok()
    pairs = want.view(2, rows, N // 32, 2, 16)
    torch.testing.assert_close(got.float(), (F.silu(pairs[..., 1, :]) * pairs[..., 0, :]).reshape(2, rows, N // 2),
                               rtol=2e-2, atol=4e-2)


def test_dense_layer_kernel_head_major_form():
    g = torch.Generator().manual_seed(9)
    B, rows, K = 2, 70, 384
    x = torch.randn(B, rows, K, generator=g).bfloat16().to(DEV)
    w, b = (torch.randn(2048, K, generator=g) * 0.05).to(DEV), torch.randn(2048, generator=g).to(DEV)
    wq, sc = fold_linear(w, b, None, None)
    planes = ops.linear(x, wq, sc, ops.LINEAR_PLANES, B=B, rows=rows)
    _ok()
    want = F.linear(x.float(), wq.float(), b).view(B, rows, 4, 16, 32).permute(2, 0, 3, 1, 4)
    torch.testing.assert_close(planes[:3].float(), want[:3], **TOL)
    torch.testing.assert_close(planes[3].float(), torch.sigmoid(want[3]), **TOL)


@pytest.mark.parametrize("case", ["a", "b"])
def test_attention_with_pair_bias_matches_the_reference_module(case):
    g = load_golden("single_track")
    layer = _attention_layer(golden_single_attention_weights(g, case))
    s, z, mask = g[f"{case}_s"].bfloat16().to(DEV), g[f"{case}_z"].bfloat16().to(DEV), g[f"{case}_mask"].to(DEV)
    got = layer(s, z, mask)
    _ok()
    assert got.dtype == torch.bfloat16 and got.shape == s.shape
    torch.testing.assert_close(got.float().cpu(), g[f"{case}_update"], **TOL)
    torch.testing.assert_close(got.float().cpu(), g[f"{case}_update_bf16"], **TOL)
    # the residual form adds in the output-projection kernel; fp32 inputs are accepted and returned as fp32
    res = layer(s.float(), z, mask, residual=s.float())
    _ok()
    assert res.dtype == torch.float32
    torch.testing.assert_close(res.cpu(), g[f"{case}_update"] + g[f"{case}_s"], **TOL)


@pytest.mark.parametrize("B,N,valid", [(1, 300, (257,)), (2, 129, (129, 5)), (1, 520, (0,))])
def test_attention_with_pair_bias_matches_the_oracle_on_larger_inputs(B, N, valid):
    w = orc.make_pair_bias_attention_weights(700 + N).to(torch.bfloat16).to(torch.float32)
    layer = _attention_layer(w)
    g = torch.Generator().manual_seed(N)
    s = torch.randn(B, N, 384, generator=g).bfloat16()
    z = torch.randn(B, N, N, 128, generator=g).bfloat16()
    mask = torch.zeros(B, N)
    for b, n in enumerate(valid):
        mask[b, :n] = 1
    got = layer(s.to(DEV), z.to(DEV), mask.to(DEV))
    _ok()
    want = orc.pair_bias_attention_forward(s.float(), z.float(), mask, w)
    torch.testing.assert_close(got.float().cpu(), want, **TOL)
    # the same through the additive mask bias and through int32 key counts
    lengths = torch.tensor(valid, dtype=torch.int32, device=DEV)
    again = layer(s.to(DEV), z.to(DEV), None, mask_bias=lengths)
    additive = ((1 - mask) * -1e9)[:, None, None, :].to(DEV)
    third = layer(s.to(DEV), z.to(DEV), mask.to(DEV), mask_bias=additive)
    _ok()
    assert torch.equal(again, got) and torch.equal(third, got)


def test_single_transition_matches_the_reference_module():
    g = load_golden("single_track")
    layer = _transition_layer(golden_single_transition_weights(g))
    x = g["t_x"].bfloat16().to(DEV)
    got = layer(x)
    _ok()
    torch.testing.assert_close(got.float().cpu(), g["t_update"], rtol=2e-2, atol=4e-2)
    keep = x.clone()
    out = layer(x, residual=True, inplace=True)
    _ok()
    assert out.data_ptr() == x.data_ptr()
    torch.testing.assert_close(x.float().cpu(), g["t_update"] + keep.float().cpu(), rtol=2e-2, atol=4e-2)
    with pytest.raises(ValueError):
        layer(keep, torch.ones(1, 40, device=DEV))


def test_pairformer_layer_with_single_track_matches_the_oracle():
    """PairformerLayerV1.forward (pairformer.py:218-252): z through the pair track, then s + attention(s, z) and
    the single transition."""
    torch.manual_seed(0)
    N, valid = 72, 61
    stack = b200.PairformerModule(num_blocks=2, dtype=torch.bfloat16, trimul_high_precision=False,
                                  attention_initial_norm=True).to(DEV)
    ws = []
    for i, layer in enumerate(stack.layers):
        w_a = orc.make_pair_bias_attention_weights(40 + i).to(torch.bfloat16).to(torch.float32)
        w_t = orc.make_transition_weights(50 + i, c=384, hidden=1536, std=0.05, identity_ln=False).to(torch.bfloat16).to(torch.float32)
        w_m = [orc.make_trimul_weights(60 + 2 * i + k, identity_ln=False).to(torch.bfloat16).to(torch.float32) for k in range(2)]
        w_n = [orc.make_node_weights(70 + 2 * i + k, identity_ln=False).to(torch.bfloat16).to(torch.float32) for k in range(2)]
        w_z = orc.make_transition_weights(80 + i, identity_ln=False).to(torch.bfloat16).to(torch.float32)
        ws.append((w_a, w_t, w_m, w_n, w_z))
        layer.attention.load_state_dict(_attention_layer(w_a).state_dict())
        layer.transition_s.load_state_dict(_transition_layer(w_t).state_dict())
        for mod, w in zip((layer.tri_mul_out, layer.tri_mul_in), w_m):
            mod.load_state_dict({"norm_in.weight": w.ln_in_w, "norm_in.bias": w.ln_in_b, "p_in.weight": w.w_p_in,
                                 "g_in.weight": w.w_g_in, "norm_out.weight": w.ln_out_w, "norm_out.bias": w.ln_out_b,
                                 "p_out.weight": w.w_p_out, "g_out.weight": w.w_g_out})
        for mod, w in zip((layer.tri_attn_start, layer.tri_attn_end), w_n):
            mod.load_state_dict({"layer_norm.weight": w.ln_w, "layer_norm.bias": w.ln_b, "pair_bias_proj.weight": w.w_bias,
                                 "mha.in_proj.weight": w.w_in, "mha.o_proj.weight": w.w_out})
        layer.transition_z.load_state_dict({"norm.weight": w_z.ln_w, "norm.bias": w_z.ln_b,
                                            "fused_fc2_fc1.weight": w_z.w1, "fc3.weight": w_z.w2})
    s = torch.randn(1, N, 384).bfloat16()
    z = torch.randn(1, N, N, 128).bfloat16()
    m = torch.zeros(1, N)
    m[0, :valid] = 1
    pair_mask = m[:, :, None] * m[:, None, :]
    got_s, got_z = stack(s.to(DEV), z.to(DEV), m.to(DEV), pair_mask.to(DEV))
    _ok()
    want_s, want_z = s.float(), z.float()
    for w_a, w_t, w_m, w_n, w_z in ws:
        want_z = orc.trimul_forward(want_z, pair_mask, w_m[0], orc.OUTGOING, residual=True)
        want_z = orc.trimul_forward(want_z, pair_mask, w_m[1], orc.INCOMING, residual=True)
        want_z = orc.node_forward(want_z, pair_mask, w_n[0], orc.STARTING, residual=True)
        want_z = orc.node_forward(want_z, pair_mask, w_n[1], orc.ENDING, residual=True)
        want_z = orc.transition_forward(want_z, None, w_z, residual=True)
        want_s = want_s + orc.pair_bias_attention_forward(want_s, want_z, m, w_a)
        want_s = orc.transition_forward(want_s, None, w_t, residual=True)
    assert got_s.dtype == torch.bfloat16 and torch.isfinite(got_s).all() and torch.isfinite(got_z).all()
    # valid tokens only: padded positions of z differ between the masked and the plain residual form of the
    # triangle multiplication, and padded queries of s read them through the pair bias
    torch.testing.assert_close(got_z.float().cpu()[:, :valid, :valid], want_z[:, :valid, :valid], rtol=3e-2, atol=6e-2)
    torch.testing.assert_close(got_s.float().cpu()[:, :valid], want_s[:, :valid], rtol=3e-2, atol=6e-2)


def test_pairformer_module_graph_replay_matches_eager():
    torch.manual_seed(5)
    N = 64
    kw = dict(num_blocks=2, dtype=torch.bfloat16, trimul_high_precision=False, attention_initial_norm=True)
    eager = b200.PairformerModule(**kw).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(11)
    for name, prm in eager.named_parameters():
        if prm.dim() == 2:
            prm.data.copy_(torch.randn(prm.shape, generator=gen, device=DEV) * 0.03)
        else:
            prm.data.fill_(0.0 if name.endswith("bias") else 1.0)
    graphed = b200.PairformerModule(use_cuda_graph=True, **kw).to(DEV)
    graphed.load_state_dict(eager.state_dict(), strict=True)
    m = (torch.arange(N, device=DEV) < 57).float()[None]
    pair_mask = m[:, :, None] * m[:, None, :]
    outs = []
    for seed in (1, 2):
        g = torch.Generator(device=DEV).manual_seed(seed)
        s = torch.randn(1, N, 384, generator=g, device=DEV).bfloat16()
        z = torch.randn(1, N, N, 128, generator=g, device=DEV).bfloat16()
        want_s, want_z = eager(s.clone(), z.clone(), m, pair_mask)
        got_s, got_z = graphed(s, z, m, pair_mask)  # first call records, second replays
        _ok()
        assert torch.equal(got_s, want_s) and torch.equal(got_z, want_z)
        outs.append(got_s)
    assert not torch.equal(outs[0], outs[1])


def test_v2_layer_equals_v1_with_the_pre_norm_as_initial_norm_and_applies_the_post_norm():
    torch.manual_seed(8)
    N = 48
    kw = dict(num_blocks=1, dtype=torch.bfloat16, trimul_high_precision=False)
    v1 = b200.PairformerModule(attention_initial_norm=True, **kw).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(12)
    for name, prm in v1.named_parameters():
        if prm.dim() == 2:
            prm.data.copy_(torch.randn(prm.shape, generator=gen, device=DEV) * 0.03)
        else:
            prm.data.copy_((0.0 if name.endswith("bias") else 1.0) + 0.1 * torch.randn(prm.shape, generator=gen, device=DEV))
    sd = {k.replace("attention.norm_s", "pre_norm_s"): v for k, v in v1.state_dict().items()}
    v2 = b200.PairformerModule(version="v2", **kw).to(DEV)
    v2.load_state_dict(sd, strict=True)
    m = (torch.arange(N, device=DEV) < 41).float()[None]
    pair_mask = m[:, :, None] * m[:, None, :]
    s = torch.randn(1, N, 384, device=DEV).bfloat16()
    z = torch.randn(1, N, N, 128, device=DEV).bfloat16()
    s1, z1 = v1(s.clone(), z.clone(), m, pair_mask)
    s2, z2 = v2(s.clone(), z.clone(), m, pair_mask)
    _ok()
    assert torch.equal(z1, z2) and torch.equal(s1, s2)
    # an attention with its own initial norm keeps the pre-norm as a separate step; with unit pre-norm weights the
    # result is attention(LN(LN(s))) and stays finite; the post norm normalises the rows of the result
    post = b200.PairformerModule(version="v2", post_layer_norm=True, **kw).to(DEV)
    sd_post = dict(sd)
    sd_post.update({"layers.0.post_norm_s.weight": torch.ones(384), "layers.0.post_norm_s.bias": torch.zeros(384)})
    post.load_state_dict(sd_post, strict=True)
    s3, _ = post(s.clone(), z.clone(), m, pair_mask)
    _ok()
    torch.testing.assert_close(s3.float(), F.layer_norm(s2.float(), (384,)), rtol=2e-2, atol=2e-2)


def test_single_track_entry_points_refuse_bad_arguments():
    x = torch.zeros(1, 8, 384, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(384, 384, dtype=torch.bfloat16, device=DEV)
    sc = torch.zeros(384, 2, device=DEV)
    with pytest.raises(ValueError):  # K must be a multiple of 128
        ops.linear(torch.zeros(1, 8, 200, dtype=torch.bfloat16, device=DEV), torch.zeros(384, 200, dtype=torch.bfloat16, device=DEV),
                   sc, ops.LINEAR_ROWS, B=1, rows=8)
    with pytest.raises(ValueError):  # the head-major form needs the 2048 columns of 4 planes x 16 heads x 32
        ops.linear(x, w, sc, ops.LINEAR_PLANES, B=1, rows=8)
    with pytest.raises(ValueError):  # a residual only with the row form
        _lib.call("b200ta_linear", x.data_ptr(), 8 * 384, 384, 128, w.data_ptr(), sc.data_ptr(), None, x.data_ptr(), 384,
                  x.data_ptr(), 192, 0, ops.LINEAR_SWIGLU, 1, 8, 384, 384, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(ValueError):
        ops.linear(x, w, sc, 7, B=1, rows=8)
    with pytest.raises(ValueError):  # row statistics hold a row in registers: K <= 2048
        ops.row_stats(torch.zeros(4, 4096, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):  # an odd head count
        ops.pack_pair_bias_weights(None, None, torch.zeros(3, 128, device=DEV), 1.0)
    z = torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16, device=DEV)
    packed = ops.pack_pair_bias_weights(None, None, torch.zeros(16, 128, device=DEV), 1.0)
    with pytest.raises(ValueError):  # the bias buffer must carry the padded key axis
        ops.pair_bias(z, packed, 16, bias=torch.zeros(1, 16, 8, 9, dtype=torch.bfloat16, device=DEV))
    # without a LayerNorm in the pack the projection runs on z as it is
    w_z = torch.randn(16, 128, device=DEV) * 0.05
    zr = torch.randn(1, 8, 8, 128, device=DEV).bfloat16()
    got = ops.pair_bias(zr, ops.pack_pair_bias_weights(None, None, w_z, 2.0), 16)
    _ok()
    torch.testing.assert_close(got.float(), 2.0 * F.linear(zr.float(), w_z).movedim(-1, 1), **TOL)
