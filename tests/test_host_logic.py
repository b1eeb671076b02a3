"""Host-side logic that needs no GPU: chunking knobs, mask forms, weight loading, state_dict contract."""

import pytest
import torch

import bionemo_inference_runtime_b200 as b200
from bionemo_inference_runtime_b200.layers import auto_chunk


def test_chunk_policy_thresholds_and_registry():
    p = b200.ChunkPolicy(chunk_size=8, min_size=16, dim=1, min_rank=4)
    assert not p.should_chunk(torch.zeros(1, 16, 16, 4))
    assert p.should_chunk(torch.zeros(1, 17, 17, 4))
    assert not p.should_chunk(torch.zeros(17, 17, 4))  # rank below min_rank
    assert not p.replace(enabled=False).should_chunk(torch.zeros(1, 17, 17, 4))
    assert b200.CHUNK_REGISTRY.get(b200.TRIANGLE_ATTENTION).chunk_size == 512
    assert b200.CHUNK_REGISTRY.get(b200.PAIR_TRANSITION).dim == 1
    assert auto_chunk.default_autochunk_min() >= 512
    assert list(b200.iter_chunks(10, 4)) == [(0, 4), (4, 4), (8, 2)]


def test_chunk_apply_matches_dense_call():
    x = torch.randn(2, 20, 5, 3)
    m = torch.randn(2, 20, 5)
    policy = b200.ChunkPolicy(chunk_size=7, min_size=4, dim=1)
    fn = lambda a, b, scale: a * b.unsqueeze(-1) * scale  # noqa: E731
    assert torch.equal(b200.chunk_apply(fn, x, m, policy=policy, scale=2.0), fn(x, m, 2.0))


def test_mask_forms_reduce_to_the_same_lengths():
    m = torch.zeros(2, 6)
    m[0, :4] = 1
    m[1, :6] = 1
    pair = m[:, :, None] * m[:, None, :]
    add = b200.precompute_pair_masks("VANILLA", pair, inf=1e9, dtype=torch.float32)
    cnt = b200.precompute_pair_masks("Heuristic", pair)
    assert add.mask_bias.shape == (2, 6, 1, 1, 6) and cnt.mask_bias.dtype == torch.int32
    assert torch.equal(b200.mask_to_lengths(add.mask_bias, 2, 6), cnt.mask_bias)
    assert torch.equal(b200.mask_to_lengths(add.mask_bias_transposed, 2, 6), cnt.mask_bias_transposed)
    assert torch.equal(b200.mask_to_lengths(cnt.mask_bias.reshape(-1), 2, 6), cnt.mask_bias)
    per_item = torch.tensor([4, 6], dtype=torch.int32)
    assert b200.mask_to_lengths(per_item, 2, 6).tolist() == [[4] * 6, [6] * 6]
    with pytest.raises(ValueError):
        b200.mask_to_lengths(torch.zeros(5, dtype=torch.int32), 2, 6)
    with pytest.raises(ValueError):
        b200.precompute_pair_masks("nope", pair)


def test_every_reference_backend_name_is_accepted():
    for name in ("VANILLA", "SDPA", "CUEQUIV", "CuTeDSL", "ClaudeKit", "Heuristic"):
        assert b200.get_attention_backend(name) is b200.B200TriangleAttention
    with pytest.raises(ValueError):
        b200.get_attention_backend("FLASH")
    with pytest.raises(ValueError):
        b200.create_attention("VANILLA", 0, 8, 32)  # unsupported head count


def test_state_dict_contract_of_the_node():
    flags = {"q": False, "k": False, "v": False, "g": True, "o": True}
    node = b200.TriangleAttentionEndingNode(128, 32, 4, dtype=torch.bfloat16, mha_bias_flags=flags)
    sd = node.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        "layer_norm.weight": (128,), "layer_norm.bias": (128,), "pair_bias_proj.weight": (4, 128),
        "mha.in_proj.weight": (512, 128), "mha.in_proj.bias": (512,), "mha.o_proj.weight": (128, 128),
        "mha.o_proj.bias": (128,)}
    assert node.node_type == b200.TriangleAttentionNodeType.ENDING
    assert all(not p.requires_grad for n, p in node.named_parameters() if "layer_norm" not in n)
    plain = b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.bfloat16)
    assert sorted(plain.state_dict()) == ["layer_norm.bias", "layer_norm.weight", "mha.in_proj.weight",
                                          "mha.o_proj.weight", "pair_bias_proj.weight"]
    node.load_state_dict(sd, strict=True)


def test_state_dict_contract_of_the_transition():
    t = b200.Transition(128, 512, dtype=torch.bfloat16)
    assert {k: tuple(v.shape) for k, v in t.state_dict().items()} == {
        "norm.weight": (128,), "norm.bias": (128,), "fused_fc2_fc1.weight": (1024, 128), "fc3.weight": (128, 512)}
    assert sorted(b200.Transition(128, 512, dtype=torch.bfloat16, normalize=False).state_dict()) == [
        "fc3.weight", "fused_fc2_fc1.weight"]
    with pytest.raises(ValueError):
        b200.Transition(200, 800)  # widths must be multiples of 128
    single = b200.Transition(384, 1536, dtype=torch.bfloat16)  # the single-track transition
    assert {k: tuple(v.shape) for k, v in single.state_dict().items()} == {
        "norm.weight": (384,), "norm.bias": (384,), "fused_fc2_fc1.weight": (3072, 384), "fc3.weight": (384, 1536)}


def test_linear_fused_segment_loading():
    lin = b200.Linear(8, 10, bias=True, dtype=torch.float32, weights_loading_config=b200.WeightsLoadingConfig(
        weight_mode=b200.WeightMode.FUSED_SEGMENTS_LINEAR, segment_sizes=(4, 4, 2)))
    segs = [{"weight": torch.ones(4, 8)}, {"weight": 2 * torch.ones(3, 8), "bias": torch.ones(3)},
            {"weight": 3 * torch.ones(2, 8)}]
    lin.load_weights(segs)
    w = lin.weight.cpu()
    assert torch.equal(w[:4], torch.ones(4, 8)) and torch.equal(w[4:7], 2 * torch.ones(3, 8))
    assert torch.equal(w[7], torch.zeros(8)) and torch.equal(w[8:], 3 * torch.ones(2, 8))
    assert lin.bias.cpu().tolist() == [0, 0, 0, 0, 1, 1, 1, 0, 0, 0]


def test_split_pair_bias_proj_moves_the_fifth_segment():
    weights = {"blocks.0.tri_attn_start.mha.in_proj": [{"weight": torch.zeros(128, 128)} for _ in range(4)]
               + [{"weight": torch.ones(4, 128)}]}
    out = b200.split_pair_bias_proj(weights)
    assert len(out["blocks.0.tri_attn_start.mha.in_proj"]) == 4
    assert torch.equal(out["blocks.0.tri_attn_start.pair_bias_proj"][0]["weight"], torch.ones(4, 128))


def test_layers_refuse_cpu_tensors_and_other_dtypes():
    node = b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        node(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="bfloat16"):
        b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.float32)(torch.zeros(1, 8, 8, 128))
    general = b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.bfloat16, pair_mask_left_aligned=False)
    assert general.pair_mask_left_aligned is False  # keys masked by bits instead of row lengths
    with pytest.raises(ValueError, match="CUDA"):
        b200.Transition(128, 512, dtype=torch.bfloat16)(torch.zeros(4, 128, dtype=torch.bfloat16))


def test_ensure_buffer_reuses_and_reallocates():
    bufs: dict = {}
    a = b200.ensure_buffer(bufs, "k", (2, 3), torch.float32, torch.device("cpu"))
    assert b200.ensure_buffer(bufs, "k", (2, 3), torch.float32, torch.device("cpu")) is a
    assert b200.ensure_buffer(bufs, "k", (2, 4), torch.float32, torch.device("cpu")) is not a
    assert b200.ensure_buffer(None, "k", (2, 3), torch.float32, torch.device("cpu")) is None


def test_triangle_multiplication_state_dict_keys_dtypes_and_errors():
    """Keys and shapes of the reference module (bionemo_ir/_torch/layers/triangle_nodes.py:378-417)."""
    node = b200.TriangleMultiplicationNode(dtype=torch.bfloat16, high_precision=False)
    shapes = {k: tuple(v.shape) for k, v in node.state_dict().items()}
    assert shapes == {"norm_in.weight": (128,), "norm_in.bias": (128,), "p_in.weight": (256, 128),
                      "g_in.weight": (256, 128), "norm_out.weight": (128,), "norm_out.bias": (128,),
                      "p_out.weight": (128, 128), "g_out.weight": (128, 128)}
    assert all(not p.requires_grad for n, p in node.named_parameters() if "norm" not in n)
    hp = b200.TriangleMultiplicationNode(dtype=torch.bfloat16, bias_flags={"p_in": True, "g_in": True, "p_out": True,
                                                                        "g_out": True}, norm_bias=False)
    sd = hp.state_dict()
    assert "norm_in.bias" not in sd and sd["p_in.bias"].shape == (256,) and sd["g_out.bias"].dtype == torch.float32
    assert sd["norm_out.weight"].dtype == torch.float32 and sd["norm_in.weight"].dtype == torch.bfloat16
    assert int(b200.TriangleMultiplicationNodeType.OUTGOING) == 0 and int(b200.TriangleMultiplicationNodeType.INCOMING) == 1
    with pytest.raises(ValueError):
        b200.TriangleMultiplicationNode(dim=64)
    with pytest.raises(ValueError):
        node(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16), None)  # no CPU path
    meta = b200.precompute_trimul_metadata(torch.zeros(1, 9, 9, 128), torch.ones(1, 9, dtype=torch.int32), None)
    assert meta.token_pad_multiple == -1 and meta.outgoing_actual_seqlen is not None
    assert b200.precompute_trimul_metadata(torch.zeros(1, 9, 9, 128), torch.ones(1, 9), None,
                                           enabled=False).outgoing_actual_seqlen is None
    b200.set_trimul_token_padding(torch.nn.Sequential(node), True)
    assert node.pad_tokens is True


def test_boltz_checkpoint_converters_feed_strict_loads():
    """Key mappings of bionemo_ir/models/convert_utils.py:29-98 into this package's layers."""
    from bionemo_inference_runtime_b200 import convert_utils as cu

    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    ckpt = {}
    p = "layers.0.tri_att_start"
    for k, shape in {"layer_norm.weight": (128,), "layer_norm.bias": (128,), "linear.weight": (4, 128),
                     "mha.linear_q.weight": (128, 128), "mha.linear_k.weight": (128, 128),
                     "mha.linear_v.weight": (128, 128), "mha.linear_g.weight": (128, 128),
                     "mha.linear_o.weight": (128, 128)}.items():
        ckpt[f"{p}.{k}"] = r(*shape)
    sd = cu.get_tri_attn_node_weights(ckpt, p, "blk.tri_attn_start", dtype="bfloat16")
    node = b200.TriangleAttentionStartingNode(128, 32, 4, dtype=torch.bfloat16)
    node.load_state_dict({k.removeprefix("blk.tri_attn_start."): v for k, v in sd.items()}, strict=True)
    w = node.mha.in_proj.weight.float()
    assert torch.equal(w[128:256], ckpt[f"{p}.mha.linear_k.weight"].bfloat16().float())
    assert torch.equal(w[384:], ckpt[f"{p}.mha.linear_g.weight"].bfloat16().float())
    assert torch.equal(node.pair_bias_proj.weight.float(), ckpt[f"{p}.linear.weight"].bfloat16().float())

    p = "layers.0.tri_mul_out"
    for k, shape in {"norm_in.weight": (128,), "norm_in.bias": (128,), "p_in.weight": (256, 128), "g_in.weight": (256, 128),
                     "norm_out.weight": (128,), "norm_out.bias": (128,), "p_out.weight": (128, 128),
                     "g_out.weight": (128, 128)}.items():
        ckpt[f"{p}.{k}"] = r(*shape)
    sd = cu.get_tri_mul_node_weights(ckpt, p, "m", dtype="bfloat16")
    assert sd["m.p_in.weight"].dtype == torch.bfloat16 and sd["m.p_out.weight"].dtype == torch.float32
    tm = b200.TriangleMultiplicationNode(dtype=torch.bfloat16, high_precision=True)
    tm.load_state_dict({k.removeprefix("m."): v for k, v in sd.items()}, strict=True)
    assert torch.equal(tm.g_out.weight, ckpt[f"{p}.g_out.weight"])

    p = "layers.0.transition_z"
    for k, shape in {"norm.weight": (128,), "norm.bias": (128,), "fc1.weight": (512, 128), "fc2.weight": (512, 128),
                     "fc3.weight": (128, 512)}.items():
        ckpt[f"{p}.{k}"] = r(*shape)
    sd = cu.get_transition_weights(ckpt, p, "t", dtype="bfloat16")
    tr = b200.Transition(128, 512, dtype=torch.bfloat16)
    tr.load_state_dict({k.removeprefix("t."): v for k, v in sd.items()}, strict=True)
    assert torch.equal(tr.fused_fc2_fc1.weight[:512].float(), ckpt[f"{p}.fc2.weight"].bfloat16().float())  # value rows first
    assert torch.equal(tr.fused_fc2_fc1.weight[512:].float(), ckpt[f"{p}.fc1.weight"].bfloat16().float())  # then gate rows
    with pytest.raises(ValueError):
        cu.get_transition_weights(ckpt, p, "t", dtype="int7")


def test_pair_track_stack_has_the_reference_submodule_names():
    """PairformerNoSeqModule / PairformerNoSeqLayer (bionemo_ir/_torch/layers/transformers/pairformer.py:255-363)."""
    stack = b200.PairformerNoSeqModule(num_blocks=2, dtype=torch.bfloat16, trimul_high_precision=False, token_s=384,
                                       num_heads=16)  # single-track arguments are accepted and unused
    keys = set(stack.state_dict())
    for i in range(2):
        for sub in ("tri_mul_out.p_in.weight", "tri_mul_in.g_out.weight", "tri_attn_start.mha.in_proj.weight",
                    "tri_attn_end.pair_bias_proj.weight", "transition_z.fused_fc2_fc1.weight", "transition_z.fc3.weight"):
            assert f"layers.{i}.{sub}" in keys
    layer = stack.layers[1]
    assert layer.tri_mul_in.multiplication_type == b200.TriangleMultiplicationNodeType.INCOMING
    assert layer.tri_attn_end.node_type == b200.TriangleAttentionNodeType.ENDING
    assert layer.no_update_s and not layer.no_update_z
    assert b200.PairformerNoSeqModule(num_blocks=0)(torch.zeros(1, 4, 4, 128), torch.ones(1, 4, 4)).shape == (1, 4, 4, 128)


def test_single_track_attention_state_dict_and_refusals():
    """AttentionPairBias as the pairformer builds it (bionemo_ir/_torch/layers/attention.py:445-626): the reference
    module's parameter names, and a ValueError for the options of other models."""
    layer = b200.AttentionPairBias(layer_idx=0, c_s=384, c_z=128, num_heads=16, dtype=torch.bfloat16, bias_proj=True,
                                   initial_norm=True)
    assert {k: tuple(v.shape) for k, v in layer.state_dict().items()} == {
        "norm_s.weight": (384,), "norm_s.bias": (384,), "in_proj.weight": (1536, 384), "in_proj.bias": (1536,),
        "proj_z.0.weight": (128,), "proj_z.0.bias": (128,), "proj_z.1.weight": (16, 128), "proj_o.weight": (384, 384)}
    plain = b200.AttentionPairBias(0, 384, 128, 16, initial_norm=False, bias_proj=True, out_bias=True, pair_norm=False)
    assert sorted(plain.state_dict()) == ["in_proj.bias", "in_proj.weight", "proj_o.bias", "proj_o.weight",
                                          "proj_z.0.weight"]
    for bad in (dict(bias_proj=False), dict(bias_proj=True, use_separate_layer_norm=True),
                dict(bias_proj=True, use_qk_norm=True), dict(bias_proj=True, output_gate_dim=384),
                dict(bias_proj=True, norm_type="rms_norm"), dict(bias_proj=True, mask_left_aligned=False),
                dict(bias_proj=True, dtype=torch.float16)):
        with pytest.raises(ValueError):
            b200.AttentionPairBias(0, 384, 128, 16, **bad)
    with pytest.raises(ValueError):
        b200.AttentionPairBias(0, 384, 128, 8, bias_proj=True)  # 16 heads only
    with pytest.raises(ValueError, match="CUDA"):
        layer(torch.zeros(1, 8, 384), torch.zeros(1, 8, 8, 128), torch.ones(1, 8))
    with pytest.raises(ValueError):
        layer(torch.zeros(1, 8, 384), torch.zeros(1, 8, 8, 128), torch.ones(1, 8), single_embedding=torch.zeros(1, 8, 384))


def test_layer_norm_fold_for_the_tensor_core_gemm():
    """fold_linear: LN(x) . W^T + b == rstd * (x . w_bf16^T) + nmr * rowsum + const, up to the bf16 rounding of W."""
    from bionemo_inference_runtime_b200.layers.attention_pair_bias import fold_linear

    g = torch.Generator().manual_seed(3)
    x = torch.randn(37, 384, generator=g) * 2 + 0.7
    w, b = torch.randn(96, 384, generator=g) * 0.05, torch.randn(96, generator=g)
    gamma, beta = 1 + 0.2 * torch.randn(384, generator=g), 0.2 * torch.randn(384, generator=g)
    wq, sc = fold_linear(w, b, gamma, beta)
    assert wq.dtype == torch.bfloat16 and tuple(sc.shape) == (96, 2)
    mean, var = x.mean(-1, keepdim=True), x.var(-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + 1e-5)
    got = rstd * (x @ wq.float().T) + (-mean * rstd) * sc[:, 0] + sc[:, 1]
    want = torch.nn.functional.linear(torch.nn.functional.layer_norm(x, (384,), gamma, beta), w, b)
    torch.testing.assert_close(got, want, rtol=0, atol=2e-2)
    wq2, sc2 = fold_linear(w, None, None, None)
    assert torch.equal(wq2, w.bfloat16()) and not sc2.any()


def test_pairformer_with_single_track_has_the_reference_submodule_names():
    """PairformerLayerV1 / PairformerModule (bionemo_ir/_torch/layers/transformers/pairformer.py:44-252, 418-510)."""
    class Config:
        version, num_blocks, token_s, token_z, num_heads = "v1", 2, 384, 128, 16
        torch_dtype, trimul_high_precision, attention_initial_norm, no_update_s = torch.bfloat16, False, True, False

    stack = b200.PairformerModule(Config())
    keys = set(stack.state_dict())
    for sub in ("attention.norm_s.weight", "attention.in_proj.bias", "attention.proj_z.1.weight",
                "attention.proj_o.weight", "transition_s.fused_fc2_fc1.weight", "transition_s.fc3.weight",
                "tri_mul_out.p_in.weight", "tri_attn_end.pair_bias_proj.weight", "transition_z.fc3.weight"):
        assert f"layers.1.{sub}" in keys
    assert tuple(stack.layers[0].transition_s.fc3.weight.shape) == (384, 1536)
    no_seq = b200.PairformerModule(num_blocks=1, no_update_s=True, dtype=torch.bfloat16)
    assert not any(k.startswith("layers.0.attention") or "transition_s" in k for k in no_seq.state_dict())
    with pytest.raises(ValueError):
        b200.PairformerModule(num_blocks=1, no_update_z=True)


def test_boltz_single_track_attention_converter_feeds_a_strict_load():
    """Boltz checkpoint names (proj_q with bias, proj_g / proj_k / proj_v without) -> in_proj in q, gate, k, v order
    (bionemo_ir/models/boltz1/convert.py:64-98)."""
    from bionemo_inference_runtime_b200.convert_utils import get_attention_pair_bias_weights

    g = torch.Generator().manual_seed(4)
    ckpt = {f"m.attention.proj_{n}.weight": torch.randn(384, 384, generator=g) for n in "qkvg"}
    ckpt.update({"m.attention.proj_q.bias": torch.randn(384, generator=g), "m.attention.norm_s.weight": torch.ones(384),
                 "m.attention.norm_s.bias": torch.zeros(384), "m.attention.proj_z.0.weight": torch.ones(128),
                 "m.attention.proj_z.0.bias": torch.zeros(128), "m.attention.proj_z.1.weight": torch.randn(16, 128, generator=g),
                 "m.attention.proj_o.weight": torch.randn(384, 384, generator=g)})
    sd = get_attention_pair_bias_weights(ckpt, "m.attention", "attention", dtype="bfloat16")
    layer = b200.AttentionPairBias(0, 384, 128, 16, dtype=torch.bfloat16, bias_proj=True, initial_norm=True)
    layer.load_state_dict({k.removeprefix("attention."): v for k, v in sd.items()}, strict=True)
    w = layer.in_proj.weight
    assert torch.equal(w[384:768].cpu(), ckpt["m.attention.proj_g.weight"].bfloat16())
    assert torch.equal(w[768:1152].cpu(), ckpt["m.attention.proj_k.weight"].bfloat16())
    assert torch.equal(layer.in_proj.bias[:384].cpu(), ckpt["m.attention.proj_q.bias"].bfloat16())
    assert not layer.in_proj.bias[384:].any()


def test_single_mask_precompute_registry_and_key_counts():
    """precompute_single_masks (bionemo_ir/_torch/attention_backend/utils.py:441-518): additive bias for the eager
    backends, int32 key counts for the left-mask kernel; the attention layer reads the same count from each."""
    mask = torch.tensor([[1., 1., 1., 0., 0.], [1., 1., 1., 1., 1.]])
    add = b200.precompute_single_masks("VANILLA", mask, inf=1e9)
    assert tuple(add.mask_bias.shape) == (2, 1, 1, 5) and add.mask_bias[0, 0, 0, 3] == -1e9 and add.mask_bias[1].abs().sum() == 0
    cnt = b200.precompute_single_masks("CuTeDSL", mask, activation_dtype=torch.bfloat16)
    assert cnt.mask_bias.dtype == torch.int32 and cnt.mask_bias.tolist() == [3, 5]
    assert cnt.excluded.shape == (2, 5, 1) and cnt.value_mask.dtype == torch.bfloat16
    with pytest.raises(ValueError):
        b200.precompute_single_masks("no-such-backend", mask)
    with pytest.raises(ValueError):
        b200.precompute_single_masks("VANILLA", mask, query_to_keys=lambda t: t)
    layer = b200.AttentionPairBias(0, 384, 128, 16, bias_proj=True)
    dev = torch.device("cpu")
    for form in (dict(mask=mask, mask_bias=None), dict(mask=mask, mask_bias=add.mask_bias),
                 dict(mask=None, mask_bias=cnt.mask_bias)):
        assert layer._lengths(form["mask"], form["mask_bias"], 2, 5, dev).tolist() == [3, 5]
    assert layer._lengths(None, None, 2, 5, dev).tolist() == [5, 5]


def test_v2_pairformer_layer_names_and_pre_norm_fold():
    """PairformerLayerV2 (bionemo_ir/_torch/layers/transformers/pairformer.py:356-416): pre_norm_s / post_norm_s."""
    stack = b200.PairformerModule(num_blocks=1, version="v2", dtype=torch.bfloat16, post_layer_norm=True)
    keys = set(stack.state_dict())
    assert {"layers.0.pre_norm_s.weight", "layers.0.pre_norm_s.bias", "layers.0.post_norm_s.weight",
            "layers.0.post_norm_s.bias"} <= keys
    layer = stack.layers[0]
    assert isinstance(layer, b200.PairformerLayerV2) and layer.attention.norm_s is None
    assert layer.attention._norm_of_s() is layer.pre_norm_s          # folded into the in-projection
    assert not any("_input_norm" in k for k in keys)                 # and not registered twice
    own_norm = b200.PairformerModule(num_blocks=1, version="v2", attention_initial_norm=True).layers[0]
    assert own_norm.attention._norm_of_s() is own_norm.attention.norm_s and not own_norm._pre_norm_folded
    assert isinstance(b200.PairformerModule(num_blocks=1, post_layer_norm=True).layers[0], b200.PairformerLayerV1)
    with pytest.raises(ValueError):
        b200.PairformerModule(num_blocks=1, version="v3")
    with pytest.raises(ValueError):
        b200.PairformerLayerV2(no_update_s=True)


def test_numa_binding_is_a_no_op_without_a_readable_topology():
    before = sorted(__import__("os").sched_getaffinity(0))
    cores = b200.bind_to_gpu_numa_node(0)  # no GPU here, or a container without NUMA nodes: nothing may change
    if cores is None:
        assert sorted(__import__("os").sched_getaffinity(0)) == before
    else:
        assert set(cores) <= set(before) and sorted(__import__("os").sched_getaffinity(0)) == cores
        __import__("os").sched_setaffinity(0, before)


def test_weight_packing_refuses_host_tensors():
    """A host address must never reach a kernel: packing checks the device before anything is launched."""
    from bionemo_inference_runtime_b200 import ops

    with pytest.raises(ValueError, match="CUDA device"):
        ops.pack_transition_weights(torch.ones(128), torch.zeros(128), torch.zeros(1024, 128), torch.zeros(128, 512))
    with pytest.raises(ValueError, match="CUDA device"):
        ops.pack_relu_transition_weights(torch.ones(128), torch.zeros(128), torch.zeros(512, 128), torch.zeros(512),
                                         torch.zeros(128, 512), torch.zeros(128))


def test_pair_transition_state_dict_contract():
    t = b200.PairTransition(128, 4, dtype=torch.bfloat16)
    assert {k: tuple(v.shape) for k, v in t.state_dict().items()} == {
        "layer_norm.weight": (128,), "layer_norm.bias": (128,), "linear_1.weight": (512, 128), "linear_1.bias": (512,),
        "linear_2.weight": (128, 512), "linear_2.bias": (128,)}
    with pytest.raises(ValueError):
        b200.PairTransition(64, 4, dtype=torch.bfloat16)
