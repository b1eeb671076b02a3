"""CPU oracle for the triangle-attention node and the pair transition.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
module: it exists so the tests, the smoke check and the CPU-baseline leg of the
benchmark can compare the CUDA path against a slow, plain restatement of the
reference algorithm.  It runs on the CPU with ordinary PyTorch tensor ops (this
path is floating point; there is no integer/byte arithmetic to restate in C) in
whatever dtype it is given, in the same order of operations as the reference's
eager path, so a bf16 run reproduces the eager path's rounding points.

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference's own modules
(``TriangleAttentionStartingNode``/``EndingNode`` with the VANILLA backend and
``transition_mlp_w_norm_reference``) run on seeded inputs by
``tests/golden/make_golden.py``; ``tests/test_oracle.py`` checks this file
against them.

Each function names the reference lines it restates (paths relative to the
reference project root).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

STARTING = 0
ENDING = 1


@dataclass
class NodeWeights:
    """Parameters of one triangle-attention node, named as in the reference state_dict."""

    ln_w: torch.Tensor  # layer_norm.weight [c]
    ln_b: torch.Tensor  # layer_norm.bias [c]
    w_bias: torch.Tensor  # pair_bias_proj.weight [H, c]
    w_in: torch.Tensor  # mha.in_proj.weight [4*H*d, c] rows q,k,v,g
    b_in: torch.Tensor | None  # mha.in_proj.bias [4*H*d] or None
    w_out: torch.Tensor  # mha.o_proj.weight [c, H*d]
    b_out: torch.Tensor | None  # mha.o_proj.bias [c] or None

    def to(self, dtype: torch.dtype) -> "NodeWeights":
        return NodeWeights(*[None if t is None else t.to(dtype) for t in
                             (self.ln_w, self.ln_b, self.w_bias, self.w_in, self.b_in, self.w_out, self.b_out)])


@dataclass
class TransitionWeights:
    ln_w: torch.Tensor  # norm.weight [c]
    ln_b: torch.Tensor  # norm.bias [c]
    w1: torch.Tensor  # fused_fc2_fc1.weight [2*hidden, c]: value rows, then gate rows
    w2: torch.Tensor  # fc3.weight [c, hidden]

    def to(self, dtype: torch.dtype) -> "TransitionWeights":
        return TransitionWeights(*[t.to(dtype) for t in (self.ln_w, self.ln_b, self.w1, self.w2)])


def make_node_weights(seed: int, c: int = 128, heads: int = 4, d: int = 32, std: float = 0.02,
                      gate_bias: float | None = None, identity_ln: bool = True,
                      out_bias: bool = False) -> NodeWeights:
    """Seeded weights in the recipe of the reference's test helper ``init_module_weights``
    (tests/_torch/__init__.py:33-63): matrices ~N(0, std²), 1-D weights 1, biases 0."""
    g = torch.Generator().manual_seed(seed)
    w_bias = torch.randn(heads, c, generator=g) * std
    w_in = torch.randn(4 * heads * d, c, generator=g) * std
    w_out = torch.randn(c, heads * d, generator=g) * std
    if identity_ln:
        ln_w, ln_b = torch.ones(c), torch.zeros(c)
    else:
        ln_w = 1 + 0.2 * torch.randn(c, generator=g)
        ln_b = 0.2 * torch.randn(c, generator=g)
    b_in = None
    if gate_bias is not None:
        b_in = torch.zeros(4 * heads * d)
        b_in[3 * heads * d:] = gate_bias
    b_out = 0.1 * torch.randn(c, generator=g) if out_bias else None
    return NodeWeights(ln_w, ln_b, w_bias, w_in, b_in, w_out, b_out)


def make_transition_weights(seed: int, c: int = 128, hidden: int = 512, std: float = 0.02,
                            identity_ln: bool = True) -> TransitionWeights:
    g = torch.Generator().manual_seed(seed)
    w1 = torch.randn(2 * hidden, c, generator=g) * std
    w2 = torch.randn(c, hidden, generator=g) * std
    if identity_ln:
        ln_w, ln_b = torch.ones(c), torch.zeros(c)
    else:
        ln_w = 1 + 0.2 * torch.randn(c, generator=g)
        ln_b = 0.2 * torch.randn(c, generator=g)
    return TransitionWeights(ln_w, ln_b, w1, w2)


def additive_mask_bias(mask: torch.Tensor, inf: float, dtype: torch.dtype) -> torch.Tensor:
    """``inf * (mask - 1)`` shaped [B, R, 1, 1, S].
    Reference: _default_precompute_pair_masks, bionemo_ir/_torch/attention_backend/utils.py:305-317."""
    m = mask.to(dtype)
    return (inf * (m - 1))[..., :, None, None, :]


def row_lengths(mask: torch.Tensor) -> torch.Tensor:
    """int32 count of valid keys per row.
    Reference: _cutedsl_precompute_pair_masks, bionemo_ir/_torch/attention_backend/utils.py:339-386."""
    return (mask > 0.5).sum(dim=-1).to(torch.int32)


def node_stages(z: torch.Tensor, mask: torch.Tensor | None, w: NodeWeights, node_type: int = STARTING,
                heads: int = 4, inf: float = 1e9, transposed_bias: bool = False, eps: float = 1e-5) -> dict:
    """Every intermediate of one node, in kernel order ([B, R, S, ...]; the ending node's R is z's second
    pair axis).

    Reference: TriangleAttentionNode.forward / _norm_and_bias (bionemo_ir/_torch/layers/triangle_nodes.py:223-265),
    TriangleAttention._attend (bionemo_ir/_torch/layers/attention.py:257-296) and the VANILLA backend
    (bionemo_ir/_torch/attention_backend/triangle_attention/vanilla.py:58-73).
    """
    dtype = w.ln_w.dtype
    x = z.to(dtype)
    ending = node_type == ENDING
    xt = x.transpose(1, 2) if ending else x  # the node works on the transposed view
    B, R, S, c = xt.shape
    d = w.w_in.shape[0] // (4 * heads)
    normed = F.layer_norm(xt, (c,), w.ln_w, w.ln_b, eps)
    tb = F.linear(normed, w.w_bias)  # [B, R, S, H]
    if transposed_bias:
        tb = tb.transpose(1, 2)
    tb = tb.permute(0, 3, 1, 2)  # [B, H, q, k]
    if mask is None:
        mask = xt.new_ones(B, R, S)
    elif ending:
        mask = mask.transpose(1, 2)
    mb = additive_mask_bias(mask, inf, dtype)  # [B, R, 1, 1, S]
    proj = F.linear(normed, w.w_in, w.b_in)
    q, k, v, g = proj.split(heads * d, dim=-1)

    def heads_first(t):  # [B, R, S, H*d] -> [B, R, H, S, d]
        return t.reshape(B, R, S, heads, d).permute(0, 1, 3, 2, 4)

    qh, kh, vh = heads_first(q), heads_first(k), heads_first(v)
    a = torch.matmul(qh, kh.transpose(-1, -2))  # [B, R, H, S, S]
    a /= math.sqrt(d)  # in place, as the reference's eager backend does (vanilla.py:61-67)
    a += mb
    a += tb.unsqueeze(1)
    p = F.softmax(a, dim=-1)
    o = torch.matmul(p, vh)  # [B, R, H, S, d]
    o = o.transpose(-3, -2).reshape(B, R, S, heads * d)
    og = o * torch.sigmoid(g)
    update = F.linear(og, w.w_out, w.b_out)
    return {"x": xt, "normed": normed, "tri_bias": tb, "q": q, "k": k, "v": v, "g": g, "logits": a, "o": o,
            "og": og, "update": update, "mask": mask}


def node_forward(z: torch.Tensor, mask: torch.Tensor | None, w: NodeWeights, node_type: int = STARTING, *,
                 residual: bool = False, **kw) -> torch.Tensor:
    """Output of the node in the caller's layout [B, I, J, c] (update, or z + update)."""
    st = node_stages(z, mask, w, node_type, **kw)
    out = st["x"] + st["update"] if residual else st["update"]
    return out.transpose(1, 2) if node_type == ENDING else out


def triangle_bias(z: torch.Tensor, w: NodeWeights, node_type: int, *, eps: float = 1e-5, slab: int = 128) -> torch.Tensor:
    """The triangle bias ``[B, H, q, k]`` of every pair row, computed ``slab`` rows at a time so that a 4096-token
    tensor never needs a full-size fp32 temporary.  Same LayerNorm + projection as ``node_stages``
    (bionemo_ir/_torch/layers/triangle_nodes.py:252-265)."""
    dtype = w.ln_w.dtype
    xt = z.transpose(1, 2) if node_type == ENDING else z
    B, R, S, c = xt.shape
    tb = torch.empty(B, w.w_bias.shape[0], R, S, dtype=dtype, device=z.device)
    for r0 in range(0, R, slab):
        normed = F.layer_norm(xt[:, r0:r0 + slab].to(dtype), (c,), w.ln_w, w.ln_b, eps)
        tb[:, :, r0:r0 + slab] = F.linear(normed, w.w_bias).permute(0, 3, 1, 2)
    return tb


def node_forward_rows(z: torch.Tensor, mask: torch.Tensor | None, w: NodeWeights, node_type: int, rows: torch.Tensor,
                      *, residual: bool = False, heads: int = 4, inf: float = 1e9, eps: float = 1e-5,
                      tri_bias: torch.Tensor | None = None) -> torch.Tensor:
    """``node_forward`` restricted to the pair rows ``rows`` of the node's own row axis (second pair axis of ``z``
    for the ending node): returns ``[B, len(rows), S, c]`` in kernel order.

    A row's attention needs only that row of q/k/v/g plus the triangle bias of *all* rows, so sampled rows are exact
    and cheap; large shapes are checked and timed through this function.  ``tri_bias`` takes the bias of all rows
    from an earlier ``triangle_bias`` call (then only the sampled rows are normalised here); ``mask`` may then be
    given for the sampled rows only, ``[B, len(rows), S]`` in kernel order.  Same reference lines as ``node_stages``.
    """
    dtype = w.ln_w.dtype
    xt = z.transpose(1, 2) if node_type == ENDING else z
    B, R, S, c = xt.shape
    d = w.w_in.shape[0] // (4 * heads)
    if tri_bias is None:
        xt = xt.to(dtype)
        normed = F.layer_norm(xt, (c,), w.ln_w, w.ln_b, eps)
        tb = F.linear(normed, w.w_bias).permute(0, 3, 1, 2)  # [B, H, q, k] from every row
        n_s, x_s = normed[:, rows], xt[:, rows]
    else:
        tb = tri_bias
        x_s = xt[:, rows].to(dtype)
        n_s = F.layer_norm(x_s, (c,), w.ln_w, w.ln_b, eps)
    if mask is None:
        m_s = x_s.new_ones(B, len(rows), S)
    elif mask.shape[1] == len(rows) and mask.shape[1] != R:
        m_s = mask
    else:
        m_s = (mask.transpose(1, 2) if node_type == ENDING else mask)[:, rows]
    r = n_s.shape[1]
    proj = F.linear(n_s, w.w_in, w.b_in)
    q, k, v, g = proj.split(heads * d, dim=-1)

    def heads_first(t):
        return t.reshape(B, r, S, heads, d).permute(0, 1, 3, 2, 4)

    a = torch.matmul(heads_first(q), heads_first(k).transpose(-1, -2))
    a /= math.sqrt(d)  # in place, as the reference's eager backend does (vanilla.py:61-67)
    a += additive_mask_bias(m_s, inf, dtype)
    a += tb.unsqueeze(1)
    o = torch.matmul(F.softmax(a, dim=-1), heads_first(v)).transpose(-3, -2).reshape(B, r, S, heads * d)
    update = F.linear(o * torch.sigmoid(g), w.w_out, w.b_out)
    return x_s + update if residual else update


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor, lengths: torch.Tensor,
                   scale: float, empty_rows: str = "zeros") -> tuple[torch.Tensor, torch.Tensor]:
    """Length-masked attention with its log-sum-exp, fp32.

    q,k,v: [BR, S, H, d]; bias: [B, H, S, S]; lengths: [BR] int.  Keys t >= len are excluded; a row with
    len == 0 gives zeros and lse = -inf ("zeros") or the mean of v over all keys ("uniform").
    Reference: the compact reference of tests/_torch/test_triangle_attention_sm100_tail.py:55-66 and the
    empty-row assertions at lines 99-101.
    """
    BR, S, H, d = q.shape
    B = bias.shape[0]
    R = BR // B
    s = torch.einsum("nqhd,nkhd->nhqk", q.float(), k.float()) * scale
    s = s + bias.float().repeat_interleave(R, dim=0)
    key = torch.arange(S)
    valid = key[None, :] < lengths.reshape(-1, 1).long()  # [BR, S]
    s = s.masked_fill(~valid[:, None, None, :], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)  # [BR, H, S]
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("nhqk,nkhd->nqhd", p, v.float())
    empty = lengths.reshape(-1) == 0
    if empty.any() and empty_rows == "uniform":
        o[empty] = v.float()[empty].mean(dim=1, keepdim=True).expand(-1, S, -1, -1)
    return o, lse.permute(0, 2, 1)  # lse [BR, S, H]


def transition_forward(x: torch.Tensor, mask: torch.Tensor | None, w: TransitionWeights, *, residual: bool = False,
                       eps: float = 1e-5) -> torch.Tensor:
    """``[x +] mask * fc3(silu(gate) * value)`` with ``[value|gate] = LN(x) @ w1.T``.

    Reference: Transition._forward_impl (bionemo_ir/_torch/layers/transition.py:323-336), the SwiGLU of
    bionemo_ir/dsl_kernels/triton/fused_swiglu.py:78-82 (silu computed in fp32 and rounded to the activation dtype
    before the multiply) and transition_mlp_w_norm_reference
    (bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:305-338).
    """
    dtype = w.ln_w.dtype
    xd = x.to(dtype)
    normed = F.layer_norm(xd, (xd.shape[-1],), w.ln_w, w.ln_b, eps)
    h = F.linear(normed, w.w1)
    value, gate = h.chunk(2, dim=-1)
    act = F.silu(gate.float()).to(dtype) * value
    y = F.linear(act, w.w2)
    if mask is not None:
        m = mask if mask.dim() == y.dim() else mask.unsqueeze(-1)
        y = y * m.to(dtype)
    return xd + y if residual else y


@dataclass
class ReluTransitionWeights:
    """Parameters of the ReLU pair transition, named as in the reference state_dict."""

    ln_w: torch.Tensor  # layer_norm.weight [c]
    ln_b: torch.Tensor  # layer_norm.bias [c]
    w1: torch.Tensor  # linear_1.weight [n*c, c]
    b1: torch.Tensor  # linear_1.bias [n*c]
    w2: torch.Tensor  # linear_2.weight [c, n*c]
    b2: torch.Tensor  # linear_2.bias [c]

    def to(self, dtype: torch.dtype) -> "ReluTransitionWeights":
        return ReluTransitionWeights(*[t.to(dtype) for t in self.__dict__.values()])


def make_relu_transition_weights(seed: int, c: int = 128, n: int = 4, std: float = 0.05) -> ReluTransitionWeights:
    g = torch.Generator().manual_seed(seed)
    return ReluTransitionWeights(1 + 0.2 * torch.randn(c, generator=g), 0.2 * torch.randn(c, generator=g),
                                 torch.randn(n * c, c, generator=g) * std, 0.1 * torch.randn(n * c, generator=g),
                                 torch.randn(c, n * c, generator=g) * std, 0.1 * torch.randn(c, generator=g))


def relu_transition_forward(z: torch.Tensor, mask: torch.Tensor | None, w: ReluTransitionWeights, *,
                            residual: bool = False, eps: float = 1e-5) -> torch.Tensor:
    """``[z +] mask * linear_2(relu(linear_1(LayerNorm(z))))``, both linears with biases.

    Reference: PairTransition._forward_impl (bionemo_ir/_torch/layers/transition.py:631-656) and
    transition_mlp_w_norm_reference with activation="relu"
    (bionemo_ir/_torch/custom_ops/transition_mlp_w_norm/ops.py:305-338).
    """
    dtype = w.ln_w.dtype
    zd = z.to(dtype)
    h = F.relu(F.linear(F.layer_norm(zd, (zd.shape[-1],), w.ln_w, w.ln_b, eps), w.w1, w.b1))
    y = F.linear(h, w.w2, w.b2)
    if mask is not None:
        m = mask if mask.dim() == y.dim() else mask.unsqueeze(-1)
        y = y * m.to(dtype)
    return y + zd if residual else y


# ------------------------------------------------------------------------------------------ triangle multiplication

OUTGOING = 0
INCOMING = 1


@dataclass
class TriMulWeights:
    """Parameters of one triangle-multiplication node, named as in the reference state_dict."""

    ln_in_w: torch.Tensor  # norm_in.weight [c]
    ln_in_b: torch.Tensor  # norm_in.bias [c]
    w_p_in: torch.Tensor  # p_in.weight [2*hidden, c]: a rows, then b rows
    w_g_in: torch.Tensor  # g_in.weight [2*hidden, c]
    ln_out_w: torch.Tensor  # norm_out.weight [hidden]
    ln_out_b: torch.Tensor  # norm_out.bias [hidden]
    w_p_out: torch.Tensor  # p_out.weight [c, hidden]
    w_g_out: torch.Tensor  # g_out.weight [c, c]
    b_p_in: torch.Tensor | None = None
    b_g_in: torch.Tensor | None = None
    b_p_out: torch.Tensor | None = None
    b_g_out: torch.Tensor | None = None

    def fields(self):
        return (self.ln_in_w, self.ln_in_b, self.w_p_in, self.w_g_in, self.ln_out_w, self.ln_out_b, self.w_p_out,
                self.w_g_out, self.b_p_in, self.b_g_in, self.b_p_out, self.b_g_out)

    def to(self, dtype: torch.dtype) -> "TriMulWeights":
        return TriMulWeights(*[None if t is None else t.to(dtype) for t in self.fields()])


def make_trimul_weights(seed: int, c: int = 128, hidden: int = 128, std: float = 0.02, identity_ln: bool = True,
                        biases: bool = False) -> TriMulWeights:
    """Seeded weights in the recipe of ``init_module_weights`` (tests/_torch/__init__.py:33-63)."""
    g = torch.Generator().manual_seed(seed)
    w_p_in = torch.randn(2 * hidden, c, generator=g) * std
    w_g_in = torch.randn(2 * hidden, c, generator=g) * std
    w_p_out = torch.randn(c, hidden, generator=g) * std
    w_g_out = torch.randn(c, c, generator=g) * std
    if identity_ln:
        ln = [torch.ones(c), torch.zeros(c), torch.ones(hidden), torch.zeros(hidden)]
    else:
        ln = [1 + 0.2 * torch.randn(c, generator=g), 0.2 * torch.randn(c, generator=g),
              1 + 0.2 * torch.randn(hidden, generator=g), 0.2 * torch.randn(hidden, generator=g)]
    bs = [None] * 4
    if biases:
        bs = [0.1 * torch.randn(n, generator=g) for n in (2 * hidden, 2 * hidden, c, c)]
    return TriMulWeights(ln[0], ln[1], w_p_in, w_g_in, ln[2], ln[3], w_p_out, w_g_out, *bs)


def trimul_stages(z: torch.Tensor, mask: torch.Tensor | None, w: TriMulWeights, direction: int = OUTGOING,
                  eps: float = 1e-5, mean_normalization: bool = False) -> dict:
    """Every intermediate of one triangle-multiplication node.

    Reference: TriangleMultiplicationNode._forward_impl (bionemo_ir/_torch/layers/triangle_nodes.py:646-727),
    the unfused dual GEMMs (bionemo_ir/_torch/custom_ops/dual_gemm_x_x/ops.py:34-58,
    dual_gemm_x0_x1/ops.py:29-52), _contract_projection (triangle_nodes.py:596-612) and the tests' mirror
    RefTriangleMultiplicationNode.forward (tests/common/test_utils/boltz/ref_layers.py:59-96).
    """
    dtype = w.ln_in_w.dtype
    x = z.to(dtype)
    B, I, J, c = x.shape
    if mask is None:
        mask = x.new_ones(B, I, J)
    mask = mask.to(dtype)
    x_in = F.layer_norm(x, (c,), w.ln_in_w, w.ln_in_b, eps)
    ab = torch.sigmoid(F.linear(x_in, w.w_g_in, w.b_g_in)) * F.linear(x_in, w.w_p_in, w.b_p_in)
    ab = ab * mask.unsqueeze(-1)
    a, b = torch.chunk(ab, 2, dim=-1)
    if mean_normalization:
        n_valid = mask[:, 0, :].sum(dim=-1)
        b = b / (n_valid[:, None, None, None] + 1e-3)
    if direction == OUTGOING:
        t = torch.einsum("bikd,bjkd->bijd", a, b)
    else:
        t = torch.einsum("bkid,bkjd->bijd", a, b)
    hidden = t.shape[-1]
    normed = F.layer_norm(t.to(w.ln_out_w.dtype), (hidden,), w.ln_out_w, w.ln_out_b, eps)
    hp = w.w_p_out.dtype
    update = torch.sigmoid(F.linear(x_in.to(hp), w.w_g_out, w.b_g_out)) * F.linear(normed.to(hp), w.w_p_out, w.b_p_out)
    return {"x_in": x_in, "ab": ab, "a": a, "b": b, "contracted": t, "normed": normed, "update": update}


def trimul_forward(z: torch.Tensor, mask: torch.Tensor | None, w: TriMulWeights, direction: int = OUTGOING, *,
                   residual: bool = False, **kw) -> torch.Tensor:
    """Output of the node [B, I, J, c]: the update, or ``z + update`` with ``residual``
    (triangle_nodes.py:723-727: the unfused path adds the residual without masking it)."""
    st = trimul_stages(z, mask, w, direction, **kw)
    return z.to(st["update"].dtype) + st["update"] if residual else st["update"]


# ------------------------------------------------------------------------------- single track: attention with pair bias


@dataclass
class PairBiasAttentionWeights:
    """Parameters of AttentionPairBias as the pairformer builds it (state_dict names in brackets)."""

    norm_s_w: torch.Tensor | None  # [c_s]        (norm_s.weight; None without initial_norm)
    norm_s_b: torch.Tensor | None  # [c_s]        (norm_s.bias)
    w_in: torch.Tensor             # [4*c_s, c_s] (in_proj.weight; rows ordered q, gate, k, v)
    b_in: torch.Tensor             # [4*c_s]      (in_proj.bias)
    norm_z_w: torch.Tensor         # [c_z]        (proj_z.0.weight)
    norm_z_b: torch.Tensor         # [c_z]        (proj_z.0.bias)
    w_z: torch.Tensor              # [H, c_z]     (proj_z.1.weight)
    w_o: torch.Tensor              # [c_s, c_s]   (proj_o.weight)
    b_o: torch.Tensor | None = None  # [c_s]      (proj_o.bias, with out_bias)

    def to(self, dtype: torch.dtype) -> "PairBiasAttentionWeights":
        return PairBiasAttentionWeights(*[None if t is None else t.to(dtype) for t in self.__dict__.values()])


def make_pair_bias_attention_weights(seed: int, c_s: int = 384, c_z: int = 128, heads: int = 16, std: float = 0.05,
                                     initial_norm: bool = True, out_bias: bool = False) -> PairBiasAttentionWeights:
    g = torch.Generator().manual_seed(seed)
    w_in = torch.randn(4 * c_s, c_s, generator=g) * std
    b_in = torch.randn(4 * c_s, generator=g) * 0.1
    w_z = torch.randn(heads, c_z, generator=g) * std
    w_o = torch.randn(c_s, c_s, generator=g) * std
    norm_z_w = 1 + 0.2 * torch.randn(c_z, generator=g)
    norm_z_b = 0.2 * torch.randn(c_z, generator=g)
    norm_s_w = 1 + 0.2 * torch.randn(c_s, generator=g) if initial_norm else None
    norm_s_b = 0.2 * torch.randn(c_s, generator=g) if initial_norm else None
    b_o = 0.1 * torch.randn(c_s, generator=g) if out_bias else None
    return PairBiasAttentionWeights(norm_s_w, norm_s_b, w_in, b_in, norm_z_w, norm_z_b, w_z, w_o, b_o)


def pair_bias_attention_forward(s: torch.Tensor, z: torch.Tensor, mask: torch.Tensor, w: PairBiasAttentionWeights, *,
                                heads: int = 16, inf: float = 1e9, eps: float = 1e-5) -> torch.Tensor:
    """The update of the single representation ``s [B, N, c_s]`` by self-attention with a bias from ``z [B, N, N, c_z]``.

    Reference: AttentionPairBias.forward without AdaLN, key gathering or output gate
    (bionemo_ir/_torch/layers/attention.py:957-1046): initial LayerNorm (_prep_inputs), ``q, g, k, v = in_proj(s)``
    (_prep_qkvg, lines 790-792), pair bias ``moveaxis(Linear(LayerNorm(z)))`` (project_pair_bias, lines 835-852;
    LNProjMoveaxisPad, bionemo_ir/_torch/custom_ops/fused_ln_proj_moveaxis_pad.py:15-22), additive key mask
    ``(1 - mask) * -inf`` (_prep_mask_bias, lines 917-921), ``softmax(q·kᵀ / sqrt(d) + mask + bias) · v``
    (VanillaPairwiseAttention.forward, bionemo_ir/_torch/attention_backend/pairwise_attention/vanilla.py:59-77) and
    ``proj_o(sigmoid(g) * o)`` (_attention_output, lines 1114-1119).
    """
    dtype = w.w_in.dtype
    B, N, c_s = s.shape
    d = c_s // heads
    x = s.to(dtype)
    if w.norm_s_w is not None:
        x = F.layer_norm(x, (c_s,), w.norm_s_w, w.norm_s_b, eps)
    q, g, k, v = F.linear(x, w.w_in, w.b_in).split(c_s, dim=-1)
    zn = F.layer_norm(z.to(dtype), (z.shape[-1],), w.norm_z_w, w.norm_z_b, eps)
    pair_bias = F.linear(zn, w.w_z).movedim(-1, -3)  # [B, H, N, N]
    mask_bias = ((1 - mask.float()) * -inf)[:, None, None, :]

    def heads_first(t):
        return t.reshape(B, N, heads, d).transpose(1, 2)  # [B, H, N, d]

    a = torch.matmul(heads_first(q), heads_first(k).transpose(-1, -2)) / math.sqrt(d)
    a = a + mask_bias.to(dtype) + pair_bias
    a = torch.softmax(a, dim=-1)
    o = torch.matmul(a, heads_first(v)).transpose(1, 2).reshape(B, N, c_s)
    return F.linear(o * torch.sigmoid(g), w.w_o, w.b_o)
