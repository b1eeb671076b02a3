"""Tensor-level wrappers over the C ABI (``include/b200ta.h``).

PyTorch is used here only for device memory and the current stream; every
computation is a call into libb200ta.so.  Shapes follow the reference layers:
``z`` is a pair tensor ``[B, I, J, 128]``; the ending node runs the same kernels
on the transposed view by swapping the two pair strides (no copy).
"""

from __future__ import annotations

import math

import torch

from . import _lib

C = 128
HEADS = 4
HEAD_DIM = 32
HIDDEN = 512
BIAS_SCALE = 5.656854249492381  # sqrt(head_dim): the kernels keep the triangle bias divided by the softmax scale


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require_cuda_bf16(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this package has no CPU path)")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")


def _weight_dtype(*tensors: torch.Tensor | None) -> int:
    """The common dtype code of a set of weights; also refuses host tensors, whose addresses a kernel must never see."""
    devices = {t.device for t in tensors if t is not None}
    if len(devices) != 1 or next(iter(devices)).type != "cuda":
        raise ValueError(f"weights must all live on one CUDA device, got {sorted(map(str, devices))}")
    dtypes = {t.dtype for t in tensors if t is not None}
    if dtypes == {torch.bfloat16}:
        return _lib.DTYPE_BF16
    if dtypes == {torch.float32}:
        return _lib.DTYPE_F32
    raise ValueError(f"weights must all be bfloat16 or all float32, got {sorted(map(str, dtypes))}")


def _contig(t: torch.Tensor | None) -> torch.Tensor | None:
    return None if t is None else t.contiguous()


def pack_node_weights(ln_w, ln_b, w_in, b_in, w_bias, w_out, b_out) -> torch.Tensor:
    """Fold LayerNorm into the q/k/v/g + triangle-bias projection; returns the opaque packed buffer."""
    ts = [_contig(t) for t in (ln_w, ln_b, w_in, b_in, w_bias, w_out, b_out)]
    if tuple(ts[2].shape) != (4 * HEADS * HEAD_DIM, C) or tuple(ts[4].shape) != (HEADS, C) or tuple(ts[5].shape) != (C, HEADS * HEAD_DIM):
        raise ValueError(
            f"kernels are specialised for c_z={C}, {HEADS} heads of {HEAD_DIM}: got in_proj {tuple(ts[2].shape)}, "
            f"pair_bias_proj {tuple(ts[4].shape)}, o_proj {tuple(ts[5].shape)}"
        )
    dt = _weight_dtype(*ts)
    packed = torch.empty(_lib.load().b200ta_node_pack_bytes(), dtype=torch.uint8, device=ts[2].device)
    _lib.call("b200ta_pack_node_weights", *[_ptr(t) for t in ts], dt, packed.data_ptr(), _stream())
    return packed


def pack_transition_weights(ln_w, ln_b, w1, w2) -> torch.Tensor:
    """Fold LayerNorm into fused_fc2_fc1 (gate rows pre-halved); returns the opaque packed buffer."""
    ts = [_contig(t) for t in (ln_w, ln_b, w1, w2)]
    if tuple(ts[2].shape) != (2 * HIDDEN, C) or tuple(ts[3].shape) != (C, HIDDEN):
        raise ValueError(f"kernel is specialised for dim={C}, hidden={HIDDEN}: got {tuple(ts[2].shape)}, {tuple(ts[3].shape)}")
    dt = _weight_dtype(*ts)
    packed = torch.empty(_lib.load().b200ta_transition_pack_bytes(), dtype=torch.uint8, device=ts[2].device)
    _lib.call("b200ta_pack_transition_weights", *[_ptr(t) for t in ts], dt, packed.data_ptr(), _stream())
    return packed


def pack_relu_transition_weights(ln_w, ln_b, w1, b1, w2, b2) -> torch.Tensor:
    """Fold LayerNorm into linear_1 of the ReLU pair transition; returns the opaque packed buffer."""
    ts = [_contig(t) for t in (ln_w, ln_b, w1, b1, w2, b2)]
    if tuple(ts[2].shape) != (HIDDEN, C) or tuple(ts[4].shape) != (C, HIDDEN):
        raise ValueError(f"kernel is specialised for width={C}, hidden={HIDDEN}: got {tuple(ts[2].shape)}, {tuple(ts[4].shape)}")
    dt = _weight_dtype(*ts)
    packed = torch.empty(_lib.load().b200ta_transition_pack_bytes(), dtype=torch.uint8, device=ts[2].device)
    _lib.call("b200ta_pack_relu_transition_weights", *[_ptr(t) for t in ts], dt, packed.data_ptr(), _stream())
    return packed


def _pair_strides(z: torch.Tensor, ending: bool) -> tuple[int, int, int, int, int, int]:
    """(B, R, S, stride_b, stride_r, stride_s) of a [B, I, J, C] tensor as the kernels see it."""
    if z.dim() != 4 or z.shape[-1] != C or z.stride(-1) != 1:
        raise ValueError(f"expected a [B, I, J, {C}] tensor with unit channel stride, got {tuple(z.shape)}")
    B, I, J, _ = z.shape
    sb, si, sj, _ = z.stride()
    return (B, J, I, sb, sj, si) if ending else (B, I, J, sb, si, sj)


def pad8(n: int) -> int:
    return -(-n // 8) * 8


def prologue(z, packed, eps: float = 1e-5, *, ending: bool = False, want_qkvg: bool = True,
             qkvg: torch.Tensor | None = None, bias: torch.Tensor | None = None,
             want_bias: bool = True, transposed_bias: bool = False):
    """LayerNorm + q/k/v/g projection + triangle-bias projection.

    Returns ``(qkvg, bias)``: ``qkvg`` is ``[4, B*R, H, S, D]`` (q, k, v, g planes, head-major; the g plane
    holds ``sigmoid(gate logit)``), ``bias`` is ``[B, H, S_q, S_pad]`` multiplied by ``BIAS_SCALE``
    (divided by the softmax scale).  With ``ending`` the rows R run over the second pair axis of ``z``.
    """
    _require_cuda_bf16("z", z)
    B, R, S, sb, sr, ss = _pair_strides(z, ending)
    S_pad = pad8(S)
    if want_qkvg and qkvg is None:
        qkvg = torch.empty((4, B * R, HEADS, S, HEAD_DIM), dtype=torch.bfloat16, device=z.device)
    if want_bias and bias is None:
        if R != S:
            raise ValueError("the triangle bias needs a square pair tensor")
        alloc = torch.zeros if transposed_bias else torch.empty
        bias = alloc((B, HEADS, R, S_pad), dtype=torch.bfloat16, device=z.device)
    if qkvg is not None:
        qs = (qkvg.stride(0), qkvg.stride(1), qkvg.stride(2), qkvg.stride(3))
    else:
        qs = (0, 0, 0, 0)
    if bias is not None:
        bs = (bias.stride(0), bias.stride(1), bias.stride(2), bias.stride(3))
        if transposed_bias:
            bs = (bs[0], bs[1], bs[3], bs[2])
    else:
        bs = (0, 0, 0, 0)
    _lib.call("b200ta_prologue", z.data_ptr(), sb, sr, ss, packed.data_ptr(), float(eps), _ptr(qkvg), *qs,
              1 if want_qkvg else 0, _ptr(bias if want_bias else None), *bs, B, R, S,
              S if transposed_bias else S_pad,  # transposed: the key padding lies along the other axis; no zero fill
              _stream())
    return qkvg, bias


def attention(qkvg: torch.Tensor, bias: torch.Tensor, lengths: torch.Tensor | None, B: int, R: int, S: int, *,
              gate: bool = True, out: torch.Tensor | None = None, lse: torch.Tensor | None = None,
              empty_row_mode: int = _lib.EMPTY_ROW_UNIFORM, scale: float | None = None,
              key_mask: torch.Tensor | None = None) -> torch.Tensor:
    """Biased, length-masked attention over the head-major ``qkvg`` planes; returns ``[B, R, S, 128]``.

    ``bias`` is the triangle bias times ``BIAS_SCALE`` and, with ``gate``, the g plane holds gate factors in
    [0, 1] (sigmoid already applied) - the forms ``prologue`` writes.  ``key_mask`` (int32 ``[B, R, ceil(S/32)]``,
    from :func:`key_mask_bits`) switches single keys of a row off; ``lengths`` must then be the bits' row lengths.
    """
    _require_cuda_bf16("qkvg", qkvg)
    _require_cuda_bf16("bias", bias)
    if out is None:
        out = torch.empty((B, R, S, C), dtype=torch.bfloat16, device=qkvg.device)
    if scale is None:
        scale = 1.0 / math.sqrt(HEAD_DIM)
    if lengths is not None:
        if lengths.dtype != torch.int32 or not lengths.is_cuda:
            raise ValueError("lengths must be a CUDA int32 tensor")
        if lengths.numel() == B * R:
            lengths = lengths.reshape(B, R)
            ls = (lengths.stride(0), lengths.stride(1))
        elif lengths.numel() == B:
            lengths = lengths.reshape(B)
            ls = (lengths.stride(0), 0)
        else:
            raise ValueError(f"lengths must hold B*R={B * R} or B={B} values, got {lengths.numel()}")
    else:
        ls = (0, 0)
    q, k, v, g = qkvg[0], qkvg[1], qkvg[2], qkvg[3]
    for t in (k, v, g):
        if t.stride() != q.stride():
            raise ValueError("q, k, v, g planes must share strides")
    o4 = out.view(B * R, S, HEADS, HEAD_DIM)
    head = (q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr() if gate else None, q.stride(0), q.stride(1), q.stride(2),
            bias.data_ptr(), bias.stride(0), bias.stride(1), bias.stride(2), _ptr(lengths), *ls)
    tail = (o4.data_ptr(), o4.stride(0), o4.stride(1), o4.stride(2), _ptr(lse), float(scale), int(empty_row_mode), B, R, S,
            bias.shape[-1], _stream())
    if key_mask is None:
        _lib.call("b200ta_attention", *head, *tail)
    else:
        words = (S + 31) // 32
        if (key_mask.dtype != torch.int32 or not key_mask.is_cuda or tuple(key_mask.shape) != (B, R, words)
                or key_mask.stride(2) != 1 or lengths is None or lengths.numel() != B * R):
            raise ValueError(f"key_mask must be a CUDA int32 tensor [B={B}, R={R}, {words}] with unit word stride, "
                             "passed together with its [B, R] row lengths")
        _lib.call("b200ta_attention_masked", *head, key_mask.data_ptr(), key_mask.stride(0), key_mask.stride(1), *tail)
    return out


def key_mask_bits(valid: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``valid`` ``[B, R, S]`` (bool: key t of pair row (b, r) takes part) -> (row lengths ``[B, R]`` int32 = last
    valid key + 1, bit words ``[B, R, ceil(S/32)]`` int32 with bit ``t % 32`` of word ``t // 32`` set for valid keys):
    the payload of ``attention(..., key_mask=...)`` for masks that are not left-aligned."""
    B, R, S = valid.shape
    words = (S + 31) // 32
    position = torch.arange(1, S + 1, device=valid.device, dtype=torch.int32)
    lengths = (valid.to(torch.int32) * position).amax(dim=-1).contiguous()
    padded = torch.zeros((B, R, words * 32), dtype=torch.int64, device=valid.device)
    padded[..., :S] = valid
    weights = torch.ones(32, dtype=torch.int64, device=valid.device) << torch.arange(32, device=valid.device)
    bits = (padded.view(B, R, words, 32) * weights).sum(dim=-1)
    return lengths, bits.to(torch.int32).contiguous()  # the conversion wraps: bit 31 becomes the sign bit


def node_workspace_bytes(B: int, N: int) -> int:
    return int(_lib.load().b200ta_node_workspace_bytes(B, N))


def node_forward(z: torch.Tensor, packed: torch.Tensor, lengths: torch.Tensor | None, eps: float = 1e-5, *,
                 ending: bool = False, residual: bool = False, out: torch.Tensor | None = None,
                 workspace: torch.Tensor | None = None, empty_row_mode: int = _lib.EMPTY_ROW_UNIFORM) -> torch.Tensor:
    """A whole triangle-attention node in one library call (``b200ta_node_forward``).

    ``z`` / ``out`` are square pair tensors ``[B, N, N, 128]`` in the caller's order; ``lengths`` is ``[B, N]`` int32
    (valid keys per kernel row, i.e. per second pair index for the ending node) or ``None``; ``workspace`` is a
    uint8 scratch tensor of at least :func:`node_workspace_bytes` bytes (allocated when omitted).
    """
    _require_cuda_bf16("z", z)
    B, R, S, sb, sr, ss = _pair_strides(z, ending)
    if R != S:
        raise ValueError("node_forward needs a square pair tensor")
    if out is None:
        out = torch.empty((B, R, S, C), dtype=torch.bfloat16, device=z.device)
    _require_cuda_bf16("out", out)
    oB, oR, oS, osb, osr, oss = _pair_strides(out, ending)
    if (oB, oR, oS) != (B, R, S):
        raise ValueError(f"out shape {tuple(out.shape)} does not match z {tuple(z.shape)}")
    need = node_workspace_bytes(B, R)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=z.device)
    elif workspace.numel() * workspace.element_size() < need or not workspace.is_contiguous():
        raise ValueError(f"workspace must be contiguous and hold at least {need} bytes")
    if lengths is not None:
        if lengths.dtype != torch.int32 or not lengths.is_cuda or lengths.numel() != B * R:
            raise ValueError(f"lengths must be a CUDA int32 tensor with B*N={B * R} values")
        lengths = lengths.reshape(B, R)
        ls = (lengths.stride(0), lengths.stride(1))
    else:
        ls = (0, 0)
    _lib.call("b200ta_node_forward", z.data_ptr(), sb, sr, ss, packed.data_ptr(), float(eps), _ptr(lengths), *ls,
              int(empty_row_mode), 1 if residual else 0, out.data_ptr(), osb, osr, oss, workspace.data_ptr(),
              workspace.numel() * workspace.element_size(), B, R, _stream())
    return out


def node_static_max_positions() -> int:
    return int(_lib.load().b200ta_node_static_max_positions())


def node_forward_static(z: torch.Tensor, packed: torch.Tensor, lengths: torch.Tensor | None, out: torch.Tensor,
                        eps: float = 1e-5, *, ending: bool = False, residual: bool = False,
                        empty_row_mode: int = _lib.EMPTY_ROW_UNIFORM) -> torch.Tensor:
    """:func:`node_forward` through ``b200ta_node_forward_static``: no workspace, nothing allocated.

    For callers that must not allocate device memory (for example inside a stream capture): the intermediates
    go to an array built into the library, which limits the problem to ``B*N*N <= node_static_max_positions()``
    and means that calls which could overlap on the GPU must be ordered by the caller.  ``out`` has to be given
    (this wrapper allocates nothing either) and may be ``z`` itself when ``residual`` is set.
    """
    _require_cuda_bf16("z", z)
    _require_cuda_bf16("out", out)
    B, R, S, sb, sr, ss = _pair_strides(z, ending)
    if R != S:
        raise ValueError("node_forward_static needs a square pair tensor")
    oB, oR, oS, osb, osr, oss = _pair_strides(out, ending)
    if (oB, oR, oS) != (B, R, S):
        raise ValueError(f"out shape {tuple(out.shape)} does not match z {tuple(z.shape)}")
    if lengths is not None:
        if lengths.dtype != torch.int32 or not lengths.is_cuda or lengths.dim() != 2 or tuple(lengths.shape) != (B, R):
            raise ValueError(f"lengths must be a CUDA int32 tensor of shape [{B}, {R}]")
        ls = (lengths.stride(0), lengths.stride(1))
    else:
        ls = (0, 0)
    _lib.call("b200ta_node_forward_static", z.data_ptr(), sb, sr, ss, packed.data_ptr(), float(eps), _ptr(lengths), *ls,
              int(empty_row_mode), 1 if residual else 0, out.data_ptr(), osb, osr, oss, B, R, _stream())
    return out


def epilogue(og: torch.Tensor, packed: torch.Tensor, residual: torch.Tensor | None, out: torch.Tensor | None = None,
             *, ending: bool = False) -> torch.Tensor:
    """``out = residual + og · W_oᵀ + b_o``.

    ``og`` is ``[B, R, S, 128]`` in kernel order; ``residual`` / ``out`` are pair tensors ``[B, I, J, 128]`` in the
    caller's order (for ``ending`` they are addressed through swapped strides).
    """
    _require_cuda_bf16("og", og)
    B, R, S, _ = og.shape
    if out is None:
        out = torch.empty((B, S, R, C) if ending else (B, R, S, C), dtype=torch.bfloat16, device=og.device)
    oB, oR, oS, osb, osr, oss = _pair_strides(out, ending)
    if (oB, oR, oS) != (B, R, S):
        raise ValueError(f"out shape {tuple(out.shape)} does not match og {tuple(og.shape)}")
    if residual is not None:
        _require_cuda_bf16("residual", residual)
        rB, rR, rS, rsb, rsr, rss = _pair_strides(residual, ending)
        if (rB, rR, rS) != (B, R, S):
            raise ValueError(f"residual shape {tuple(residual.shape)} does not match og {tuple(og.shape)}")
    else:
        rsb = rsr = rss = 0
    _lib.call("b200ta_epilogue", og.data_ptr(), og.stride(0), og.stride(1), og.stride(2), packed.data_ptr(),
              _ptr(residual), rsb, rsr, rss, out.data_ptr(), osb, osr, oss, B, R, S, _stream())
    return out


def transition(x: torch.Tensor, packed: torch.Tensor, mask: torch.Tensor | None = None, eps: float = 1e-5, *,
               residual: bool = False, out: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """Fused LayerNorm -> SwiGLU MLP (-> mask) (-> + x) over the rows of ``x[..., 128]``; with ``relu`` the ReLU
    form ``linear_2(relu(linear_1(LayerNorm(x))))`` (``packed`` from :func:`pack_relu_transition_weights`)."""
    _require_cuda_bf16("x", x)
    if x.shape[-1] != C:
        raise ValueError(f"last dimension must be {C}")
    x2 = x.reshape(-1, C) if x.is_contiguous() else None
    if x2 is None:
        raise ValueError("transition needs a contiguous input")
    if out is None:
        out = torch.empty_like(x)
    elif not out.is_contiguous() or out.shape != x.shape:
        raise ValueError("out must be contiguous and shaped like x")
    if mask is not None:
        mask = mask.to(torch.bfloat16).expand(x.shape[:-1]).contiguous()
    _lib.call("b200ta_transition_relu" if relu else "b200ta_transition", x2.data_ptr(), C, _ptr(mask), packed.data_ptr(),
              float(eps), out.data_ptr(), C, x2.shape[0], 1 if residual else 0, _stream())
    return out


# ------------------------------------------------------------------------------------------ triangle multiplication

TRI_HIDDEN = 128


def pad16(n: int) -> int:
    return -(-n // 16) * 16


def pack_trimul_weights(ln_in_w, ln_in_b, w_p_in, b_p_in, w_g_in, b_g_in, ln_out_w, ln_out_b, w_p_out, b_p_out, w_g_out,
                        b_g_out) -> torch.Tensor:
    """Fold norm_in into p_in / g_in / g_out and norm_out into p_out; returns the opaque packed buffer."""
    ts = [_contig(t) for t in (ln_in_w, ln_in_b, w_p_in, b_p_in, w_g_in, b_g_in, ln_out_w, ln_out_b, w_p_out, b_p_out,
                               w_g_out, b_g_out)]
    if (tuple(ts[2].shape) != (2 * TRI_HIDDEN, C) or tuple(ts[4].shape) != (2 * TRI_HIDDEN, C)
            or tuple(ts[8].shape) != (C, TRI_HIDDEN) or tuple(ts[10].shape) != (C, C)):
        raise ValueError(f"kernels are specialised for dim={C}, hidden_dim={TRI_HIDDEN}: got p_in {tuple(ts[2].shape)}, "
                         f"g_in {tuple(ts[4].shape)}, p_out {tuple(ts[8].shape)}, g_out {tuple(ts[10].shape)}")
    dt = _weight_dtype(*ts)
    packed = torch.empty(_lib.load().b200ta_trimul_pack_bytes(), dtype=torch.uint8, device=ts[2].device)
    _lib.call("b200ta_pack_trimul_weights", *[_ptr(t) for t in ts], dt, packed.data_ptr(), _stream())
    return packed


def _mask_strides(mask: torch.Tensor | None, B: int, I: int, J: int, swap: bool):
    if mask is None:
        return None, (0, 0, 0)
    if mask.dtype != torch.float32 or not mask.is_cuda or tuple(mask.shape) != (B, I, J):
        raise ValueError(f"mask must be a CUDA float32 tensor of shape {(B, I, J)}, got {mask.dtype} {tuple(mask.shape)}")
    sb, si, sj = mask.stride()
    return mask, ((sb, sj, si) if swap else (sb, si, sj))


def trimul_project(z: torch.Tensor, mask: torch.Tensor | None, packed: torch.Tensor, eps: float = 1e-5, *,
                   incoming: bool = False, b_scale: torch.Tensor | None = None,
                   ab: torch.Tensor | None = None) -> torch.Tensor:
    """Gated, masked input projection, channel-major: returns ``ab [B, 256, N, pitch]`` (a planes, then b planes;
    the contraction index is the last axis).  ``incoming`` walks ``z`` and ``mask`` through swapped pair strides."""
    _require_cuda_bf16("z", z)
    B, R, S, sb, sr, ss = _pair_strides(z, incoming)
    if R != S:
        raise ValueError("triangle multiplication needs a square pair tensor")
    pitch = pad16(S)
    if ab is None:
        ab = torch.empty((B, 2 * TRI_HIDDEN, R, pitch), dtype=torch.bfloat16, device=z.device)
    mask, ms = _mask_strides(mask, B, z.shape[1], z.shape[2], incoming)
    _lib.call("b200ta_trimul_project", z.data_ptr(), sb, sr, ss, _ptr(mask), *ms, _ptr(b_scale), packed.data_ptr(),
              float(eps), ab.data_ptr(), pitch, B, R, S, _stream())
    return ab


def trimul_contract(ab: torch.Tensor, N: int, x: torch.Tensor | None = None) -> torch.Tensor:
    """``x[b, d, i, j] = sum_k a[b, d, i, k] * b[b, d, j, k]`` on the planes ``trimul_project`` wrote."""
    B, _, _, pitch = ab.shape
    if x is None:
        x = torch.empty((B, TRI_HIDDEN, N, pitch), dtype=torch.bfloat16, device=ab.device)
    _lib.call("b200ta_trimul_contract", ab.data_ptr(), x.data_ptr(), B, N, pitch, _stream())
    return x


def trimul_output(z: torch.Tensor, x: torch.Tensor, packed: torch.Tensor, eps: float = 1e-5, *, residual: bool = False,
                  mask: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Output normalisation, projection and gate (+ ``z``, then ``* mask`` when a mask is given)."""
    _require_cuda_bf16("z", z)
    B, I, J, sb, si, sj = _pair_strides(z, False)
    if out is None:
        out = torch.empty((B, I, J, C), dtype=torch.bfloat16, device=z.device)
    oB, oI, oJ, osb, osi, osj = _pair_strides(out, False)
    if (oB, oI, oJ) != (B, I, J):
        raise ValueError(f"out has shape {tuple(out.shape)}, expected {(B, I, J, C)}")
    mask, ms = _mask_strides(mask, B, I, J, False)
    _lib.call("b200ta_trimul_output", z.data_ptr(), sb, si, sj, x.data_ptr(), x.shape[-1], _ptr(mask), *ms,
              packed.data_ptr(), float(eps), 1 if residual else 0, out.data_ptr(), osb, osi, osj, B, I, _stream())
    return out


# ---- single track: pair bias and dense layers ---------------------------------------------------------------------

LINEAR_PLANES, LINEAR_ROWS, LINEAR_SWIGLU = 0, 1, 2
SINGLE_HEADS = 16  # heads of the single-track attention the head-major form of ``linear`` writes


def pack_pair_bias_weights(ln_w, ln_b, w_z: torch.Tensor, bias_scale: float) -> torch.Tensor:
    """Fold LayerNorm into the pair-bias projection ``w_z [heads, 128]``; the result is multiplied by ``bias_scale``."""
    ts = [_contig(t) for t in (ln_w, ln_b, w_z)]
    heads = ts[2].shape[0]
    if ts[2].dim() != 2 or ts[2].shape[1] != C or not 0 < heads <= 16 or heads % 2:
        raise ValueError(f"the pair-bias kernel takes an even number of at most 16 heads over c_z={C}; got {tuple(ts[2].shape)}")
    dt = _weight_dtype(*ts)
    packed = torch.empty(_lib.load().b200ta_node_pack_bytes(), dtype=torch.uint8, device=ts[2].device)
    _lib.call("b200ta_pack_pair_bias_weights", _ptr(ts[0]), _ptr(ts[1]), _ptr(ts[2]), heads, float(bias_scale), dt,
              packed.data_ptr(), _stream())
    return packed


def pair_bias(z: torch.Tensor, packed: torch.Tensor, heads: int, eps: float = 1e-5,
              bias: torch.Tensor | None = None) -> torch.Tensor:
    """``bias[b, h, q, k] = scale * LayerNorm(z[b, q, k]) · w_z[h]`` as ``[B, heads, Q, pad8(K)]`` (pad written as 0)."""
    _require_cuda_bf16("z", z)
    B, Q, K, sb, sq, sk = _pair_strides(z, False)
    if bias is None:
        bias = torch.empty((B, heads, Q, pad8(K)), dtype=torch.bfloat16, device=z.device)
    _require_cuda_bf16("bias", bias)
    if tuple(bias.shape) != (B, heads, Q, pad8(K)):
        raise ValueError(f"bias must have shape {(B, heads, Q, pad8(K))}, got {tuple(bias.shape)}")
    _lib.call("b200ta_pair_bias", z.data_ptr(), sb, sq, sk, packed.data_ptr(), float(eps), bias.data_ptr(),
              *bias.stride(), heads, B, Q, K, pad8(K), _stream())
    return bias


def row_stats(x: torch.Tensor, eps: float = 1e-5, stats: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm statistics ``{rstd, -mean * rstd}`` of every row of ``x [..., K]`` (contiguous bf16) as ``[rows, 2]``."""
    _require_cuda_bf16("x", x)
    if not x.is_contiguous():
        raise ValueError("row_stats needs a contiguous tensor")
    K = x.shape[-1]
    rows = x.numel() // K
    if stats is None:
        stats = torch.empty((rows, 2), dtype=torch.float32, device=x.device)
    _lib.call("b200ta_row_stats", x.data_ptr(), K, rows, K, float(eps), stats.data_ptr(), _stream())
    return stats


def linear(a: torch.Tensor, w: torch.Tensor, sc: torch.Tensor, mode: int, *, B: int, rows: int,
           a_strides: tuple[int, int, int] | None = None, stats: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``finish(A · wᵀ)`` on the tensor cores (``b200ta_linear``).

    ``a``: bf16 ``[B, rows, K]`` contiguous, or any layout with ``a_strides = (batch, row, 128-channel chunk)`` in
    elements; ``w``: bf16 ``[N, K]``; ``sc``: fp32 ``[N, 2]`` {rowsum, const}; ``stats`` from :func:`row_stats`.
    Returns ``[4, B, 16, rows, 32]`` (``LINEAR_PLANES``), ``[B, rows, N]`` (``LINEAR_ROWS``, plus ``residual``) or
    ``[B, rows, N // 2]`` (``LINEAR_SWIGLU``).
    """
    _require_cuda_bf16("a", a)
    _require_cuda_bf16("w", w)
    N, K = w.shape
    if not w.is_contiguous() or sc.dtype != torch.float32 or tuple(sc.shape) != (N, 2) or not sc.is_contiguous():
        raise ValueError("w must be contiguous [N, K] and sc a contiguous fp32 [N, 2]")
    if a_strides is None:
        if not a.is_contiguous() or a.numel() != B * rows * K:
            raise ValueError(f"a must be a contiguous [B={B}, rows={rows}, K={K}] tensor, got {tuple(a.shape)}")
        a_strides = (rows * K, K, C)
    if mode == LINEAR_PLANES:
        shape = (4, B, SINGLE_HEADS, rows, HEAD_DIM)
    elif mode == LINEAR_ROWS:
        shape = (B, rows, N)
    elif mode == LINEAR_SWIGLU:
        shape = (B, rows, N // 2)
    else:
        raise ValueError(f"unknown mode {mode}")
    if out is None:
        out = torch.empty(shape, dtype=torch.bfloat16, device=a.device)
    _require_cuda_bf16("out", out)
    if tuple(out.shape) != shape or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous tensor of shape {shape}")
    if residual is not None:
        _require_cuda_bf16("residual", residual)
        if tuple(residual.shape) != shape or not residual.is_contiguous():
            raise ValueError(f"residual must be a contiguous tensor of shape {shape}")
    os_row = 0 if mode == LINEAR_PLANES else shape[-1]
    plane_stride = out.stride(0) if mode == LINEAR_PLANES else 0
    _lib.call("b200ta_linear", a.data_ptr(), *a_strides, w.data_ptr(), sc.data_ptr(), _ptr(stats), _ptr(residual),
              0 if residual is None else shape[-1], out.data_ptr(), os_row, plane_stride, mode, B, rows, K, N, _stream())
    return out
