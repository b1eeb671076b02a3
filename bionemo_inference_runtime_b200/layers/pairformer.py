"""Pair-track Pairformer blocks on the sm_100a kernels.

Counterparts of ``PairformerNoSeqLayer`` and ``PairformerNoSeqModule``
(``bionemo_ir/_torch/layers/transformers/pairformer.py:255-363``), the reference's Pairformer without the single
track: per block triangle multiplication outgoing and incoming, triangle attention starting and ending node and the
pair transition, every update added to ``z`` (``_transform_z``, lines 174-216 of the same file).  Submodule names
(``tri_mul_out``, ``tri_mul_in``, ``tri_attn_start``, ``tri_attn_end``, ``transition_z``) and therefore the
``state_dict`` keys are the reference's, so the pair-track part of a Pairformer checkpoint loads unchanged.

The module can replay its whole stack from one CUDA graph (``use_cuda_graph=True``): at 15 kernel launches per block
the launch overhead is what the reference removes with graph capture at small token counts
(``bionemo_ir/_torch/graph_optimization/region.py``).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .attention_backend import AttentionMetadata, PrecomputedPairMasks, precompute_pair_masks
from .auto_chunk import CHUNK_REGISTRY, PAIR_TRANSITION
from .buffers import PreallocatedBuffers
from .transition import Transition
from .triangle_multiplication import (TriangleMultiplicationMetadata, TriangleMultiplicationNode,
                                      TriangleMultiplicationNodeType, precompute_trimul_metadata)
from .triangle_nodes import TriangleAttentionEndingNode, TriangleAttentionStartingNode


class PairformerNoSeqLayer(nn.Module):
    def __init__(self, *, layer_idx: int, token_z: int = 128, pairwise_head_width: int = 32, pairwise_num_heads: int = 4,
                 dtype: torch.dtype = None, eps: float = 1e-5, inf: float = 1e9, triangle_attn_backend: str = "VANILLA",
                 skip_create_weights: bool = False, trimul_high_precision: bool = True,
                 trimul_mean_normalization: bool = False, pair_mask_left_aligned: bool = True,
                 pair_transition_factor: int = 4, tri_attn_transposed_bias: bool = False, **kwargs):
        """Arguments as the reference layer takes them for its pair track (pairformer.py:45-67); arguments of the
        single track (``token_s``, ``num_heads``, ``pairwise_attn_backend``, ...) are accepted and unused."""
        super().__init__()
        self.dtype = dtype
        self.no_update_s, self.no_update_z = True, False
        self.token_z = token_z
        self.triangle_attn_backend = triangle_attn_backend
        self.pair_mask_left_aligned = pair_mask_left_aligned

        def trimul(kind):
            return TriangleMultiplicationNode(layer_idx=layer_idx, dim=token_z, eps=eps, multiplication_type=kind,
                                              dtype=dtype, skip_create_weights=skip_create_weights,
                                              high_precision=trimul_high_precision,
                                              mean_normalization=trimul_mean_normalization,
                                              pair_mask_left_aligned=pair_mask_left_aligned)

        self.tri_mul_out = trimul(TriangleMultiplicationNodeType.OUTGOING)
        self.tri_mul_in = trimul(TriangleMultiplicationNodeType.INCOMING)
        node_kw = dict(inf=inf, layer_idx=layer_idx, dtype=dtype, skip_create_weights=skip_create_weights,
                       attn_backend=triangle_attn_backend, pair_mask_left_aligned=pair_mask_left_aligned)
        self.tri_attn_start = TriangleAttentionStartingNode(token_z, pairwise_head_width, pairwise_num_heads, **node_kw)
        self.tri_attn_end = TriangleAttentionEndingNode(token_z, pairwise_head_width, pairwise_num_heads,
                                                        transposed_bias=tri_attn_transposed_bias, **node_kw)
        self.transition_z = Transition(token_z, token_z * pair_transition_factor, layer_idx=layer_idx, eps=eps,
                                       dtype=dtype, skip_create_weights=skip_create_weights,
                                       auto_chunk_policy=CHUNK_REGISTRY.get(PAIR_TRANSITION))

    def forward(self, z: torch.Tensor, pair_mask: torch.Tensor, trimul_metadata: TriangleMultiplicationMetadata,
                attn_metadatas: dict[str, AttentionMetadata] | None = None,
                precomputed_masks: PrecomputedPairMasks | None = None, precomputed_single_masks=None,
                buffers: PreallocatedBuffers | None = None, inplace_safe: bool = False, **kwargs) -> torch.Tensor:
        can_update_inplace = inplace_safe and not torch.cuda.is_current_stream_capturing()
        z = self.tri_mul_out(z, mask=pair_mask, trimul_metadata=trimul_metadata, residual=True, buffers=buffers)
        z = self.tri_mul_in(z, mask=pair_mask, trimul_metadata=trimul_metadata, residual=True, buffers=buffers)
        if self.dtype is not None:
            z = z.to(self.dtype)
        tri_attn_metadata = (attn_metadatas or {}).get("triangle_attn")
        if precomputed_masks is not None:
            mb_start, mb_end = precomputed_masks.mask_bias, precomputed_masks.mask_bias_transposed
        else:
            mb_start = mb_end = None
        for node, node_mask_bias in ((self.tri_attn_start, mb_start), (self.tri_attn_end, mb_end)):
            z = node(z, mask=pair_mask, mask_bias=node_mask_bias, attn_metadata=tri_attn_metadata, buffers=buffers,
                     residual=True, inplace_residual=can_update_inplace)
        return self.transition_z(z, residual=True, inplace=True)


class PairformerNoSeqModule(nn.Module):
    def __init__(self, num_blocks: int = 8, token_z: int = 128, pairwise_head_width: int = 32,
                 pairwise_num_heads: int = 4, use_cuda_graph: bool = False, **kwargs):
        """``use_cuda_graph`` (not in the reference, whose graph capture lives in its runtime) records one forward
        of the whole stack per (shape, mask object) and replays it; inputs are copied into the graph's buffers."""
        super().__init__()
        self.layers = nn.ModuleList([
            PairformerNoSeqLayer(layer_idx=i, token_z=token_z, pairwise_head_width=pairwise_head_width,
                                 pairwise_num_heads=pairwise_num_heads, **kwargs) for i in range(num_blocks)])
        self.pair_mask_left_aligned = self.layers[0].pair_mask_left_aligned if self.layers else False
        self.use_cuda_graph = use_cuda_graph
        self._graph = None
        self._graph_key = None
        self._graph_in = self._graph_mask = self._graph_out = None

    def _run(self, z, pair_mask, attn_metadatas, buffers, **kwargs):
        first = self.layers[0]
        precomputed = precompute_pair_masks(first.triangle_attn_backend, pair_mask, inf=first.tri_attn_start.inf,
                                            dtype=first.dtype)
        if buffers is None:
            buffers = {}
        int_lengths = precomputed.mask_bias.dtype == torch.int32
        trimul_metadata = precompute_trimul_metadata(
            z, precomputed.mask_bias if int_lengths else None,
            precomputed.mask_bias_transposed if int_lengths else None, enabled=self.pair_mask_left_aligned)
        for layer in self.layers:
            z = layer(z, pair_mask, trimul_metadata, attn_metadatas, precomputed_masks=precomputed, buffers=buffers,
                      **kwargs)
        return z

    def forward(self, z: torch.Tensor, pair_mask: torch.Tensor,
                attn_metadatas: dict[str, AttentionMetadata] | None = None,
                buffers: PreallocatedBuffers | None = None, **kwargs) -> torch.Tensor:
        if not self.layers:
            return z
        if not (self.use_cuda_graph and z.is_cuda) or torch.cuda.is_current_stream_capturing():
            return self._run(z, pair_mask, attn_metadatas, buffers, **kwargs)
        key = (tuple(z.shape), z.dtype, z.device, tuple(pair_mask.shape), pair_mask.dtype)
        if self._graph is None or key != self._graph_key:
            self._graph_in, self._graph_mask = z.clone(), pair_mask.clone()
            graph_buffers: dict = {}
            side = torch.cuda.Stream(z.device)
            side.wait_stream(torch.cuda.current_stream(z.device))
            with torch.cuda.stream(side):
                self._run(self._graph_in, self._graph_mask, attn_metadatas, graph_buffers, **kwargs)  # warm-up, folds
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self._graph_out = self._run(self._graph_in, self._graph_mask, attn_metadatas, graph_buffers, **kwargs)
            torch.cuda.current_stream(z.device).wait_stream(side)
            self._graph, self._graph_key, self._graph_buffers = graph, key, graph_buffers
        self._graph_in.copy_(z)
        self._graph_mask.copy_(pair_mask)
        self._graph.replay()
        return self._graph_out.clone()
