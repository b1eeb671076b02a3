"""Module-level API: the reference's pair-track layers on the sm_100a kernels."""

from .attention_backend import (AttentionBackend, AttentionMetadata, AttentionType, B200TriangleAttention,
                                PrecomputedPairMasks, PrecomputedSingleMasks, create_attention, get_attention_backend,
                                mask_to_lengths, precompute_pair_masks, precompute_single_masks,
                                register_precompute_pair_masks, register_precompute_single_masks)
from .attention_pair_bias import AttentionPairBias
from .auto_chunk import (CHUNK_REGISTRY, PAIR_TRANSITION, TRIANGLE_ATTENTION, ChunkPolicy, chunk_apply,
                         default_autochunk_min, iter_chunks)
from .buffers import PreallocatedBuffers, ensure_buffer
from .linear import Linear, WeightMode, WeightsLoadingConfig
from .pairformer import (PairformerLayerV1, PairformerLayerV2, PairformerModule, PairformerNoSeqLayer,
                         PairformerNoSeqModule)
from .transition import PairTransition, Transition
from .triangle_multiplication import (TriangleMultiplicationMetadata, TriangleMultiplicationNode,
                                      TriangleMultiplicationNodeType, precompute_trimul_metadata,
                                      set_trimul_token_padding)
from .triangle_nodes import (TriangleAttention, TriangleAttentionEndingNode, TriangleAttentionNode,
                             TriangleAttentionNodeType, TriangleAttentionStartingNode, split_pair_bias_proj)

__all__ = [
    "AttentionBackend", "AttentionMetadata", "AttentionType", "B200TriangleAttention", "PrecomputedPairMasks",
    "create_attention", "get_attention_backend", "mask_to_lengths", "precompute_pair_masks",
    "register_precompute_pair_masks", "CHUNK_REGISTRY", "PAIR_TRANSITION", "TRIANGLE_ATTENTION", "ChunkPolicy",
    "chunk_apply", "default_autochunk_min", "iter_chunks", "PreallocatedBuffers", "ensure_buffer", "Linear",
    "WeightMode", "WeightsLoadingConfig", "Transition", "PairTransition", "TriangleAttention", "TriangleAttentionEndingNode",
    "TriangleAttentionNode", "TriangleAttentionNodeType", "TriangleAttentionStartingNode", "split_pair_bias_proj",
    "TriangleMultiplicationMetadata", "TriangleMultiplicationNode", "TriangleMultiplicationNodeType",
    "precompute_trimul_metadata", "set_trimul_token_padding", "PairformerNoSeqLayer", "PairformerNoSeqModule",
    "AttentionPairBias", "PairformerLayerV1", "PairformerLayerV2", "PairformerModule", "PrecomputedSingleMasks", "precompute_single_masks",
    "register_precompute_single_masks",
]
