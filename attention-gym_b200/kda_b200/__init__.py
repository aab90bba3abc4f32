"""kda_b200: the KDA (Kimi Delta Attention) gated delta-rule path of attn_gym.linear on B200.

Same public names as ``attn_gym.linear`` / ``attn_gym.linear.kda`` for this path
(attn_gym/linear/__init__.py:37-56, attn_gym/linear/kda/__init__.py:15-57); the fused
implementations call hand-written sm_100a CUDA kernels through the C ABI in include/kda_b200.h.
"""

from .api import chunk_kda, recurrent_kda
from .chunk_schedule import (RaggedChunkMetadata, chunk_capacity,
                             prepare_ragged_chunk_metadata)
from .masking import active_token_mask, mask_inactive_token_gradients, mask_inactive_tokens
from .decode import decode_step
from .layer import KDAAttention, KDAAttentionOutput
from .preops import (bounded_gate_cumsum, causal_conv1d, causal_conv1d_decode, gated_output_norm,
                     l2norm)
from .types import Impl

__all__ = [
    "Impl", "KDAAttention", "KDAAttentionOutput", "RaggedChunkMetadata", "active_token_mask", "bounded_gate_cumsum", "causal_conv1d",
    "causal_conv1d_decode", "chunk_capacity", "chunk_kda", "decode_step", "gated_output_norm",
    "l2norm",
    "mask_inactive_token_gradients", "mask_inactive_tokens", "prepare_ragged_chunk_metadata",
    "recurrent_kda",
]
