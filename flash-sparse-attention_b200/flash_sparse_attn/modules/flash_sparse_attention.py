"""Attention layer around the gated operator: projections -> ``flash_gated_attn_func`` -> output projection.

Same constructor, parameter names (``q_proj k_proj v_proj a_proj d_proj o_proj``, no biases) and return value
as the reference layer (flash_sparse_attn/modules/flash_sparse_attention.py:9-95), so a state dict moves
across unchanged. One difference in how the gate inputs are produced: the kernels read ``alpha`` and
``delta`` as ``[batch, heads, positions]`` rows, and the reference operator makes that layout with a
transpose-and-copy of the ``[batch, positions, heads]`` projections (ops/triton/interface.py:646-648).
Here the two small projections are computed as ``W x^T`` and land in that layout directly; the operator is
handed a transposed view, for which its own ``.contiguous()`` is a no-op, and autograd routes the gradients
back through the same views.
"""

from typing import Optional

import torch
import torch.nn as nn

from flash_sparse_attn.ops.triton.interface import flash_gated_attn_func


class FlashSparseAttentionConfig:
    def __init__(
        self,
        hidden_size: int,
        num_attention_heads: int,
        num_key_value_heads: Optional[int] = None,
        head_dim: Optional[int] = None,
        softmax_threshold: Optional[float] = None,
        gate_threshold: Optional[float] = None,
        max_position_embeddings: int = 32768,
    ):
        self.hidden_size = hidden_size
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads or num_attention_heads
        self.head_dim = head_dim or (hidden_size // num_attention_heads)
        self.softmax_threshold = softmax_threshold
        self.gate_threshold = gate_threshold
        self.max_position_embeddings = max_position_embeddings


class FlashSparseAttention(nn.Module):
    def __init__(self, config: FlashSparseAttentionConfig, layer_idx: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_attention_heads // self.num_key_value_heads
        self.scaling = self.head_dim**-0.5
        self.is_causal = True
        self.softmax_threshold = config.softmax_threshold
        self.gate_threshold = config.gate_threshold

        hidden = config.hidden_size
        self.q_proj = nn.Linear(hidden, self.num_attention_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(hidden, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(hidden, self.num_key_value_heads * self.head_dim, bias=False)
        self.a_proj = nn.Linear(hidden, self.num_attention_heads, bias=False)
        self.d_proj = nn.Linear(hidden, self.num_key_value_heads, bias=False)
        self.o_proj = nn.Linear(self.num_attention_heads * self.head_dim, hidden, bias=False)

    @staticmethod
    def _gate_rows(weight: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        """``[heads, hidden] x [batch, positions, hidden] -> [batch, heads, positions]`` (positions contiguous)."""
        return torch.matmul(weight, hidden_states.transpose(1, 2))

    def forward(self, hidden_states: torch.Tensor, **kwargs):
        bsz, seq_len, _ = hidden_states.size()
        query_states = self.q_proj(hidden_states).view(bsz, seq_len, self.num_attention_heads, self.head_dim)
        key_states = self.k_proj(hidden_states).view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        value_states = self.v_proj(hidden_states).view(bsz, seq_len, self.num_key_value_heads, self.head_dim)
        # [B, H, S] buffers, passed as the [B, S, H] views the operator's signature asks for
        alpha_states = self._gate_rows(self.a_proj.weight, hidden_states).transpose(1, 2)
        delta_states = self._gate_rows(self.d_proj.weight, hidden_states).transpose(1, 2)

        attn_output = flash_gated_attn_func(
            query_states,
            key_states,
            value_states,
            alpha_states,
            delta_states,
            is_causal=self.is_causal,
            softmax_scale=self.scaling,
            softmax_threshold=self.softmax_threshold,
            gate_threshold=self.gate_threshold,
        )
        attn_output = self.o_proj(attn_output.view(bsz, seq_len, -1))
        return attn_output, (key_states, value_states)
