"""``SparseAttention`` over [batch, seq_len, model_dim] tensors, the layer of
src/layers/sparse_attention.py:26-110: one head of width model_dim, sliding
window [i-w, i+w], native kernels in eval mode and the differentiable torch path
in training mode (as the reference's fallback_training=True)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .ma_core_bridge import MACoreAttention


class SparseAttention(nn.Module):
    def __init__(self, window_size: int = 3, use_ma_core: bool = True):
        super().__init__()
        if not isinstance(window_size, int):
            raise TypeError("window_size must be an integer for SparseAttention")
        if window_size <= 0:
            raise ValueError("window_size must be > 0 for SparseAttention")
        self.window_size = window_size
        self.use_ma_core = use_ma_core  # kept for signature compatibility; the native path is the only one
        self.ma_core_attention = MACoreAttention(sparse=True, window_size=window_size,
                                                 fallback_training=True)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if q.dim() != 3:
            raise ValueError("Expected tensors with shape [batch, seq_len, model_dim]")
        out = self.ma_core_attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2))
        return out.squeeze(2)
