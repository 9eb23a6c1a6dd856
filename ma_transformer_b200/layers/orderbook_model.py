"""Order-book transformer forward: the caller around the sparse-attention hot path
for the order-book configuration (ticks [B, N, 40] -> Linear(40->256) -> 4
pre-LayerNorm blocks with 4 heads of width 64 and dilated causal window attention
(64 taps, dilation 2), GELU feed-forward of width 1024 -> last-token Linear(256->3)).

The block follows the reference's integration example
(examples/pytorch_integration_example.py:21-107: q/k/v/out projections around
``MACoreAttention`` on [batch, seq, heads, head_dim]) and its model skeleton
(src/model.py:55-87: input projection, encoder layers, head on the last token).
The projections are plain library GEMMs.  Q, K and V come out of ONE fused projection
[d_model -> 3*d_model]; its output [B, S, 3, H, 64] is handed to the attention kernel as three
views (token stride 3*H*64), so no split, transpose or copy sits between the projection and the
attention, and the attention output [B, S, H, 64] is already the [B, S, d_model] the output
projection reads.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import sparse_attention_cuda
from ..patterns import PatternSpec
from .ma_core_bridge import MACoreAttention


def synthetic_ticks(batch: int, n: int, levels: int = 10, seed: int = 0, tick: float = 0.01) -> torch.Tensor:
    """Synthetic 10-level order-book ticks [batch, n, 4*levels]: per level bid price,
    ask price, bid size, ask size.  Mid price is a random walk 100 + cumsum(N(0,1)*tick),
    prices sit ``level`` ticks either side of it, sizes are lognormal(mu=4, sigma=1).
    (The reference ships only a 6-column top-of-book generator,
    data/generate_synthetic_ticks.py:7-65.)"""
    g = torch.Generator().manual_seed(seed)
    mid = 100.0 + torch.cumsum(torch.randn(batch, n, generator=g) * tick, dim=1)
    lv = torch.arange(1, levels + 1, dtype=torch.float32) * tick
    bid = mid[..., None] - lv
    ask = mid[..., None] + lv
    sizes = torch.exp(4.0 + torch.randn(batch, n, 2 * levels, generator=g))
    return torch.cat([bid, ask, sizes], dim=-1)


class DilatedAttentionBlock(nn.Module):
    """Pre-LayerNorm transformer block whose attention is the native sparse forward."""

    def __init__(self, d_model: int, n_heads: int, ffn: int, pattern: PatternSpec):
        super().__init__()
        assert d_model % n_heads == 0
        self.n_heads, self.head_dim = n_heads, d_model // n_heads
        self.qkv_proj = nn.Linear(d_model, 3 * d_model)   # rows [0, d) -> Q, [d, 2d) -> K, [2d, 3d) -> V
        self.out_proj = nn.Linear(d_model, d_model)
        self.attention = MACoreAttention(sparse=True, window_size=max(1, pattern.left), pattern=pattern,
                                         fallback_training=False)
        self.norm1 = nn.LayerNorm(d_model)
        self.norm2 = nn.LayerNorm(d_model)
        self.ff1 = nn.Linear(d_model, ffn)
        self.ff2 = nn.Linear(ffn, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, Dm = x.shape
        y = self.norm1(x)
        qkv = self.qkv_proj(y).view(B, S, 3, self.n_heads, self.head_dim)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]      # views: token stride 3 * d_model
        strided_ok = (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and self.head_dim == 64
                      and not (torch.is_grad_enabled() and qkv.requires_grad))
        if strided_ok:   # the kernel reads the three views in place
            a = sparse_attention_cuda.forward_strided(q, k, v, self.attention.pattern)
        else:            # fp32, other head widths, or a graph to differentiate: the module (packed copies)
            a = self.attention(q, k, v)
        x = x + self.out_proj(a.reshape(B, S, Dm))
        return x + self.ff2(F.gelu(self.ff1(self.norm2(x))))


class OrderBookTransformer(nn.Module):
    def __init__(self, n_features: int = 40, d_model: int = 256, n_heads: int = 4, n_layers: int = 4,
                 ffn: int = 1024, taps: int = 64, dilation: int = 2, n_classes: int = 3):
        super().__init__()
        self.pattern = PatternSpec.causal_window(taps, dilation)
        self.embed = nn.Linear(n_features, d_model)
        self.blocks = nn.ModuleList(DilatedAttentionBlock(d_model, n_heads, ffn, self.pattern)
                                    for _ in range(n_layers))
        self.norm = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, n_classes)
        self.d_model = d_model

    def forward(self, ticks: torch.Tensor) -> torch.Tensor:
        """ticks [B, N, n_features] -> imbalance logits [B, n_classes] from the last token."""
        x = self.embed(ticks) * math.sqrt(self.d_model)   # src/model.py:79 scales the embedding
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x[:, -1]))
