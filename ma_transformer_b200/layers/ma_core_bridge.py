"""The reference's PyTorch bridge (src/layers/ma_core_bridge.py) with the same
public names, signatures, validation and error behaviour, served by the sm_100a
library instead of the CPU engine / fp32-only CUDA extension.

What changes behind the unchanged surface:
  * CUDA tensors of fp32, bf16 and fp16 all take the native kernels (the
    reference sends non-fp32 to a python loop, ma_core_bridge.py:77-79);
  * CPU tensors are computed on the GPU through the host-buffer entry point
    (copy in, compute, copy out) instead of the single-threaded C++ engine
    (ma_core_bridge.py:102-112).  There is no CPU compute path: without a GPU the
    call raises.
  * ``MACoreAttention`` takes one additive keyword, ``pattern``, to select a
    causal / dilated / block-sparse / Longformer key set.
  * CUDA tensors take the native forward AND backward kernels in training mode
    too (the reference's ``fallback_training`` python path remains for host
    tensors only).
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from .. import sparse_attention_cuda
from ..patterns import PatternSpec

_HAS_SPARSE_CUDA = True  # the extension is this package's own library; import fails if absent


def pytorch_sparse_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                             window_size: int = 64) -> torch.Tensor:
    """Differentiable torch implementation of sliding-window attention with keys
    [i-window_size, i+window_size]: the reference's test oracle and training
    path (ma_core_bridge.py:224-247; the query is scaled before the dot, :238).
    Vectorised over rows (banded gather) instead of the reference's python loops."""
    B, S, H, D = query.shape
    w = int(window_size)
    scale = 1.0 / (D ** 0.5)
    q = query * scale
    if 2 * w + 1 >= S:  # the band covers (nearly) everything: masked dense scores
        scores = torch.einsum("bihd,bjhd->bhij", q, key)
        i = torch.arange(S, device=query.device)
        band = (i[None, :] - i[:, None]).abs() <= w
        scores = scores.masked_fill(~band, float("-inf"))
        return torch.einsum("bhij,bjhd->bihd", torch.softmax(scores, dim=-1), value)
    offs = torch.arange(-w, w + 1, device=query.device)
    idx = torch.arange(S, device=query.device)[:, None] + offs[None, :]   # [S, 2w+1]
    valid = (idx >= 0) & (idx < S)
    idx = idx.clamp(0, S - 1)
    kw = key[:, idx]      # [B, S, W, H, D]
    vw = value[:, idx]
    scores = torch.einsum("bshd,bswhd->bshw", q, kw)
    scores = scores.masked_fill(~valid[None, :, None, :], float("-inf"))
    return torch.einsum("bshw,bswhd->bshd", torch.softmax(scores, dim=-1), vw)


def pytorch_dense_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                            use_causal_mask: bool = False) -> torch.Tensor:
    """Torch implementation of dense attention (ma_core_bridge.py:184-221):
    scaled query, optional causal mask filled with -1e9, softmax, P*V."""
    B, S, H, D = query.shape
    scores = torch.einsum("bihd,bjhd->bhij", query * (1.0 / (D ** 0.5)), key)
    if use_causal_mask:
        keep = torch.tril(torch.ones(S, S, device=query.device, dtype=torch.bool))
        scores = scores.masked_fill(~keep, -1e9)
    return torch.einsum("bhij,bjhd->bihd", torch.softmax(scores, dim=-1), value).contiguous()


class HostTensor:
    """Contiguous host array in [batch, seq, heads, dim] order: what the reference
    hands to its CPU engine as ``ma_core.Tensor`` (src/csrc/main.cpp:58-90)."""

    def __init__(self, array: np.ndarray):
        if array.ndim != 4:
            raise RuntimeError("Shape must have 4 dimensions: [batch, seq, heads, dim]")
        self._a = np.ascontiguousarray(array)

    def shape(self) -> Tuple[int, ...]:
        return tuple(self._a.shape)

    def size(self) -> int:
        return int(self._a.size)

    def nbytes(self) -> int:
        return int(self._a.nbytes)

    def to_numpy(self) -> np.ndarray:
        return self._a


def pytorch_to_ma_core(tensor: torch.Tensor) -> HostTensor:
    """Detach, move to the host, make contiguous (ma_core_bridge.py:157-168)."""
    t = tensor.detach().cpu().contiguous()
    return HostTensor(t.float().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.numpy())


def ma_core_to_pytorch(mc_tensor: HostTensor, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Back to a torch tensor of the given device and dtype (ma_core_bridge.py:171-181)."""
    out = torch.from_numpy(mc_tensor.to_numpy())
    if out.dtype != dtype:
        out = out.to(dtype)
    return out.to(device) if torch.device(device).type != "cpu" else out


def _native_forward(query, key, value, sparse, window_size, use_causal_mask, pattern):
    if query.is_cuda and key.is_cuda and value.is_cuda:
        cq, ck, cv = query.contiguous(), key.contiguous(), value.contiguous()
        if pattern is not None:
            return sparse_attention_cuda.forward_pattern(cq, ck, cv, pattern)
        if sparse:
            return sparse_attention_cuda.forward(cq, ck, cv, int(window_size))
        return sparse_attention_cuda.dense_forward(cq, ck, cv, bool(use_causal_mask))
    if query.is_cuda or key.is_cuda or value.is_cuda:
        raise RuntimeError("query, key and value must live on the same device")
    if not torch.cuda.is_available():
        raise RuntimeError("this build computes on a B200 only: no GPU is visible and there is no CPU fallback")
    S = query.shape[1]
    spec = pattern
    if spec is None:
        spec = PatternSpec.sliding_window(int(window_size)) if sparse else \
            PatternSpec(left=S, right=0 if use_causal_mask else S)
    dt = query.dtype
    work = dt if dt in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
    out = sparse_attention_cuda.forward_host(query.detach().to(work).contiguous(),
                                             key.detach().to(work).contiguous(),
                                             value.detach().to(work).contiguous(), spec)
    return out.to(dt)


class MACoreAttentionFunction(torch.autograd.Function):
    """Autograd function around the native forward (ma_core_bridge.py:44-154)."""

    @staticmethod
    def forward(ctx, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                sparse: bool = False, window_size: int = 64,
                use_causal_mask: bool = False, pattern: Optional[PatternSpec] = None) -> torch.Tensor:
        ctx.save_for_backward(query, key, value)
        ctx.sparse, ctx.window_size, ctx.use_causal_mask = sparse, window_size, use_causal_mask
        ctx.pattern = pattern
        return _native_forward(query, key, value, sparse, window_size, use_causal_mask, pattern)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        query, key, value = ctx.saved_tensors
        if query.is_cuda:
            args = (query.contiguous(), key.contiguous(), value.contiguous(), grad_output.contiguous())
            if ctx.pattern is not None:
                dq, dk, dv = sparse_attention_cuda.backward_pattern(*args, ctx.pattern)
            elif ctx.sparse:
                dq, dk, dv = sparse_attention_cuda.backward(*args, int(ctx.window_size))
            else:
                dq, dk, dv = sparse_attention_cuda.dense_backward(*args, bool(ctx.use_causal_mask))
        else:
            # host tensors: the gradients are computed on the GPU by the same kernels (copy in, run, copy
            # back), as the forward was; there is no CPU arithmetic here
            if not torch.cuda.is_available():
                raise RuntimeError("this build computes on a B200 only: no GPU is visible and there is no CPU fallback")
            dt = query.dtype
            work = dt if dt in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
            args = tuple(t.detach().to("cuda", work).contiguous() for t in (query, key, value, grad_output))
            if ctx.pattern is not None:
                grads = sparse_attention_cuda.backward_pattern(*args, ctx.pattern)
            elif ctx.sparse:
                grads = sparse_attention_cuda.backward(*args, int(ctx.window_size))
            else:
                grads = sparse_attention_cuda.dense_backward(*args, bool(ctx.use_causal_mask))
            dq, dk, dv = (g.to("cpu", dt) for g in grads)
        need = ctx.needs_input_grad
        return (dq if need[0] else None, dk if need[1] else None, dv if need[2] else None,
                None, None, None, None)


class MACoreAttention(nn.Module):
    """Attention over [batch, seq_len, num_heads, head_dim] tensors; constructor
    arguments, checks and messages follow ma_core_bridge.py:250-330."""

    def __init__(self, sparse: bool = False, window_size: int = 64, use_causal_mask: bool = False,
                 fallback_training: bool = True, pattern: Optional[PatternSpec] = None):
        super().__init__()
        self.sparse = sparse
        if self.sparse:
            if not isinstance(window_size, int):
                raise TypeError("window_size must be an integer for sparse attention")
            if window_size <= 0:
                raise ValueError("window_size must be > 0 for sparse attention")
        self.window_size = window_size
        self.use_causal_mask = use_causal_mask
        self.fallback_training = fallback_training
        self.pattern = pattern

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
        if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
            raise ValueError("Expected tensors with shape [batch, seq_len, num_heads, head_dim]")
        # seq_len and num_heads swapped in Q/K relative to V: put them back (ma_core_bridge.py:300-304)
        if (query.shape[0] == value.shape[0] and query.shape[1] == value.shape[2]
                and query.shape[2] == value.shape[1] and query.shape[3] == value.shape[3]
                and key.shape == query.shape):
            query = query.transpose(1, 2).contiguous()
            key = key.transpose(1, 2).contiguous()
        if query.shape != key.shape or key.shape != value.shape:
            raise ValueError("Tensor size mismatch: query, key, and value must have identical shapes "
                             "[batch, sequence length, num_heads, head_dim]")
        b, s, h, d = query.shape
        if b <= 0 or s <= 0 or h <= 0 or d <= 0:
            raise ValueError("All tensor dimensions must be > 0")
        if self.sparse and self.window_size <= 0:
            raise ValueError("window_size must be > 0 for sparse attention")

        # Training mode.  The reference returns its differentiable python implementation here
        # (ma_core_bridge.py:317-325) because its extension's backward was an afterthought.  This library
        # has native backward kernels, so CUDA tensors always take the native forward and backward,
        # training or not.  Host tensors in training mode keep the reference's behaviour (its torch
        # implementation, whose graph supports double backward): that is the reference's own host-side
        # training path, not a substitute for a kernel.
        if (self.training and self.fallback_training and self.pattern is None
                and not (query.is_cuda and key.is_cuda and value.is_cuda)):
            for t in (query, key, value):
                if t.requires_grad and t.grad_fn is not None:
                    t.retain_grad()
            if self.sparse:
                return pytorch_sparse_attention(query, key, value, self.window_size)
            return pytorch_dense_attention(query, key, value, self.use_causal_mask)

        return MACoreAttentionFunction.apply(query, key, value, self.sparse, self.window_size,
                                             self.use_causal_mask, self.pattern)


def create_attention_layer(attention_type: str = "dense", **kwargs) -> nn.Module:
    """Factory of ma_core_bridge.py:333-352: "dense", "sparse" or "auto" (= sparse)."""
    if attention_type == "dense":
        return MACoreAttention(sparse=False, **kwargs)
    if attention_type in ("sparse", "auto"):
        return MACoreAttention(sparse=True, **kwargs)
    raise ValueError(f"Unknown attention type: {attention_type}")
