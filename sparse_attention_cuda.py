"""Top-level ``sparse_attention_cuda``: the module name the reference imports.

The reference's bridge binds its CUDA extension by this bare name
(src/layers/ma_core_bridge.py:19-28: ``import sparse_attention_cuda``), and so do
its tests (tests/python/test_cuda_sparse_kernel_launch.py:17,
tests/integration/test_cuda_extensive.py:196-204, tests/python/test_cuda_backward.py:54).
With this directory on ``sys.path`` that import finds this file, and the
reference's unmodified ``src/layers`` runs on libmat_sparse_attn: no edit on the
reference's side.

The four entry points of the extension (src/cuda/sparse_attention_kernel.cu:501-510)
keep their names, positional order, keyword names and defaults.  One addition to
the extension's behaviour: when grad mode is on and an input requires grad, the
returned tensors are marked as requiring grad, so that a caller may differentiate
an expression of the output with respect to the output itself, as
tests/python/test_cuda_backward.py:58-60 does; inside ``autograd.Function.forward``
(the bridge's call site) grad mode is off and nothing changes.
"""
from typing import List

import torch

from ma_transformer_b200 import sparse_attention_cuda as _impl

__all__ = ["forward", "dense_forward", "backward", "dense_backward"]


def _mark(out: torch.Tensor, *inputs: torch.Tensor) -> torch.Tensor:
    if torch.is_grad_enabled() and any(t.requires_grad for t in inputs):
        out.requires_grad_(True)
    return out


def forward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, window_size: int = 64) -> torch.Tensor:
    """Sparse attention forward (CUDA): keys [i-window_size, i+window_size]."""
    return _mark(_impl.forward(query, key, value, window_size), query, key, value)


def dense_forward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                  use_causal_mask: bool = False) -> torch.Tensor:
    """Dense attention forward (CUDA)."""
    return _mark(_impl.dense_forward(query, key, value, use_causal_mask), query, key, value)


def backward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, grad_out: torch.Tensor,
             window_size: int = 64) -> List[torch.Tensor]:
    """Sparse attention backward (CUDA) -> [dQ, dK, dV]."""
    return _impl.backward(query, key, value, grad_out, window_size)


def dense_backward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, grad_out: torch.Tensor,
                   use_causal_mask: bool = False) -> List[torch.Tensor]:
    """Dense attention backward (CUDA) -> [dQ, dK, dV]."""
    return _impl.dense_backward(query, key, value, grad_out, use_causal_mask)
