"""B200-native sparse-attention forward for ma-transformer.

Importing the package loads libmat_sparse_attn.so (hand-written sm_100a
kernels behind a C ABI); it raises if the library has not been built.
"""
from . import _native  # noqa: F401  (fails loudly when the library is missing)
from . import sparse_attention_cuda
from .patterns import (PatternSpec, band_random_block_layout, bigbird_block_layout, estimate_flops,
                       estimate_memory_usage, pattern_flops, pattern_statistics, random_block_layout,
                       tridiagonal_block_layout)
from .layers.ma_core_bridge import (MACoreAttention, MACoreAttentionFunction, create_attention_layer,
                                    pytorch_dense_attention, pytorch_sparse_attention)
from .layers.sparse_attention import SparseAttention

__all__ = [
    "sparse_attention_cuda", "PatternSpec", "band_random_block_layout", "tridiagonal_block_layout",
    "bigbird_block_layout", "random_block_layout", "pattern_statistics", "estimate_flops", "estimate_memory_usage",
    "pattern_flops",
    "MACoreAttention", "MACoreAttentionFunction", "create_attention_layer",
    "pytorch_dense_attention", "pytorch_sparse_attention", "SparseAttention",
]
