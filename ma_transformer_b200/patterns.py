"""Attention-pattern descriptions: which keys each query row attends to.

``PatternSpec`` mirrors the reference's ``AttentionConfig`` / ``AttentionPattern``
vocabulary (src/csrc/attention_types.hpp:26-56: window_size, block_size,
num_global_tokens, use_causal_mask) in the closed form the kernels consume; it
never materialises the COO lists the reference's generators build
(src/csrc/sparse_attention.cpp:181-259, src/csrc/ma_core.cpp:34-48).  The row
sets are available on the host through ``rowset`` / ``nnz`` for checking masks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import _native as nat

WINDOW, BLOCK, LONGFORMER = nat.MAT_WINDOW, nat.MAT_BLOCK, nat.MAT_LONGFORMER


@dataclass
class PatternSpec:
    kind: int = WINDOW
    left: int = 0           # taps before the query (dilation steps)
    right: int = 0          # taps after the query
    dilation: int = 1
    causal: bool = False    # block layouts: drop keys behind the query
    block: int = 0
    blk_rowptr: Optional[np.ndarray] = None   # int32 [n_qblocks+1]
    blk_colidx: Optional[np.ndarray] = None   # int32, distinct within a row
    global_idx: Optional[np.ndarray] = None   # int64, sorted, unique
    q_offset: int = 0       # key-coordinate position of query row 0 (sequence shards)
    _dev: Dict[str, tuple] = field(default_factory=dict, repr=False, compare=False)

    def __post_init__(self) -> None:
        if self.kind not in (WINDOW, BLOCK, LONGFORMER):
            raise ValueError(f"unknown pattern kind {self.kind}")
        if self.left < 0 or self.right < 0:
            raise ValueError("window taps must be >= 0")
        if self.dilation < 1:
            raise ValueError("dilation must be >= 1")
        if self.kind == BLOCK:
            if self.block < 1:
                raise ValueError("block size must be >= 1")
            rp = np.ascontiguousarray(self.blk_rowptr, dtype=np.int32)
            ci = np.ascontiguousarray(self.blk_colidx, dtype=np.int32)
            if rp.ndim != 1 or len(rp) < 1 or rp[0] != 0 or rp[-1] != len(ci) or np.any(np.diff(rp) < 0):
                raise ValueError("malformed block-CSR row pointers")
            for r in range(len(rp) - 1):
                row = ci[rp[r]:rp[r + 1]]
                if len(np.unique(row)) != len(row) or np.any(row < 0):
                    raise ValueError(f"block row {r}: column ids must be distinct and >= 0")
                ci[rp[r]:rp[r + 1]] = np.sort(row)   # the library wants them ascending within a row
            self.blk_rowptr, self.blk_colidx = rp, ci
        if self.kind == LONGFORMER:
            g = np.unique(np.asarray(self.global_idx if self.global_idx is not None else [], dtype=np.int64))
            if np.any(g < 0):
                raise ValueError("global positions must be >= 0")
            self.global_idx = g

    # ---- constructors ------------------------------------------------------
    @staticmethod
    def sliding_window(window_size: int) -> "PatternSpec":
        """The reference's key set [i-w, i+w] (src/csrc/ma_core.cpp:197-198)."""
        return PatternSpec(WINDOW, left=int(window_size), right=int(window_size))

    @staticmethod
    def causal_window(taps: int, dilation: int = 1) -> "PatternSpec":
        """``taps`` keys ending at the query: i-(taps-1)*dil, ..., i-dil, i."""
        if taps < 1:
            raise ValueError("taps must be >= 1")
        return PatternSpec(WINDOW, left=int(taps) - 1, right=0, dilation=int(dilation))

    @staticmethod
    def dilated_window(window_size: int, dilation: int) -> "PatternSpec":
        """Two-sided dilated set { i - t*d : t in [-w, w] }
        (doc/sparse_attention_whitepaper.md:102-105)."""
        return PatternSpec(WINDOW, left=int(window_size), right=int(window_size), dilation=int(dilation))

    @staticmethod
    def block_sparse(block: int, rowptr: Sequence[int], colidx: Sequence[int],
                     causal: bool = False) -> "PatternSpec":
        return PatternSpec(BLOCK, block=int(block), causal=bool(causal),
                           blk_rowptr=np.asarray(rowptr), blk_colidx=np.asarray(colidx))

    @staticmethod
    def longformer(left: int, right: int, global_idx: Sequence[int]) -> "PatternSpec":
        return PatternSpec(LONGFORMER, left=int(left), right=int(right),
                           global_idx=np.asarray(global_idx, dtype=np.int64))

    def shifted(self, q_offset: int) -> "PatternSpec":
        """Same pattern for a shard whose first query sits at key row ``q_offset``."""
        return PatternSpec(self.kind, self.left, self.right, self.dilation, self.causal, self.block,
                           self.blk_rowptr, self.blk_colidx, self.global_idx, int(q_offset))

    def check_against(self, s_kv: int) -> None:
        """Raises RuntimeError when the pattern names a key position outside ``[0, s_kv)``.

        The library reads the global positions on the device, where it cannot refuse them; a
        position past the sequence would name memory that is not the caller's.  (Block column ids
        past the sequence are harmless: their keys are simply absent.)"""
        if self.kind == LONGFORMER and self.global_idx is not None and len(self.global_idx):
            if int(self.global_idx[-1]) >= int(s_kv) or int(self.global_idx[0]) < 0:
                raise RuntimeError(f"global position {int(self.global_idx[-1])} lies outside the sequence of "
                                   f"{int(s_kv)} keys: global positions must be in [0, S)")

    # ---- C structs -----------------------------------------------------------
    def _fill(self, s: nat.MatPatternSpec) -> None:
        s.kind, s.causal = int(self.kind), int(bool(self.causal))
        s.left, s.right, s.dilation = int(self.left), int(self.right), int(self.dilation)
        s.block, s.q_offset = int(self.block), int(self.q_offset)
        s.n_qblocks = len(self.blk_rowptr) - 1 if self.blk_rowptr is not None else 0
        s.n_global = len(self.global_idx) if self.global_idx is not None else 0

    def host_struct(self) -> nat.MatPatternSpec:
        s = nat.MatPatternSpec()
        self._fill(s)
        if self.blk_rowptr is not None:
            s.blk_rowptr = self.blk_rowptr.ctypes.data
            s.blk_colidx = self.blk_colidx.ctypes.data
        if self.global_idx is not None and len(self.global_idx):
            s.global_idx = self.global_idx.ctypes.data
        return s

    def device_struct(self, device) -> nat.MatPatternSpec:
        """Struct whose index arrays live on ``device`` (uploaded once, cached)."""
        import torch
        key = str(torch.device(device))
        if key not in self._dev:
            rp = ci = g = None
            if self.blk_rowptr is not None:
                rp = torch.from_numpy(self.blk_rowptr).to(device)
                ci = torch.from_numpy(self.blk_colidx).to(device) if len(self.blk_colidx) else \
                    torch.zeros(1, dtype=torch.int32, device=device)
            if self.global_idx is not None and len(self.global_idx):
                g = torch.from_numpy(self.global_idx).to(device)
            self._dev[key] = (rp, ci, g)
        rp, ci, g = self._dev[key]
        s = nat.MatPatternSpec()
        self._fill(s)
        if rp is not None:
            s.blk_rowptr, s.blk_colidx = rp.data_ptr(), ci.data_ptr()
        if g is not None:
            s.global_idx = g.data_ptr()
        return s

    def transposed_layout(self):
        """Block layouts: (rowptr, colidx) of the transposed layout as int32 numpy arrays: for every key
        block the ascending query blocks whose layout row holds it (what the backward's dK / dV pass walks)."""
        if self.kind != BLOCK:
            raise ValueError("only block layouts have a transposed layout")
        n = len(self.blk_rowptr) - 1
        rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(self.blk_rowptr))
        cols = self.blk_colidx.astype(np.int64)
        if len(cols) and int(cols.max()) >= n:
            raise ValueError("the backward needs a square layout (key blocks within the sequence)")
        order = np.lexsort((rows, cols))
        t_colidx = rows[order].astype(np.int32)
        t_rowptr = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(np.bincount(cols, minlength=n), out=t_rowptr[1:])
        return t_rowptr, t_colidx

    def device_transposed_layout(self, device):
        """The transposed layout on ``device`` (uploaded once, cached) as two int32 tensors."""
        import torch
        key = "T" + str(torch.device(device))
        if key not in self._dev:
            rp, ci = self.transposed_layout()
            self._dev[key] = (torch.from_numpy(rp).to(device),
                              torch.from_numpy(ci).to(device) if len(ci) else torch.zeros(1, dtype=torch.int32, device=device))
        return self._dev[key]

    # ---- host index sets -------------------------------------------------------
    def rowset(self, s_kv: int, i: int) -> np.ndarray:
        """Sorted unique key positions of query row ``i`` (int64)."""
        s = self.host_struct()
        n = C.c_int64(0)
        cap = int(s_kv)
        out = np.empty(max(cap, 1), dtype=np.int64)
        nat.check(nat.lib.mat_pattern_rowset(C.byref(s), s_kv, i, out.ctypes.data, cap, C.byref(n)))
        return out[:n.value].copy()

    def nnz(self, s_q: int, s_kv: Optional[int] = None) -> int:
        s = self.host_struct()
        n = C.c_int64(0)
        nat.check(nat.lib.mat_pattern_nnz(C.byref(s), s_q, s_kv if s_kv is not None else s_q, C.byref(n)))
        return int(n.value)


# ---- block layouts -------------------------------------------------------------

def tridiagonal_block_layout(seq_len: int, block: int) -> Tuple[np.ndarray, np.ndarray]:
    """The reference's block-sparse layout: block row r holds columns r-1, r, r+1
    (src/csrc/sparse_attention.cpp:212-227)."""
    nb = (seq_len + block - 1) // block
    rowptr, colidx = [0], []
    for r in range(nb):
        colidx += [c for c in (r - 1, r, r + 1) if 0 <= c < nb]
        rowptr.append(len(colidx))
    return np.asarray(rowptr, np.int32), np.asarray(colidx, np.int32)


def band_random_block_layout(n_blocks: int, band: int = 4, n_random: int = 2,
                             seed: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """Causal local band plus random earlier blocks: block row r holds columns
    max(0, r-band+1)..r and ``n_random`` columns drawn without replacement from
    the blocks before the band (fewer when fewer exist), columns sorted."""
    rng = np.random.default_rng(seed)
    rowptr, colidx = [0], []
    for r in range(n_blocks):
        lo = max(0, r - band + 1)
        cols = list(range(lo, r + 1))
        if lo > 0 and n_random > 0:
            cols += sorted(rng.choice(lo, size=min(n_random, lo), replace=False).tolist())
        colidx += sorted(cols)
        rowptr.append(len(colidx))
    return np.asarray(rowptr, np.int32), np.asarray(colidx, np.int32)


def bigbird_block_layout(n_blocks: int, window_blocks: int = 3, n_global_blocks: int = 1,
                         n_random_blocks: int = 3, seed: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """BIG_BIRD of the reference's vocabulary (``AttentionPattern::BIG_BIRD`` with
    ``num_global_tokens`` / ``num_random_blocks``, src/csrc/attention_types.hpp:26-56; the
    reference's factory throws on it, src/csrc/attention_factory.cpp:25-28) as a block layout:
    block row r holds a centred band of ``window_blocks`` columns, the first
    ``n_global_blocks`` columns, ``n_random_blocks`` further columns drawn without replacement
    by a seeded generator; the first ``n_global_blocks`` rows hold every column."""
    rng = np.random.default_rng(seed)
    half = window_blocks // 2
    rowptr, colidx = [0], []
    for r in range(n_blocks):
        if r < n_global_blocks:
            cols = set(range(n_blocks))
        else:
            cols = {c for c in range(r - half, r + half + 1) if 0 <= c < n_blocks}
            cols |= set(range(min(n_global_blocks, n_blocks)))
            rest = np.asarray([c for c in range(n_blocks) if c not in cols], dtype=np.int64)
            if n_random_blocks > 0 and rest.size:
                cols |= set(rng.choice(rest, size=min(n_random_blocks, rest.size), replace=False).tolist())
        colidx += sorted(cols)
        rowptr.append(len(colidx))
    return np.asarray(rowptr, np.int32), np.asarray(colidx, np.int32)


def random_block_layout(n_blocks: int, density: float, seed: int = 0,
                        keep_diagonal: bool = True) -> Tuple[np.ndarray, np.ndarray]:
    """RANDOM_SPARSE at block granularity: about ``density`` of the block columns of every row,
    drawn by a seeded generator (the reference draws single (i, j) pairs from an unseeded
    ``std::random_device``, src/csrc/sparse_attention.cpp:286-308, which no test can pin and no
    tiled kernel can use); the diagonal block is kept so that no row is empty."""
    if not 0.0 <= density <= 1.0:
        raise ValueError(f"density must be in [0, 1], got {density}")
    rng = np.random.default_rng(seed)
    per_row = min(n_blocks, max(1 if keep_diagonal else 0, int(round(density * n_blocks))))
    rowptr, colidx = [0], []
    for r in range(n_blocks):
        cols = set(rng.choice(n_blocks, size=per_row, replace=False).tolist())
        if keep_diagonal and r not in cols:
            if len(cols) >= per_row and cols:
                cols.pop()
            cols.add(r)
        colidx += sorted(cols)
        rowptr.append(len(colidx))
    return np.asarray(rowptr, np.int32), np.asarray(colidx, np.int32)


# ---- statistics and estimates ------------------------------------------------------

def pattern_statistics(spec: PatternSpec, seq_len: int) -> str:
    """The text of the reference's ``get_pattern_statistics`` (src/csrc/ma_core.cpp:50-63) for any
    pattern, from the closed form (no COO list is built)."""
    total = int(seq_len) * int(seq_len)
    nnz = spec.nnz(seq_len)
    sparsity = np.float32(1.0) - np.float32(nnz) / np.float32(total) if total else np.float32(0.0)
    return ("Pattern Statistics:\n"
            f"  Total elements: {total}\n"
            f"  Non-zero elements: {nnz}\n"
            f"  Sparsity ratio: {float(sparsity * np.float32(100.0)):.6f}%\n")


def estimate_flops(pattern: str, batch: int, seq_len: int, heads: int, head_dim: int,
                   window_size: int = 64, block_size: int = 64) -> int:
    """``attention_utils::estimate_flops`` (src/csrc/sparse_attention.cpp:312-334), same
    conventions: one matmul counted, ``window_size`` keys per row for a sliding window, three
    blocks per block row for a block-sparse layout, the conservative S*S*D elsewhere."""
    p = pattern.upper()
    if p in ("FULL", "CAUSAL"):
        return batch * heads * seq_len * seq_len * head_dim * 2
    if p == "SLIDING_WINDOW":
        return batch * heads * seq_len * window_size * head_dim * 2
    if p == "BLOCK_SPARSE":
        nb = (seq_len + block_size - 1) // block_size
        return batch * heads * nb * 3 * block_size * block_size * head_dim
    return batch * heads * seq_len * seq_len * head_dim


def estimate_memory_usage(pattern: str, batch: int, seq_len: int, heads: int,
                          window_size: int = 64, block_size: int = 64) -> int:
    """``attention_utils::estimate_memory_usage`` (src/csrc/sparse_attention.cpp:336-357): elements
    of the score and weight arrays the reference's class path would hold (this library holds none
    of them: scores live in registers or TMEM)."""
    p = pattern.upper()
    if p in ("FULL", "CAUSAL"):
        return batch * heads * seq_len * seq_len * 2
    if p == "SLIDING_WINDOW":
        return batch * heads * seq_len * window_size * 2
    if p == "BLOCK_SPARSE":
        nb = (seq_len + block_size - 1) // block_size
        return batch * heads * nb * 3 * block_size * block_size
    return batch * heads * seq_len * seq_len


def pattern_flops(spec: PatternSpec, batch: int, seq_len: int, heads: int, head_dim: int) -> int:
    """FLOPs the forward actually needs for a pattern: two products of 2*D per (query, key) pair."""
    return 4 * batch * heads * head_dim * spec.nnz(seq_len)
