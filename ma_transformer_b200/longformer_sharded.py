"""Longformer (window + global tokens) over a sequence spread across GPUs.

One process per GPU, each owning a contiguous chunk of the sequence.  Besides the
window halo (read in place from the neighbour GPUs by the kernel, as for plain
windows) the pattern needs two small collectives, because a global token is a key
for every row and a query over every key:

  1. all-gather of the Q, K and V rows at the global positions (n_global rows);
  2. every rank computes, for ALL global queries, the partial result over its own
     keys (tcgen05 pass); all-gather of those partials; the rank that owns a global
     token merges its partials and writes that row.

The reference has no distributed path; its single-process pattern is
LongformerAttention (src/csrc/sparse_attention.cpp:234-259).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import _native as nat
from .patterns import LONGFORMER, PatternSpec
from .sharded import PeerHaloAttention, PeerShard

_DT = {torch.bfloat16: nat.MAT_BF16, torch.float16: nat.MAT_F16}


def _stream(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def shard_pass1(q, k, v, left: int, right: int, kg, vg, g_pos: torch.Tensor, prev_kv=None, next_kv=None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Every local row over its window plus the keys at all global positions
    (``mat_longformer_shard_fwd``).  g_pos: int64 device tensor, positions of the
    global tokens relative to this shard's first row."""
    B, S, H, D = q.shape
    if out is None:
        out = torch.empty_like(q)
    ptr = lambda t: t.data_ptr() if t is not None else None
    kp, vp = prev_kv if prev_kv is not None else (None, None)
    kn, vn = next_kv if next_kv is not None else (None, None)
    n_global = int(g_pos.numel())
    with torch.cuda.device(q.device):
        nat.check(nat.lib.mat_longformer_shard_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), ptr(kp), ptr(vp), kp.shape[1] if kp is not None else 0,
            ptr(kn), ptr(vn), kn.shape[1] if kn is not None else 0, ptr(kg) if n_global else None,
            ptr(vg) if n_global else None, g_pos.data_ptr() if n_global else None, n_global, B, S, H, D, _DT[q.dtype],
            int(left), int(right), 0.0, _stream(q)))
    return out


def partial_layout(B: int, n_global: int, s_kv: int, H: int) -> Tuple[int, int, int]:
    """(bytes, key splits, padded rows) of one shard's partial buffer."""
    ns, pad = C.c_int32(0), C.c_int32(0)
    nbytes = nat.lib.mat_global_rows_partial_layout(B, n_global, s_kv, H, C.byref(ns), C.byref(pad))
    return int(nbytes), int(ns.value), int(pad.value)


def global_rows_partial(qg, k, v, partial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Partials of the global queries qg [B, n_global, H, 64] over this shard's keys
    (``mat_global_rows_partial``): float32 [B, H, n_splits, ng_pad, 66]."""
    B, ng, H, D = qg.shape
    nbytes, ns, pad = partial_layout(B, ng, k.shape[1], H)
    if partial is None:
        partial = torch.empty(B, H, ns, pad, 66, dtype=torch.float32, device=qg.device)
    assert partial.numel() * 4 >= nbytes
    with torch.cuda.device(qg.device):
        nat.check(nat.lib.mat_global_rows_partial(qg.data_ptr(), k.data_ptr(), v.data_ptr(), partial.data_ptr(), B, ng,
                                                  k.shape[1], H, D, _DT[qg.dtype], 0.0, _stream(qg)))
    return partial


def global_rows_merge(partials: torch.Tensor, out: torch.Tensor, g_pos: torch.Tensor, e_first: int, n_rows: int) -> None:
    """partials: [n_parts, B, H, n_splits, ng_pad, 66] (one part per shard).  Writes the rows
    of the global tokens [e_first, e_first + n_rows) of ``out`` (``mat_global_rows_merge``)."""
    n_parts, B, H, ns, pad, _ = partials.shape
    with torch.cuda.device(out.device):
        nat.check(nat.lib.mat_global_rows_merge(partials.data_ptr(), n_parts, partials.stride(0), out.data_ptr(),
                                                g_pos.data_ptr(), int(e_first), int(n_rows), B, out.shape[1], H, ns, pad,
                                                _DT[out.dtype], 0.0, _stream(out)))


def _all_gather(t: torch.Tensor, group) -> List[torch.Tensor]:
    """All-gather of equally shaped device tensors (NCCL directly; other backends through the host)."""
    world = dist.get_world_size(group)
    if dist.get_backend(group) == "nccl":
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return parts
    objs = [None] * world
    dist.all_gather_object(objs, t.cpu(), group=group)
    return [o.to(t.device) for o in objs]


class ShardedLongformerAttention:
    """Longformer forward over a sequence cut into ``world`` contiguous chunks."""

    def __init__(self, spec: PatternSpec, seq_len: int, group: Optional[dist.ProcessGroup] = None):
        if spec.kind != LONGFORMER:
            raise ValueError("expected a Longformer pattern")
        self.spec, self.group = spec, group
        self.halo = PeerHaloAttention(PatternSpec(left=spec.left, right=spec.right), seq_len, group)
        self.rank, self.world, self.rows = self.halo.rank, self.halo.world, self.halo.rows
        g = np.asarray(spec.global_idx, dtype=np.int64)
        self.g = g
        self.owner_count = [int(((g >= r * self.rows) & (g < (r + 1) * self.rows)).sum()) for r in range(self.world)]
        self.e_first = int(sum(self.owner_count[:self.rank]))   # my tokens are a contiguous run of the sorted list
        self.n_mine = self.owner_count[self.rank]

    def register(self, k_local: torch.Tensor, v_local: torch.Tensor) -> PeerShard:
        return self.halo.register(k_local, v_local)

    def forward(self, q: torch.Tensor, shard: PeerShard, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        dev, a = q.device, self.rank * self.rows
        B, S, H, D = q.shape
        ng = len(self.g)
        g_pos = torch.from_numpy(self.g - a).to(dev)
        if ng == 0:
            return shard_pass1(q, shard.k, shard.v, self.spec.left, self.spec.right, None, None, g_pos,
                               shard.prev_kv, shard.next_kv, out)
        # 1. the Q/K/V rows at the global positions: each rank contributes the ones it owns
        pad = max(self.owner_count)
        mine = torch.zeros(3, B, pad, H, D, dtype=q.dtype, device=dev)
        if self.n_mine:
            idx = g_pos[self.e_first:self.e_first + self.n_mine]
            mine[0, :, :self.n_mine] = q[:, idx]
            mine[1, :, :self.n_mine] = shard.k[:, idx]
            mine[2, :, :self.n_mine] = shard.v[:, idx]
        parts = _all_gather(mine, self.group)
        qkv_g = torch.cat([p[:, :, :n] for p, n in zip(parts, self.owner_count)], dim=2).contiguous()   # [3, B, ng, H, D]
        qg, kg, vg = qkv_g[0], qkv_g[1], qkv_g[2]
        # 2. every local row: window (halo in place from the neighbours) + the global keys
        out = shard_pass1(q, shard.k, shard.v, self.spec.left, self.spec.right, kg, vg, g_pos,
                          shard.prev_kv, shard.next_kv, out)
        # 3. all global queries over my keys; exchange; the owner merges
        partial = global_rows_partial(qg, shard.k, shard.v)
        partials = torch.stack(_all_gather(partial, self.group))
        global_rows_merge(partials, out, g_pos, self.e_first, self.n_mine)
        return out
