"""Sequence-sharded forward: one process per GPU, each owning a contiguous chunk
of the sequence.  Two ways to get the K/V halo rows a chunk's windows reach:

``PeerHaloAttention``         no exchange step: every rank keeps only its own chunk
                              and the attention kernel's edge tiles read the
                              neighbour's rows in place over NVLink (the default on GPUs).
``SequenceShardedAttention``  the halo rows are exchanged between neighbours by
                              send/recv (NCCL on GPUs, gloo on CPU in the tests)
                              into an extended K/V buffer.  Described first, below.

The reference has no distributed path at all; this is the one parallel strategy
the long-sequence configuration needs.  Window patterns only need the
``left*dilation`` key rows before the chunk and the ``right*dilation`` rows after
it, so the collective is a neighbour exchange and nothing else:

  rank r-1  ... | chunk r-1 ]──last `halo_left` rows──▶[ halo | chunk r | halo ]◀──first `halo_right` rows──[ chunk r+1 | ...

Each rank keeps K and V resident in an *extended* buffer
``[B, halo_left + chunk + halo_right, H, D]`` (the first rank has no front halo,
the last no back halo); the exchange receives straight into the halo rows, so the
kernel sees one dense tensor and ``PatternSpec.q_offset`` tells it where the
chunk's first query sits.  Queries whose windows stay inside the chunk do not
wait for the exchange: they are launched first, the edge rows after the receive.

(batch, head) pairs are independent, so block-sparse and Longformer layouts
shard over those instead (``shard_batch_heads``) and need no exchange.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .patterns import PatternSpec, WINDOW


@dataclass
class ShardLayout:
    """Where one rank's rows sit in the global sequence and in its extended K/V buffer."""
    rank: int
    world: int
    seq_len: int       # global sequence length
    start: int         # first global row of the chunk
    rows: int          # rows in the chunk
    halo_front: int    # halo rows stored before the chunk (0 on the first rank)
    halo_back: int     # halo rows stored after the chunk (0 on the last rank)

    @property
    def kv_rows(self) -> int:
        return self.halo_front + self.rows + self.halo_back


def front_halo_rows(spec: PatternSpec) -> int:
    """Key rows a shard keeps in front of its chunk: the window's reach
    ``left*dilation`` rounded up to a multiple of ``16*dilation``, so the chunk's
    first query stays aligned to the kernels' 16-key column pairs (63 -> 64)."""
    unit = 16 * spec.dilation
    return -(-(spec.left * spec.dilation) // unit) * unit


def shard_layout(spec: PatternSpec, seq_len: int, rank: int, world: int) -> ShardLayout:
    if spec.kind != WINDOW:
        raise ValueError("sequence sharding applies to window patterns; shard (batch, head) pairs for the others")
    if seq_len % world:
        raise ValueError(f"sequence length {seq_len} is not divisible by {world} ranks")
    rows = seq_len // world
    reach_l, reach_r = front_halo_rows(spec), spec.right * spec.dilation
    if max(reach_l, reach_r) > rows:
        raise ValueError("window reaches past the neighbouring chunk: use fewer ranks")
    if rows % spec.dilation:
        raise ValueError("chunk length must be a multiple of the dilation")
    return ShardLayout(rank, world, seq_len, rank * rows, rows,
                       reach_l if rank > 0 else 0, reach_r if rank < world - 1 else 0)


def shard_batch_heads(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of the (batch*head) units rank ``rank`` owns; no communication needed."""
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class SequenceShardedAttention:
    """Forward of a window pattern over a sequence cut into ``world`` contiguous chunks.

    ``forward_fn(q, k_ext, v_ext, spec, out=...)`` computes one shard into ``out``;
    it defaults to the native ``sparse_attention_cuda.forward_pattern``.
    """

    def __init__(self, spec: PatternSpec, seq_len: int, group: Optional[dist.ProcessGroup] = None,
                 forward_fn: Optional[Callable] = None, overlap: bool = True):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.spec = spec
        self.layout = shard_layout(spec, seq_len, self.rank, self.world)
        self.local_spec = spec.shifted(self.layout.halo_front)
        if forward_fn is None:
            from . import sparse_attention_cuda
            forward_fn = sparse_attention_cuda.forward_pattern
        self.forward_fn = forward_fn
        self.overlap = overlap

    # ---- buffers -----------------------------------------------------------
    def alloc_kv(self, B: int, H: int, D: int, dtype, device) -> torch.Tensor:
        """Extended K (or V) buffer; write the chunk's rows through ``chunk_view``."""
        return torch.zeros(B, self.layout.kv_rows, H, D, dtype=dtype, device=device)

    def chunk_view(self, ext: torch.Tensor) -> torch.Tensor:
        L = self.layout
        return ext[:, L.halo_front:L.halo_front + L.rows]

    # ---- halo exchange -----------------------------------------------------
    def _p2p_ops(self, k_ext: torch.Tensor, v_ext: torch.Tensor):
        """send/recv pairs for both tensors; returns (ops, copies_after_recv)."""
        L, spec = self.layout, self.spec
        reach_l, reach_r = front_halo_rows(spec), spec.right * spec.dilation
        ops, after = [], []
        peer = lambda r: r if self.group is None else dist.get_global_rank(self.group, r)

        def send(t: torch.Tensor, dst: int):
            ops.append(dist.P2POp(dist.isend, t if t.is_contiguous() else t.contiguous(), peer(dst), self.group))

        def recv(view: torch.Tensor, src: int):
            if view.is_contiguous():
                ops.append(dist.P2POp(dist.irecv, view, peer(src), self.group))
            else:  # B > 1: the halo rows of the batch items are not adjacent
                tmp = torch.empty(view.shape, dtype=view.dtype, device=view.device)
                ops.append(dist.P2POp(dist.irecv, tmp, peer(src), self.group))
                after.append((view, tmp))

        for ext in (k_ext, v_ext):
            c0 = L.halo_front
            if self.rank < self.world - 1 and reach_l:      # my last rows are the next rank's front halo
                send(ext[:, c0 + L.rows - reach_l:c0 + L.rows], self.rank + 1)
            if self.rank > 0 and reach_r:                   # my first rows are the previous rank's back halo
                send(ext[:, c0:c0 + reach_r], self.rank - 1)
            if L.halo_front:
                recv(ext[:, :L.halo_front], self.rank - 1)
            if L.halo_back:
                recv(ext[:, c0 + L.rows:], self.rank + 1)
        return ops, after

    def exchange_halos(self, k_ext: torch.Tensor, v_ext: torch.Tensor):
        """Starts the neighbour exchange; returns a callable that completes it."""
        ops, after = self._p2p_ops(k_ext, v_ext)
        works = dist.batch_isend_irecv(ops) if ops else []

        def finish():
            for w in works:
                w.wait()
            for view, tmp in after:
                view.copy_(tmp)
        return finish

    # ---- forward -------------------------------------------------------------
    def edge_rows(self) -> Tuple[int, int]:
        """Rows at the front / back of the chunk whose windows reach into a halo,
        rounded up to whole query tiles."""
        L, spec = self.layout, self.spec
        unit = 64 * spec.dilation
        up = lambda x: min(L.rows, -(-x // unit) * unit) if x else 0
        return up(L.halo_front), up(L.halo_back)

    def forward(self, q: torch.Tensor, k_ext: torch.Tensor, v_ext: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q: this rank's [B, rows, H, D]; k_ext / v_ext: extended buffers holding
        the chunk's own rows.  Exchanges halos, then computes the chunk."""
        L = self.layout
        if q.shape[1] != L.rows or k_ext.shape[1] != L.kv_rows:
            raise ValueError("tensor lengths do not match this rank's shard layout")
        if out is None:
            out = torch.empty_like(q)
        finish = self.exchange_halos(k_ext, v_ext)
        front, back = self.edge_rows()
        if not self.overlap or q.shape[0] != 1 or front + back >= L.rows:
            finish()
            self._run(q, k_ext, v_ext, out, 0, L.rows)
            return out
        # interior rows first: their windows never leave the chunk.  They are handed the chunk's own key rows
        # only: the tiled kernels stage whole groups of keys around a window, and a halo row that has not been
        # received yet (arbitrary bits, possibly NaN) must not sit in such a group, not even under a zero weight.
        self._run(q, k_ext, v_ext, out, front, L.rows - back, own_rows_only=True)
        finish()
        if front:
            self._run(q, k_ext, v_ext, out, 0, front)
        if back:
            self._run(q, k_ext, v_ext, out, L.rows - back, L.rows)
        return out

    def _run(self, q, k_ext, v_ext, out, a: int, b: int, own_rows_only: bool = False) -> None:
        if b <= a:
            return
        L = self.layout
        if own_rows_only:   # batch 1 here, so a row range of the extended buffer is still contiguous
            k_ext, v_ext = k_ext[:, L.halo_front:L.halo_front + L.rows], v_ext[:, L.halo_front:L.halo_front + L.rows]
            spec = self.spec.shifted(a)
        else:
            spec = self.spec.shifted(L.halo_front + a)
        whole = a == 0 and b == q.shape[1]
        self.forward_fn(q if whole else q[:, a:b], k_ext, v_ext, spec,
                        out=out if whole else out[:, a:b])


class PeerTensor:
    """A contiguous [B, S, H, D] tensor that lives on a neighbouring GPU, mapped into
    this process for kernels on this rank's device: just an address and a shape."""

    def __init__(self, ptr: int, shape: Tuple[int, ...], dtype: torch.dtype):
        self._ptr, self.shape, self.dtype = int(ptr), tuple(shape), dtype

    def data_ptr(self) -> int:
        return self._ptr

    def dim(self) -> int:
        return len(self.shape)

    def is_contiguous(self) -> bool:
        return True


@dataclass
class PeerShard:
    """One rank's K/V chunk plus its neighbours' chunks mapped into this process."""
    k: torch.Tensor
    v: torch.Tensor
    prev_kv: Optional[Tuple[PeerTensor, PeerTensor]]
    next_kv: Optional[Tuple[PeerTensor, PeerTensor]]


class PeerHaloAttention:
    """Sequence-sharded forward WITHOUT an exchange step: each rank keeps only its own
    chunk of K and V, and the kernel's edge tiles read the halo rows they need straight
    out of the neighbouring GPUs' memory over NVLink (peer-mapped pointers, plain tiled
    TMA loads issued by the same kernel that does the attention).  One launch per step,
    no send/recv, no halo copy, nothing for the host to wait on.

    ``register`` is collective: every rank passes its own contiguous [B, rows, H, 64]
    K and V once; CUDA IPC handles go to the neighbours, which map them.  The tensors
    must then be updated in place.  Ordering is the caller's: a rank may launch
    ``forward`` only when its neighbours' K/V for that step are complete, and may rewrite
    its own K/V only when its neighbours' kernels of the previous step have read them.
    Static K/V need nothing; a pipeline that rewrites K/V in place calls ``step_barrier``
    after the writes and again after the forward (or orders the steps some other way, e.g.
    with a stream-ordered flag).
    """

    def __init__(self, spec: PatternSpec, seq_len: int, group: Optional[dist.ProcessGroup] = None):
        if spec.kind != WINDOW:
            raise ValueError("sequence sharding applies to window patterns")
        self.group, self.spec = group, spec
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if seq_len % self.world:
            raise ValueError(f"sequence length {seq_len} is not divisible by {self.world} ranks")
        self.rows = seq_len // self.world
        unit = 16 * spec.dilation
        if self.rows % unit:
            raise ValueError(f"chunk length {self.rows} must be a multiple of 16*dilation = {unit}")
        if max(spec.left, spec.right) * spec.dilation > self.rows:
            raise ValueError("window reaches past the neighbouring chunk: use fewer ranks")
        self.start = self.rank * self.rows
        self._opened = {}   # IPC handle bytes -> mapped base address

    def register(self, k_local: torch.Tensor, v_local: torch.Tensor) -> PeerShard:
        import ctypes as C
        from . import _native as nat
        for t in (k_local, v_local):
            if not (t.is_cuda and t.is_contiguous() and t.dim() == 4 and t.shape[1] == self.rows):
                raise ValueError("expected contiguous CUDA tensors [B, rows, H, D] holding this rank's chunk")
        my_dev = k_local.device.index

        def export(t):
            handle = C.create_string_buffer(64)
            off = C.c_int64(0)
            with torch.cuda.device(my_dev):
                nat.check(nat.lib.mat_ipc_export(t.data_ptr(), handle, C.byref(off)))
            return bytes(handle.raw), int(off.value), tuple(t.shape), t.dtype

        torch.cuda.synchronize(my_dev)   # the chunk's contents are in place before anyone maps it
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (export(k_local), export(v_local)), group=self.group)

        def open_one(desc):
            handle, off, shape, dtype = desc
            base = self._opened.get(handle)
            if base is None:   # one mapping per exported allocation and process
                out = C.c_void_p()
                nat.check(nat.lib.mat_ipc_open(handle, my_dev, C.byref(out)))
                base = self._opened[handle] = int(out.value)
            return PeerTensor(base + off, shape, dtype)

        def open_neighbour(r):
            return tuple(open_one(d) for d in everyone[r])

        prev_kv = open_neighbour(self.rank - 1) if self.rank > 0 and self.spec.left else None
        next_kv = open_neighbour(self.rank + 1) if self.rank < self.world - 1 and self.spec.right else None
        dist.barrier(group=self.group)   # every mapping exists before anyone may free or reuse memory
        return PeerShard(k_local, v_local, prev_kv, next_kv)

    def step_barrier(self) -> None:
        """Collective.  Everything this rank has enqueued on its current stream (writes of its K/V
        chunk, or a ``forward`` that reads the neighbours' chunks) completes, then all ranks meet:
        after it a neighbour's rows are safe to read, or this rank's rows are safe to rewrite.
        Host-side (a stream synchronise and a barrier of the group), so it costs a launch gap."""
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)

    def close(self) -> None:
        """Unmaps every neighbour allocation this object opened (collective use not required)."""
        from . import _native as nat
        dev = torch.cuda.current_device()
        for base in self._opened.values():
            nat.check(nat.lib.mat_ipc_close(base, dev))
        self._opened.clear()

    def forward(self, q: torch.Tensor, shard: PeerShard, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from . import sparse_attention_cuda
        return sparse_attention_cuda.forward_sharded(q, shard.k, shard.v, self.spec, shard.prev_kv,
                                                     shard.next_kv, out=out)


def gather_sequence(out_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather of the per-rank outputs along the sequence axis (checking aid)."""
    world = dist.get_world_size(group)
    parts: List[torch.Tensor] = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)
