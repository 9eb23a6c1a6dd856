"""The multi-rank path on CPU: two gloo ranks run the sequence-sharded forward
(halo exchange by send/recv) with the oracle standing in for the kernel, and the
gathered result must equal the single-process oracle bit for bit."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _oracle_forward(q, k, v, spec, out=None):
    from helpers import oracle_out
    res = torch.from_numpy(oracle_out(q, k, v, spec))
    if out is None:
        return res
    out.copy_(res)
    return out


def _worker(rank, world, port, cases, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ma_transformer_b200.patterns import PatternSpec
        from ma_transformer_b200.sharded import SequenceShardedAttention, gather_sequence
        from helpers import seeded_qkv
        for n, (B, S, H, D, left, right, dil, overlap) in enumerate(cases):
            spec = PatternSpec(left=left, right=right, dilation=dil)
            q, k, v = seeded_qkv(100 + n, B, S, H, D)
            sh = SequenceShardedAttention(spec, S, forward_fn=_oracle_forward, overlap=overlap)
            L = sh.layout
            k_ext = sh.alloc_kv(B, H, D, torch.float32, "cpu")
            v_ext = sh.alloc_kv(B, H, D, torch.float32, "cpu")
            k_ext.fill_(float("nan"))   # a halo row that never arrives poisons the result
            v_ext.fill_(float("nan"))
            sh.chunk_view(k_ext).copy_(k[:, L.start:L.start + L.rows])
            sh.chunk_view(v_ext).copy_(v[:, L.start:L.start + L.rows])
            out = sh.forward(q[:, L.start:L.start + L.rows].contiguous(), k_ext, v_ext)
            full = gather_sequence(out)
            if rank == 0:
                want = _oracle_forward(q, k, v, spec)
                results.put((n, bool(torch.equal(full, want)), float((full - want).abs().max())))
    finally:
        dist.destroy_process_group()


CASES = [
    # B, S, H, D, left, right, dilation, overlap
    (1, 256, 2, 8, 63, 0, 1, True),     # the causal 64-tap halo of the long-sequence configuration
    (1, 256, 2, 8, 5, 9, 1, True),      # two-sided: both neighbours
    (2, 128, 1, 4, 7, 7, 1, True),      # B > 1: strided halo rows, no overlap split
    (1, 512, 1, 4, 15, 0, 2, True),     # dilated
    (1, 256, 1, 4, 0, 0, 1, False),     # nothing to exchange
]


def test_two_rank_halo_exchange_matches_single_process():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, CASES, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, "a rank failed or hung"
    got = sorted(results.get(timeout=5) for _ in CASES)
    for n, same, err in got:
        assert same, f"case {n}: sharded result differs from the single-process oracle (max err {err})"


def test_shard_layout_rules():
    from ma_transformer_b200.patterns import PatternSpec
    from ma_transformer_b200.sharded import shard_batch_heads, shard_layout
    spec = PatternSpec.causal_window(64)
    L = [shard_layout(spec, 65536, r, 8) for r in range(8)]
    assert [x.halo_front for x in L] == [0] + [64] * 7   # 63 rows of reach, rounded up to 16 and all(x.halo_back == 0 for x in L)
    assert all(x.rows == 8192 for x in L) and L[3].start == 3 * 8192
    with pytest.raises(ValueError):
        shard_layout(PatternSpec.causal_window(64), 100, 0, 8)        # not divisible
    with pytest.raises(ValueError):
        shard_layout(PatternSpec.sliding_window(600), 1024, 0, 2)     # reaches past the neighbour
    with pytest.raises(ValueError):
        shard_layout(PatternSpec.longformer(4, 4, [0]), 1024, 0, 2)   # not a window pattern
    cover = [shard_batch_heads(32, r, 5) for r in range(5)]
    assert cover[0][0] == 0 and cover[-1][1] == 32 and all(a[1] == b[0] for a, b in zip(cover, cover[1:]))
