"""Sequence-sharded forward on real GPUs (NCCL halo exchange), checked against the
single-process CPU oracle.  Needs at least two GPUs; skipped otherwise."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ma_transformer_b200 import _native as nat
        from ma_transformer_b200.patterns import PatternSpec
        from ma_transformer_b200.sharded import SequenceShardedAttention, gather_sequence
        from helpers import oracle_out, seeded_qkv
        cases = [(PatternSpec.causal_window(64), 1, 4096, torch.bfloat16),
                 (PatternSpec.sliding_window(20), 1, 2048, torch.bfloat16),
                 (PatternSpec.causal_window(16, dilation=2), 1, 2048, torch.bfloat16),
                 (PatternSpec.causal_window(32), 2, 1024, torch.float32)]
        for n, (spec, B, S, dtype) in enumerate(cases):
            q, k, v = seeded_qkv(200 + n, B, S, 4, 64, dtype)
            sh = SequenceShardedAttention(spec, S)
            L = sh.layout
            k_ext = sh.alloc_kv(B, 4, 64, dtype, dev)
            v_ext = sh.alloc_kv(B, 4, 64, dtype, dev)
            k_ext.fill_(float("nan"))
            v_ext.fill_(float("nan"))
            sh.chunk_view(k_ext).copy_(k[:, L.start:L.start + L.rows])
            sh.chunk_view(v_ext).copy_(v[:, L.start:L.start + L.rows])
            out = sh.forward(q[:, L.start:L.start + L.rows].contiguous().to(dev), k_ext, v_ext)
            full = gather_sequence(out)
            torch.cuda.synchronize()
            if rank == 0:
                want = torch.from_numpy(oracle_out(q, k, v, spec))
                err = float((full.float().cpu() - want).abs().max())
                tol = 2e-2 if dtype == torch.bfloat16 else 1e-5 * float(want.abs().max())
                results.put((n, err <= tol, err))
        assert nat.device_status() == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_forward_on_gpus_matches_oracle():
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29700 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0, "a rank failed or hung"
    for _ in range(4):
        n, ok, err = results.get(timeout=5)
        assert ok, f"case {n}: max error {err}"
