"""The allocation-free Longformer entry point (mat_sparse_attn_fwd_longformer_noalloc),
called straight through the C ABI, against the ordinary entry point that takes a
caller workspace.

Who needs it: a host that may not obtain device memory once it is running, such as
a server whose own arena took all of HBM at start-up, or a latency-critical loop that
cannot accept the device-wide stall an allocation brings.  Such a caller passes inputs
and output only; the scratch is a fixed array inside the library.

Collected last on purpose (file name), so a run that stops at the first failure has
already run every other test.  Passes alone in a fresh process and after the others.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from ma_transformer_b200 import _native as nat
from ma_transformer_b200 import sparse_attention_cuda as ext
from ma_transformer_b200.patterns import PatternSpec
from helpers import BF16_ABS, oracle_out, seeded_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {torch.bfloat16: nat.MAT_BF16, torch.float16: nat.MAT_F16}


def _call_noalloc(q, k, v, out, spec_struct):
    B, S, H, D = q.shape
    stream = torch.cuda.current_stream(q.device).cuda_stream
    return nat.lib.mat_sparse_attn_fwd_longformer_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, D, DT[q.dtype],
        C.byref(spec_struct), 0.0, C.c_void_p(stream))


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row():
    g = torch.Generator().manual_seed(9)
    S = 4096
    glob = torch.randperm(S, generator=g)[:32].sort().values.numpy()
    spec = PatternSpec.longformer(64, 64, glob)
    s = spec.device_struct(DEV)          # global positions on the device, uploaded before the calls
    for call, seed in enumerate((71, 72)):   # two calls in a row share the built-in scratch
        q, k, v = (t.to(DEV) for t in seeded_qkv(seed, 2, S, 4, 64, torch.bfloat16))
        want = ext.forward_pattern(q, k, v, spec)          # existing entry point, caller workspace
        out = torch.full_like(q, float("nan"))             # caller-owned output, poisoned
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(DEV)
        rc = _call_noalloc(q, k, v, out, s)
        assert rc == 0, nat.lib.mat_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(DEV) == before  # nothing came from torch's allocator either
        assert nat.last_kernel() == "mma_longformer_static"
        diff = float((out.float() - want.float()).abs().max())
        assert diff <= BF16_ABS, f"call {call}: differs from the workspace entry point by {diff}"
        # and both against the oracle, rows at global positions included
        ref = oracle_out(q.cpu(), k.cpu(), v.cpu(), spec)
        assert float(np.abs(out.float().cpu().numpy() - ref).max()) <= BF16_ABS
        assert float(np.abs(out.float().cpu().numpy()[:, glob] - ref[:, glob]).max()) <= BF16_ABS
    assert nat.device_status() == 0


def test_noalloc_entry_refuses_what_it_cannot_hold():
    q = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    # not a Longformer pattern
    s = PatternSpec.causal_window(8).device_struct(DEV)
    assert _call_noalloc(q, q, q, out, s) == 2
    assert b"LONGFORMER" in nat.lib.mat_last_error()
    # fp32 is outside the tiled kernels
    qf = q.float()
    sl = PatternSpec.longformer(2, 2, [0, 7]).device_struct(DEV)
    B, S, H, D = qf.shape
    rc = nat.lib.mat_sparse_attn_fwd_longformer_noalloc(qf.data_ptr(), qf.data_ptr(), qf.data_ptr(), qf.data_ptr(),
                                                        B, S, H, D, nat.MAT_F32, C.byref(sl), 0.0, None)
    assert rc == 2
    # partials beyond the built-in 4 MiB even without splitting: B*H*ceil64(globals)*264 bytes
    big = torch.zeros(8, 2048, 32, 64, dtype=torch.bfloat16, device=DEV)   # 8*32*64*264 = 4.3 MB
    sb = PatternSpec.longformer(2, 2, [1, 5]).device_struct(DEV)
    assert _call_noalloc(big, big, big, torch.empty_like(big), sb) == 2
    assert b"scratch" in nat.lib.mat_last_error()
    # the python wrapper turns the refusal into RuntimeError
    with pytest.raises(RuntimeError, match="scratch"):
        ext.forward_longformer_noalloc(big, big, big, PatternSpec.longformer(2, 2, [1, 5]), torch.empty_like(big))
