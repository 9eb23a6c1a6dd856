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
from helpers import BF16_ABS, F16_ABS, oracle_out, seeded_qkv

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
        # the driver's own count of free device memory sees every allocation in the process, whoever made
        # it; the first call on a device may load the library's device code, so it is the warm-up
        free_before = torch.cuda.mem_get_info(DEV)[0]
        rc = _call_noalloc(q, k, v, out, s)
        assert rc == 0, nat.lib.mat_last_error().decode()
        torch.cuda.synchronize()
        if call > 0:
            assert torch.cuda.mem_get_info(DEV)[0] == free_before
        assert nat.last_kernel() == "mma_longformer_static"
        diff = float((out.float() - want.float()).abs().max())
        assert diff <= BF16_ABS, f"call {call}: differs from the workspace entry point by {diff}"
        # and both against the oracle, rows at global positions included
        ref = oracle_out(q.cpu(), k.cpu(), v.cpu(), spec)
        assert float(np.abs(out.float().cpu().numpy() - ref).max()) <= BF16_ABS
        assert float(np.abs(out.float().cpu().numpy()[:, glob] - ref[:, glob]).max()) <= BF16_ABS
    assert nat.device_status() == 0


@pytest.mark.parametrize("B,S,H,n_glob,window,dtype", [
    (4, 16384, 16, 32, 8, torch.bfloat16),   # 1.08 MB of partials per key split: 3 splits fit where 32 are wanted
    (4, 4096, 32, 32, 8, torch.bfloat16),    # 2.16 MB per split: a single split, nothing to merge across
    (1, 2048, 2, 100, 16, torch.bfloat16),   # more than 64 global positions: two tiles of global rows
    (2, 1024, 3, 5, 64, torch.float16),      # fp16
], ids=["three-splits-fit", "one-split", "two-tiles", "fp16"])
def test_noalloc_entry_when_the_scratch_limits_the_key_splits(B, S, H, n_glob, window, dtype):
    g = torch.Generator().manual_seed(10)
    glob = torch.randperm(S, generator=g)[:n_glob].sort().values.numpy()
    spec = PatternSpec.longformer(window, window, glob)
    s = spec.device_struct(DEV)
    q, k, v = seeded_qkv(73, B, S, H, 64, dtype)
    out = torch.full((B, S, H, 64), float("nan"), dtype=dtype, device=DEV)
    rc = _call_noalloc(q.to(DEV), k.to(DEV), v.to(DEV), out, s)
    assert rc == 0, nat.lib.mat_last_error().decode()
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    tol = BF16_ABS if dtype == torch.bfloat16 else F16_ABS
    # the rows at the global positions (every key, merged over the splits) in full
    qg = q[:, glob].contiguous()
    want_g = oracle_out(qg, k, v, PatternSpec(left=S, right=S))     # a global row takes every key
    assert float(np.abs(got[:, glob] - want_g).max()) <= tol
    # and every other row of the first and last 512 positions plus a block in the middle
    for a in (0, S // 2 - 256, S - 512):
        # these query rows against the whole key axis (window, global keys, and all keys for global rows)
        sl = PatternSpec.longformer(window, window, glob).shifted(a)
        want = oracle_out(q[:, a:a + 512].contiguous(), k, v, sl)
        assert float(np.abs(got[:, a:a + 512] - want).max()) <= tol, a
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
    ext.forward_pattern(q, q, q, PatternSpec.causal_window(8))
    kernel_before = nat.last_kernel()
    poisoned = torch.full_like(big, 3.0)
    torch.cuda.synchronize()
    assert _call_noalloc(big, big, big, poisoned, sb) == 2
    assert b"scratch" in nat.lib.mat_last_error()
    # a refused call has launched nothing: the output keeps its contents, no kernel was noted
    torch.cuda.synchronize()
    assert bool((poisoned == 3.0).all())
    assert nat.last_kernel() == kernel_before
    # the python wrapper turns the refusal into RuntimeError
    with pytest.raises(RuntimeError, match="scratch"):
        ext.forward_longformer_noalloc(big, big, big, PatternSpec.longformer(2, 2, [1, 5]), poisoned)
    assert bool((poisoned == 3.0).all())
