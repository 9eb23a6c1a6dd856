"""Every row of every full-size configuration against the CPU oracle.

The five benchmark configurations at their real sizes, not reduced ones: grid
shapes (tile indices past 65535, the last partly filled wave, key splits sized
to the machine), 32-bit offsets and layout walks of full length only show up
there.  The oracle finishes each of them in seconds on the host cores, so every
output row is compared, not a sample.  Bars as everywhere: fp32
max|gpu-oracle| / max|oracle| <= 1e-5; bf16 max|gpu-oracle| <= 2e-2 against the
fp32 oracle fed the bf16-rounded inputs.
"""
import numpy as np
import pytest
import torch

from ma_transformer_b200 import _native as nat
from ma_transformer_b200 import sparse_attention_cuda as ext
from ma_transformer_b200.patterns import PatternSpec, band_random_block_layout
from helpers import BF16_ABS, FP32_REL, oracle_out, rel_err, seeded_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(spec, q, k, v):
    out = ext.forward_pattern(q.to(DEV), k.to(DEV), v.to(DEV), spec)
    torch.cuda.synchronize()
    assert nat.device_status() == 0
    return out.float().cpu().numpy()


def _worst_rows(got, want, n=3):
    err = np.abs(got - want).max(axis=(2, 3))          # [B, S]
    flat = np.argsort(err, axis=None)[::-1][:n]
    return [(int(i // err.shape[1]), int(i % err.shape[1]), float(err.flat[i])) for i in flat]


def test_cfg1_full_size_fp32():
    # B=1, H=4, N=1024, d=64, 32 causal taps, fp32
    spec = PatternSpec.causal_window(32)
    q, k, v = seeded_qkv(1, 1, 1024, 4, 64)
    got = _run(spec, q, k, v)
    assert rel_err(got, oracle_out(q, k, v, spec)) <= FP32_REL


def test_cfg2_full_size_every_row():
    # B=1, H=8, N=65536, d=64, 64 causal taps, bf16, values N(0,1)*0.5
    spec = PatternSpec.causal_window(64)
    q, k, v = seeded_qkv(2, 1, 65536, 8, 64, torch.bfloat16, scale=0.5)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "umma_band"
    want = oracle_out(q, k, v, spec)
    assert np.isfinite(got).all()
    e = float(np.abs(got - want).max())
    assert e <= BF16_ABS, (e, _worst_rows(got, want))


def test_cfg2_shape_reference_default_window_every_row():
    # the window every unmodified caller of the reference gets (window_size=64: keys i-64..i+64) at the same shape
    spec = PatternSpec.sliding_window(64)
    q, k, v = seeded_qkv(6, 1, 65536, 8, 64, torch.bfloat16, scale=0.5)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "umma_band"
    want = oracle_out(q, k, v, spec)
    e = float(np.abs(got - want).max())
    assert e <= BF16_ABS, (e, _worst_rows(got, want))


def test_cfg3_full_size_every_row():
    # B=4, H=8, N=16384, d=64, block 64, causal band of 4 + 2 seeded random earlier blocks, bf16
    B, S, H = 4, 16384, 8
    rp, ci = band_random_block_layout(S // 64, 4, 2, seed=2)
    assert len(rp) == 257 and rp[-1] == 1521           # 256 layout rows, 1521 block entries
    spec = PatternSpec.block_sparse(64, rp, ci, causal=True)
    q, k, v = seeded_qkv(3, B, S, H, 64, torch.bfloat16)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "umma_block"
    want = oracle_out(q, k, v, spec)
    assert np.isfinite(got).all()
    e = float(np.abs(got - want).max())
    assert e <= BF16_ABS, (e, _worst_rows(got, want))
    # every distinct number of blocks per layout row occurs and was covered (1..6)
    assert set(np.diff(rp).tolist()) == {1, 2, 3, 4, 5, 6}


def test_cfg4_full_size_every_row():
    # B=2, H=12, N=32768, d=64, window +-64, 32 seeded global positions, bf16
    B, S, H = 2, 32768, 12
    g = torch.Generator().manual_seed(4)
    glob = torch.randperm(S, generator=g)[:32].sort().values.numpy()
    spec = PatternSpec.longformer(64, 64, glob)
    q, k, v = seeded_qkv(4, B, S, H, 64, torch.bfloat16)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "umma_longformer"
    want = oracle_out(q, k, v, spec)
    assert np.isfinite(got).all()
    e = float(np.abs(got - want).max())
    assert e <= BF16_ABS, (e, _worst_rows(got, want))
    # the rows at the global positions (every key, split over CTAs and merged) on their own
    eg = float(np.abs(got[:, glob] - want[:, glob]).max())
    assert eg <= BF16_ABS, eg


def test_cfg5_attention_full_size_every_row():
    # the order-book model's attention: B=16, N=8192, 4 heads of 64, 64 causal taps with dilation 2, bf16
    spec = PatternSpec.causal_window(64, dilation=2)
    q, k, v = seeded_qkv(5, 16, 8192, 4, 64, torch.bfloat16)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "umma_band"
    want = oracle_out(q, k, v, spec)
    e = float(np.abs(got - want).max())
    assert e <= BF16_ABS, (e, _worst_rows(got, want))


@pytest.mark.parametrize("D,H", [(64, 8), (128, 4), (256, 2)])
def test_reference_precision_default_window_long_sequence_every_row(D, H):
    # what an unmodified caller of the reference passes: fp32, window_size=64 (keys i-64..i+64); 65536 tokens x 512
    # columns as 8 heads of 64, 4 of 128, 2 of 256 (its layer passes one head of width model_dim)
    spec = PatternSpec.sliding_window(64)
    q, k, v = seeded_qkv(8, 1, 65536, H, D)
    got = _run(spec, q, k, v)
    assert nat.last_kernel() == "mma_window_f32"
    assert np.isfinite(got).all()
    assert rel_err(got, oracle_out(q, k, v, spec)) <= FP32_REL


@pytest.mark.parametrize("D,H,dtype", [(128, 4, torch.float32), (256, 2, torch.float32), (256, 2, torch.bfloat16)])
@pytest.mark.parametrize("left,right", [(63, 0), (64, 64)])
def test_wide_head_backward_long_sequence_against_warp_kernels(monkeypatch, D, H, dtype, left, right):
    # 65536 tokens: tile indices and offsets of full size; the one-warp-per-row kernels (fp32 arithmetic, no tensor
    # cores, no slicing of the head) are the independent implementation at a size autograd through a dense mask
    # cannot reach
    spec = PatternSpec(left=left, right=right)
    q, k, v = seeded_qkv(9, 1, 65536, H, D, dtype, scale=0.5)
    go = torch.randn(1, 65536, H, D, generator=torch.Generator().manual_seed(10)).to(dtype)
    args = tuple(t.to(DEV) for t in (q, k, v, go))
    got = ext.backward_pattern(*args, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == ("bwd_f32_mma" if dtype == torch.float32 else "bwd_d_mma") and nat.device_status() == 0
    monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
    want = ext.backward_pattern(*args, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "bwd_window"
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert torch.isfinite(a).all(), name
        err = float((a.float() - b.float()).abs().max())
        assert err <= tol * max(1.0, float(b.float().abs().max())), f"{name}: {err}"
