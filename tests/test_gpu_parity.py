"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle
and the committed golden vectors of the reference.  Bars: fp32 rel-err <= 1e-5
(max|gpu-oracle| / max|oracle|), bf16 max-abs <= 2e-2 against the fp32 oracle fed
the bf16-rounded inputs, index sets bit-exact."""
import numpy as np
import pytest
import torch

import ma_transformer_b200 as mt
from ma_transformer_b200 import _native as nat
from ma_transformer_b200 import sparse_attention_cuda as ext
from ma_transformer_b200.patterns import PatternSpec, band_random_block_layout, tridiagonal_block_layout
from helpers import (check_close, expected_window_kernel, masked_attention_with, masked_dense_attention, oracle_out,
                     pattern_mask, rel_err, seeded_qkv,
                     to_oracle)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run(spec, q, k, v, scale=None):
    out = ext.forward_pattern(q.to(DEV), k.to(DEV), v.to(DEV), spec, scale)
    torch.cuda.synchronize()
    return out


# ---- the reference's own cases (golden vectors) ------------------------------------

def test_golden_vectors_fp32(golden):
    worst = 0.0
    for n, (seed, B, S, H, D, W) in enumerate(golden["meta"].tolist()):
        tag = f"{seed}_{B}_{S}_{H}_{D}"
        q, k, v = (torch.from_numpy(golden[f"{t}_{tag}"]).to(DEV) for t in "qkv")
        got = ext.forward(q, k, v, W).cpu().numpy()
        want = golden[f"ref_cpp{n}"]
        worst = max(worst, rel_err(got, want))
        # the reference's own CUDA tolerance (tests/integration/test_cuda_parity.py:42-57)
        assert np.abs(got - golden[f"ref_torch{n}"]).max() < 1e-4
    assert worst <= 1e-5, worst
    # (the last case's head width decides the kernel: the reference's cases use 16, 32 and 64 columns and odd widths)
    assert nat.last_kernel() == ("mma_window_f32" if D % 4 == 0 and D <= 512 else "rowwarp")


def test_cfg1_causal_window_fp32():
    # B=1, H=4, N=1024, d=64, 32 causal taps, scale 1/8
    spec = PatternSpec.causal_window(32)
    q, k, v = seeded_qkv(1, 1, 1024, 4, 64)
    check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), torch.float32)
    assert nat.last_kernel() == "mma_window_f32"
    check_close(run(spec, q, k, v, scale=0.125), oracle_out(q, k, v, spec, 0.125), torch.float32)


@pytest.mark.parametrize("D", [8, 16, 32, 40, 48, 64, 80, 96, 112, 128, 200, 256, 512])
@pytest.mark.parametrize("spec", [PatternSpec.causal_window(32), PatternSpec.sliding_window(64), PatternSpec.sliding_window(3),
                                  PatternSpec(left=0, right=60), PatternSpec.causal_window(64, dilation=2),
                                  PatternSpec(left=100, right=28), PatternSpec.causal_window(1)],
                         ids=lambda s: f"l{s.left}r{s.right}d{s.dilation}")
@pytest.mark.parametrize("kernel", ["default", "chunks", "tiled"])
def test_fp32_window_kernels_vs_oracle(monkeypatch, kernel, spec, D):
    """fp32 windows of at most 128 taps with head width 32, 64, 128 or 256, ragged lengths and shard offsets included,
    at the fp32 bar of 1e-5: on the tensor cores as three TF32 products of error-compensated halves (the default, with
    every warp walking its own key range, wide heads 64 columns at a time; MAT_F32_KERNEL=chunks keeps these windows on the
    variant that walks 64-key chunks per tile, which wider windows use), and on the tiled FMA-pipe kernel (64- or
    128-row tiles, K/V window staged once per tile; head width 128, and MAT_F32_KERNEL=tiled)."""
    if kernel != "default":
        monkeypatch.setenv("MAT_F32_KERNEL", kernel)
    for B, S, H, off in [(1, 1024, 2, 0), (2, 330, 3, 0), (1, 64, 1, 0), (1, 200, 2, 48), (1, 7, 1, 0)]:
        S = S - S % spec.dilation if S >= spec.dilation else spec.dilation
        off = off - off % spec.dilation
        sp = spec.shifted(off)
        q, k, v = seeded_qkv(23, B, S, H, D, torch.float32, Skv=S + off + 3 * spec.dilation)
        got = run(sp, q, k, v)
        skv1 = (S + off + 3 * spec.dilation) // spec.dilation          # taps clamp to the keys that exist
        wide_here = min(spec.left, skv1) + min(spec.right, skv1) > 64
        if kernel != "tiled":   # (head widths 128 and 256: 64 columns at a time, these windows in one pass per warp)
            assert nat.last_kernel() == "mma_window_f32"
        else:
            assert nat.last_kernel() == ("tiled_f32" if D in (32, 64) or (D == 128 and not wide_here) else "rowwarp")
        check_close(got, oracle_out(q, k, v, sp), torch.float32)
    # inputs x100 stay finite and close (tests/integration/test_cuda_extensive.py:77-92)
    q, k, v = seeded_qkv(24, 1, 130, 2, D, torch.float32, scale=100.0)
    got = run(spec, q, k, v).cpu().numpy()
    # (scores of this size sit where fp32 rounding of a dot product decides between neighbouring keys; the longer the
    # dot product, the further two correct evaluation orders can be apart)
    assert np.isfinite(got).all() and np.abs(got - oracle_out(q, k, v, spec)).max() <= 0.5 * max(1.0, D / 256)


@pytest.mark.parametrize("S,spec", [(1000, PatternSpec.sliding_window(3000)), (1000, PatternSpec.causal_window(3000)),
                                    (1500, PatternSpec.sliding_window(400)), (2100, PatternSpec(left=513, right=0)),
                                    (4096, PatternSpec.sliding_window(4096))],
                         ids=["dense1000", "causal1000", "pm400", "l513", "dense4096"])
@pytest.mark.parametrize("D", [16, 32, 40, 64, 80, 96, 128, 256])
def test_fp32_wide_windows_on_tensor_cores(S, spec, D):
    """fp32 windows of any width, dense and causal dense included, as three TF32 products per product: the fp32 bar
    holds on rows of thousands of keys (the sums of a chunk end with the chunk, and chunks are combined by
    ordinary FMAs: the tensor core's own fp32 accumulation does not round to nearest)."""
    q, k, v = seeded_qkv(31, 1, S, 2, D, torch.float32)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "mma_window_f32"
    check_close(got, oracle_out(q, k, v, spec), torch.float32)


@pytest.mark.parametrize("D", [16, 32, 48, 80, 96, 112, 128])
@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.sliding_window(32), PatternSpec.sliding_window(64),
                                  PatternSpec(left=0, right=60), PatternSpec.causal_window(16, dilation=2),
                                  PatternSpec(left=5, right=90), PatternSpec.causal_window(300), PatternSpec.sliding_window(5000),
                                  PatternSpec.causal_window(1)],
                         ids=lambda s: f"l{s.left}r{s.right}d{s.dilation}")
def test_16bit_windows_with_head_width_32_and_128(monkeypatch, spec, D):
    """16-bit windows with a head width that is a multiple of 16 up to 128 (other than 64) on the warp-level tensor-core kernel (64-row tiles, keys
    through cp.async, online softmax; per-warp key ranges for narrow windows, 64-key chunks for wide ones): narrow, wide (several chunks), dense-as-window, dilated, ragged lengths,
    shard offsets; and the one-warp-per-row kernel on the same inputs."""
    for dtype in (torch.bfloat16, torch.float16):
        for B, S, H, off in [(1, 1024, 2, 0), (2, 330, 3, 0), (1, 64, 1, 0), (1, 200, 2, 48), (1, 7, 1, 0)]:
            S = S - S % spec.dilation if S >= spec.dilation else spec.dilation
            off = off - off % spec.dilation
            sp = spec.shifted(off)
            q, k, v = seeded_qkv(29, B, S, H, D, dtype, Skv=S + off + 3 * spec.dilation)
            got = run(sp, q, k, v)
            assert nat.last_kernel() == "mma_window_d"
            check_close(got, oracle_out(q, k, v, sp), dtype)
    # narrow windows default to the variant in which every warp walks its own key range (a head of 128 columns 64
    # columns at a time; "whole" keeps it in one piece); the 64-key chunks on them
    for force in ("chunks", "whole"):
        monkeypatch.setenv("MAT_WINDOW_D_KERNEL", force)
        for B, S, H, off in [(2, 330, 3, 0), (1, 200, 2, 48)]:
            S, off = S - S % spec.dilation, off - off % spec.dilation
            sp = spec.shifted(off)
            q, k, v = seeded_qkv(29, B, S, H, D, torch.bfloat16, Skv=S + off + 3 * spec.dilation)
            got = run(sp, q, k, v)
            assert nat.last_kernel() == "mma_window_d"
            check_close(got, oracle_out(q, k, v, sp), torch.bfloat16)
    monkeypatch.setenv("MAT_WINDOW_D_KERNEL", "rowwarp")
    q, k, v = seeded_qkv(30, 1, 330, 2, D, torch.bfloat16)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "rowwarp"
    check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)


@pytest.mark.parametrize("D", [8, 40, 144, 192, 200, 256, 512])
@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.sliding_window(64), PatternSpec.sliding_window(3),
                                  PatternSpec(left=0, right=60), PatternSpec.causal_window(32, dilation=2),
                                  PatternSpec(left=100, right=28), PatternSpec.causal_window(1)],
                         ids=lambda s: f"l{s.left}r{s.right}d{s.dilation}")
def test_16bit_windows_with_wide_heads(spec, D):
    """16-bit windows of at most 128 taps between their sides with one wide head (the reference's layer passes
    D = model_dim, src/layers/sparse_attention.py:71-78): the head dimension goes through the warp-level tensor-core
    kernel 64 columns at a time."""
    for dtype in (torch.bfloat16, torch.float16):
        for B, S, H, off in [(1, 1024, 1, 0), (2, 330, 2, 0), (1, 64, 1, 0), (1, 200, 2, 48), (1, 7, 1, 0)]:
            S = S - S % spec.dilation if S >= spec.dilation else spec.dilation
            off = off - off % spec.dilation
            sp = spec.shifted(off)
            q, k, v = seeded_qkv(33, B, S, H, D, dtype, Skv=S + off + 3 * spec.dilation)
            got = run(sp, q, k, v)
            assert nat.last_kernel() == "mma_window_d"
            check_close(got, oracle_out(q, k, v, sp), dtype)
    # wider windows, up to dense: several passes per warp, the partial rows in an fp32 scratch (the workspace)
    for wide, S in ((PatternSpec.causal_window(300), 330), (PatternSpec.sliding_window(200), 1000), (PatternSpec.sliding_window(5000), 700)):
        for dtype in (torch.bfloat16, torch.float16):
            q, k, v = seeded_qkv(34, 2, S, 2, D, dtype)
            got = run(wide, q, k, v)
            assert nat.last_kernel() == "mma_window_d"
            check_close(got, oracle_out(q, k, v, wide), dtype)


@pytest.mark.parametrize("B,S,H,D", [(1, 1, 1, 1), (1, 7, 2, 5), (2, 33, 1, 13), (1, 100, 3, 40), (1, 65, 2, 96),
                                     (1, 40, 1, 200), (1, 18, 1, 512)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_rowwarp_odd_shapes(B, S, H, D, dtype):
    for spec in (PatternSpec.sliding_window(4), PatternSpec.causal_window(9, dilation=3),
                 PatternSpec(left=2, right=5, dilation=2)):
        q, k, v = seeded_qkv(7, B, S, H, D, dtype)
        check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), dtype)
        whole = S % spec.dilation == 0   # (these windows are narrow: wide heads in multiples of 64 go 64 columns at a time)
        if dtype == torch.float32:
            want = "mma_window_f32" if whole and D % 4 == 0 else "rowwarp"
        else:
            want = "mma_window_d" if whole and D % 8 == 0 else "rowwarp"
        assert nat.last_kernel() == want


def test_head_width_beyond_maximum_is_refused_loudly():
    q = torch.zeros(1, 2, 1, 520, device=DEV)
    with pytest.raises(RuntimeError, match="512"):
        ext.forward(q, q, q, 1)


# ---- tensor-core window kernel --------------------------------------------------------

WINDOW_SPECS = [
    PatternSpec.causal_window(64),
    PatternSpec.causal_window(32),
    PatternSpec.causal_window(1),
    PatternSpec.sliding_window(17),
    PatternSpec.sliding_window(64),
    PatternSpec(left=5, right=90),
    PatternSpec.causal_window(200),
    PatternSpec.sliding_window(1000),
]


@pytest.mark.parametrize("spec", WINDOW_SPECS, ids=lambda s: f"l{s.left}r{s.right}")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H", [(1, 256, 2), (2, 333, 3), (1, 64, 1), (1, 17, 2), (1, 1, 1)])
def test_mma_window_vs_oracle(spec, dtype, B, S, H):
    q, k, v = seeded_qkv(11, B, S, H, 64, dtype)
    got = run(spec, q, k, v)
    # dense attention and windows of more than 64 taps run on the tcgen05 pipeline when the sequence is long enough
    assert nat.last_kernel() == expected_window_kernel(spec, S)
    check_close(got, oracle_out(q, k, v, spec), dtype)


@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.causal_window(64, dilation=2),
                                  PatternSpec.sliding_window(64), PatternSpec(left=3, right=40, dilation=3)],
                         ids=["causal64", "dil2", "pm64", "dil3"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_views_of_a_fused_projection_are_read_in_place(spec, dtype):
    """q, k, v as views of one [B, S, 3, H, 64] tensor (token stride 3*H*64) through the strided entry point:
    bit-identical to the same values passed as packed tensors, and right against the oracle; a strided
    output view as well."""
    B, S, H = 2, 768, 3
    g = torch.Generator().manual_seed(19)
    qkv = torch.randn(B, S, 3, H, 64, generator=g).to(dtype).to(DEV)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    assert not q.is_contiguous()
    got = ext.forward_strided(q, k, v, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "umma_band"
    packed = ext.forward_pattern(q.contiguous(), k.contiguous(), v.contiguous(), spec)
    assert torch.equal(got, packed)
    check_close(got, oracle_out(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), spec), dtype)
    wide = torch.full((B, S, 2, H, 64), float("nan"), dtype=dtype, device=DEV)
    ext.forward_strided(q, k, v, spec, out=wide[:, :, 1])
    assert torch.equal(wide[:, :, 1], packed) and bool(torch.isnan(wide[:, :, 0]).all())
    # what the strided entry point does not take is refused, not copied behind the caller's back
    with pytest.raises(RuntimeError, match="token-strided"):
        ext.forward_strided(q, k, v, PatternSpec.sliding_window(300))
    with pytest.raises(RuntimeError):
        ext.forward_strided(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), spec)


def test_window_kernel_choice_by_size(monkeypatch):
    """Without MAT_WINDOW_KERNEL the library sends small narrow-window problems to the warp-level kernel (the
    persistent kernel's start-up and drain would dominate) and large ones to the persistent tcgen05 kernel;
    windows of more than 64 taps go to the tcgen05 kernel at every size.  Same answers either way."""
    monkeypatch.delenv("MAT_WINDOW_KERNEL", raising=False)
    spec = PatternSpec.causal_window(64)
    q, k, v = seeded_qkv(17, 1, 2048, 2, 64, torch.bfloat16)
    want = oracle_out(q, k, v, spec)
    check_close(run(spec, q, k, v), want, torch.bfloat16)
    assert nat.last_kernel() == "mma_window"
    qb, kb, vb = (t.repeat(1, 24, 4, 1) for t in (q, k, v))            # 49152 tokens x 8 heads: 3072 items
    run(spec, qb, kb, vb)
    assert nat.last_kernel() == "umma_band"
    check_close(run(PatternSpec.sliding_window(64), q, k, v), oracle_out(q, k, v, PatternSpec.sliding_window(64)), torch.bfloat16)
    assert nat.last_kernel() == "umma_band"
    monkeypatch.setenv("MAT_WINDOW_KERNEL", "mma")
    for s in (spec, PatternSpec.sliding_window(64), PatternSpec.sliding_window(20)):
        check_close(run(s, q, k, v), oracle_out(q, k, v, s), torch.bfloat16)
        assert nat.last_kernel() == "mma_window"


@pytest.mark.parametrize("kernel", ["band", "mma"])
@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.causal_window(33), PatternSpec.sliding_window(17),
                                  PatternSpec.sliding_window(64), PatternSpec(left=5, right=90), PatternSpec.causal_window(128)],
                         ids=lambda s: f"l{s.left}r{s.right}")
def test_both_window_kernels_vs_oracle(monkeypatch, kernel, spec):
    monkeypatch.setenv("MAT_WINDOW_KERNEL", kernel)
    for B, S, H in [(2, 1000, 3), (1, 130, 2)]:
        q, k, v = seeded_qkv(18, B, S, H, 64, torch.bfloat16)
        got = run(spec, q, k, v)
        assert nat.last_kernel() == ("umma_band" if kernel == "band" else "mma_window")
        check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)


@pytest.mark.parametrize("spec", [PatternSpec.sliding_window(65), PatternSpec.causal_window(130),
                                  PatternSpec.causal_window(200), PatternSpec(left=40, right=90),
                                  PatternSpec(left=300, right=17), PatternSpec.sliding_window(1000),
                                  PatternSpec(left=0, right=129)], ids=lambda s: f"l{s.left}r{s.right}")
@pytest.mark.parametrize("B,S,H", [(1, 1024, 2), (2, 1000, 3), (1, 4160, 2), (1, 257, 1)])
def test_wide_windows_on_tcgen05(spec, B, S, H):
    """Windows of more than 128 taps as a key range and an edge mask on the tcgen05 pipeline;
    MAT_WINDOW_KERNEL=mma keeps them on the warp-level kernel."""
    for dtype in (torch.bfloat16, torch.float16):
        q, k, v = seeded_qkv(15, B, S, H, 64, dtype)
        got = run(spec, q, k, v)
        assert nat.last_kernel() == expected_window_kernel(spec, S) in ("umma_window", "umma_dense", "umma_band")
        check_close(got, oracle_out(q, k, v, spec), dtype)


def test_wide_window_with_halo_prefix_and_kernel_switch(monkeypatch):
    """A sequence shard whose K/V carry 128 halo rows in front (q_offset = 128) on the tcgen05 window path,
    and the same call forced onto the warp-level kernel."""
    spec = PatternSpec(left=100, right=40).shifted(128)
    q, k, v = seeded_qkv(16, 1, 512, 2, 64, torch.bfloat16, Skv=640)
    want = oracle_out(q, k, v, spec)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "umma_window"
    check_close(got, want, torch.bfloat16)
    monkeypatch.setenv("MAT_WINDOW_KERNEL", "mma")
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "mma_window"
    check_close(got, want, torch.bfloat16)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,S,H", [(1, 1024, 2), (2, 1000, 3), (1, 256, 1), (1, 4160, 2)])
def test_dense_forward_on_tcgen05(causal, B, S, H):
    """dense_forward (src/cuda/sparse_attention_kernel.cu:348-382) for 16-bit inputs: the window that
    covers the sequence, run by the tcgen05 pipeline."""
    for dtype in (torch.bfloat16, torch.float16):
        q, k, v = seeded_qkv(14, B, S, H, 64, dtype)
        got = ext.dense_forward(q.to(DEV), k.to(DEV), v.to(DEV), causal)
        torch.cuda.synchronize()
        assert nat.last_kernel() == "umma_dense"
        spec = PatternSpec(left=S, right=0 if causal else S)
        check_close(got, oracle_out(q, k, v, spec), dtype)


@pytest.mark.parametrize("dil", [2, 3, 4])
@pytest.mark.parametrize("spec0", [PatternSpec.causal_window(64), PatternSpec.sliding_window(9)], ids=["causal64", "pm9"])
def test_mma_window_dilated(spec0, dil):
    spec = PatternSpec(left=spec0.left, right=spec0.right, dilation=dil)
    S = 96 * dil
    q, k, v = seeded_qkv(12, 2, S, 2, 64, torch.bfloat16)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "umma_band"
    check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)
    # ragged against the dilation: the general kernel takes over, same answer
    q, k, v = seeded_qkv(13, 1, S + 1, 2, 64, torch.bfloat16)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "rowwarp"
    check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)


def test_cfg2_shape_reduced_length_bf16():
    # cfg-2's heads, width, taps and value distribution at a length the oracle finishes quickly
    spec = PatternSpec.causal_window(64)
    q, k, v = seeded_qkv(2, 1, 4096, 8, 64, torch.bfloat16, scale=0.5)
    check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), torch.bfloat16)
    assert nat.last_kernel() == "umma_band"


def test_large_magnitudes_stay_finite():
    # tests/integration/test_cuda_extensive.py:77-92 scales the inputs by 100
    spec = PatternSpec.sliding_window(8)
    for dtype in (torch.float32, torch.bfloat16):
        q, k, v = seeded_qkv(3, 1, 130, 2, 64, dtype, scale=100.0)
        got = run(spec, q, k, v).float().cpu().numpy()
        want = oracle_out(q, k, v, spec)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= (5e-3 if dtype == torch.float32 else 2.0) * 100


# ---- sequence shards: halo rows in front of / behind the shard's keys -------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.sliding_window(20),
                                  PatternSpec.causal_window(16, dilation=2)], ids=["causal64", "pm20", "dil2"])
def test_shard_with_halo_equals_full_run(spec, dtype):
    S, P = 512, 4
    q, k, v = seeded_qkv(21, 1, S, 2, 64, dtype)
    full = run(spec, q, k, v)
    chunk = S // P
    for r in range(P):
        lo = max(0, r * chunk - spec.left * spec.dilation)
        hi = min(S, (r + 1) * chunk + spec.right * spec.dilation)
        part = run(spec.shifted(r * chunk - lo), q[:, r * chunk:(r + 1) * chunk].contiguous(),
                   k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous())
        ref = full[:, r * chunk:(r + 1) * chunk]
        if dtype == torch.float32:   # same key order per row; the row sums regroup with the shard's origin (last-bit effects)
            assert (part - ref).abs().max() <= 1e-6 * float(ref.abs().max()), f"shard {r}"
        else:  # tiled kernel: key chunks align to the shard's own origin, so sums regroup (a few bf16 ulps)
            assert (part.float() - ref.float()).abs().max() <= 2 ** -6, f"shard {r}"
    check_close(full, oracle_out(q, k, v, spec), dtype)


@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.causal_window(33), PatternSpec.sliding_window(20),
                                  PatternSpec(left=10, right=40), PatternSpec.causal_window(16, dilation=2),
                                  PatternSpec.causal_window(200), PatternSpec.sliding_window(100)],
                         ids=["causal64", "causal33", "pm20", "l10r40", "dil2", "causal200", "pm100"])
@pytest.mark.parametrize("B", [1, 2])
def test_neighbour_shards_read_in_place(spec, B):
    """The sharded entry point: every chunk is its own tensor and the edge tiles read
    their halo rows from the neighbouring chunks' tensors (here on the same GPU; across
    GPUs the pointers are peer-mapped).  Must equal the unsharded run."""
    S, P = 1024, 4
    q, k, v = seeded_qkv(22, B, S, 2, 64, torch.bfloat16)
    want = oracle_out(q, k, v, spec)
    chunk = S // P
    parts = [tuple(t[:, r * chunk:(r + 1) * chunk].contiguous().to(DEV) for t in (q, k, v)) for r in range(P)]
    for r in range(P):
        qr, kr, vr = parts[r]
        prev_kv = parts[r - 1][1:] if r > 0 else None
        next_kv = parts[r + 1][1:] if r < P - 1 and spec.right else None
        out = ext.forward_sharded(qr, kr, vr, spec, prev_kv, next_kv)
        torch.cuda.synchronize()
        assert nat.last_kernel() == expected_window_kernel(spec, chunk, neighbours=True)
        check_close(out, want[:, r * chunk:(r + 1) * chunk], torch.bfloat16)


def test_neighbour_shards_argument_checks():
    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16, device=DEV)
    short = torch.zeros(1, 32, 2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="previous shard"):
        ext.forward_sharded(q, q, q, PatternSpec.causal_window(64), (short, short))
    with pytest.raises(RuntimeError, match="window patterns"):
        ext.forward_sharded(q, q, q, PatternSpec.longformer(4, 4, [0]), (q, q))
    with pytest.raises(RuntimeError):
        ext.forward_sharded(q.float(), q.float(), q.float(), PatternSpec.causal_window(64), (q.float(), q.float()))


# ---- block-sparse -----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_block_sparse_band_random(dtype):
    # cfg-3's layout (band of 4 + 2 random earlier blocks, causal diagonal) at reduced length
    S, block = 1024, 64
    rp, ci = band_random_block_layout(S // block, 4, 2, seed=5)
    spec = PatternSpec.block_sparse(block, rp, ci, causal=True)
    q, k, v = seeded_qkv(31, 2, S, 2, 64, dtype)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == ("rowwarp" if dtype == torch.float32 else "umma_block")   # tcgen05 / TMEM path
    check_close(got, oracle_out(q, k, v, spec), dtype)


def test_block_sparse_reference_tridiagonal_ragged():
    # the reference's own layout |bi-bj| <= 1 (sparse_attention.cpp:212-227), ragged last block
    for S, block, dtype in [(200, 64, torch.bfloat16), (300, 128, torch.bfloat16), (50, 4, torch.float32),
                            (37, 8, torch.bfloat16)]:
        rp, ci = tridiagonal_block_layout(S, block)
        spec = PatternSpec.block_sparse(block, rp, ci)
        q, k, v = seeded_qkv(32, 1, S, 2, 64, dtype)
        check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), dtype)


def test_block_sparse_empty_rows_give_zeros():
    spec = PatternSpec.block_sparse(64, [0, 1, 1, 3], [0, 0, 2])
    for dtype in (torch.float32, torch.bfloat16):
        q, k, v = seeded_qkv(33, 1, 192, 1, 64, dtype)
        got = run(spec, q, k, v)
        assert torch.count_nonzero(got[:, 64:128]) == 0
        check_close(got, oracle_out(q, k, v, spec), dtype)


def test_bigbird_and_random_block_layouts_vs_oracle():
    """BIG_BIRD (band + global blocks + seeded random blocks, global rows over everything) and
    block-granular RANDOM_SPARSE layouts, two-sided, on the tcgen05 kernel and on the fp32 kernel."""
    from ma_transformer_b200.patterns import bigbird_block_layout, random_block_layout
    S, block = 768, 64
    for rp, ci in (bigbird_block_layout(S // block, 3, 1, 2, seed=11), random_block_layout(S // block, 0.3, seed=12)):
        spec = PatternSpec.block_sparse(block, rp, ci)
        for dtype in (torch.bfloat16, torch.float32):
            q, k, v = seeded_qkv(36, 1, S, 2, 64, dtype)
            got = run(spec, q, k, v)
            assert nat.last_kernel() == ("rowwarp" if dtype == torch.float32 else "umma_block")
            check_close(got, oracle_out(q, k, v, spec), dtype)


# ---- Longformer -----------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_longformer_vs_oracle(dtype):
    g = torch.Generator().manual_seed(41)
    S = 512
    glob = torch.randperm(S, generator=g)[:8].sort().values.numpy()
    for spec in (PatternSpec.longformer(16, 16, glob), PatternSpec.longformer(64, 64, glob[:3]),
                 PatternSpec.longformer(2, 2, [0, 1]), PatternSpec.longformer(4, 0, [])):
        q, k, v = seeded_qkv(42, 2, S, 3, 64, dtype)
        check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_longformer_cfg4_shape_reduced_length(monkeypatch, dtype):
    # cfg-4's window (+-64), 32 seeded global positions, 12 heads, at a length the oracle finishes quickly
    g = torch.Generator().manual_seed(4)
    S = 4096
    glob = torch.randperm(S, generator=g)[:32].sort().values.numpy()
    spec = PatternSpec.longformer(64, 64, glob)
    q, k, v = seeded_qkv(43, 2, S, 12, 64, dtype)
    want = oracle_out(q, k, v, spec)
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "umma_longformer"      # window pass on the tcgen05 band kernel
    check_close(got, want, dtype)
    monkeypatch.setenv("MAT_WINDOW_KERNEL", "mma")      # and on the warp-level kernel
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "mma_longformer"
    check_close(got, want, dtype)
    monkeypatch.delenv("MAT_WINDOW_KERNEL")
    # many global positions: several gathered chunks and several tiles of global rows
    glob = torch.randperm(1500, generator=g)[:200].sort().values.numpy()
    spec = PatternSpec.longformer(10, 3, glob)
    q, k, v = seeded_qkv(44, 1, 1500, 2, 64, dtype)
    check_close(run(spec, q, k, v), oracle_out(q, k, v, spec), dtype)
    assert nat.last_kernel() == "mma_longformer"       # more than 32 global positions: the warp-level first pass


@pytest.mark.parametrize("left,right,n_glob,S,B,H", [
    (64, 64, 32, 1000, 2, 3),     # ragged against the 96-row items
    (16, 16, 1, 96, 1, 1),        # one item, one global position
    (0, 100, 7, 300, 1, 2),       # looking ahead
    (112, 16, 32, 2048, 1, 2),    # lopsided, the widest window the 224 band columns hold
    (3, 3, 5, 50, 1, 1),          # shorter than one item
    (17, 30, 9, 700, 1, 2),       # first tap off a multiple of 16: the band starts inside its first column group
    (64, 64, 32, 3000, 3, 5),     # folded: every lane of CTAs crosses batch boundaries (32 tiles, 29 lanes per head)
    (8, 8, 3, 60, 5, 2),          # folded: fewer tiles than lanes, so most CTAs only leave empty partials
    (32, 32, 4, 400, 1, 80),      # more heads than half the SMs: never folded
])
@pytest.mark.parametrize("fold", ["1", "0"])
def test_longformer_window_pass_on_band_kernel(monkeypatch, fold, left, right, n_glob, S, B, H):
    """The Longformer first pass on the persistent tcgen05 kernel: 96-row items, the keys at the global positions
    as 32 extra columns (de-duplicated against each row's window).  The rows AT the global positions ride along
    as rows 96..127 of every query tile and are merged over the CTAs (fold = 1, the default), or are finished
    by the separate split pass (fold = 0)."""
    monkeypatch.setenv("MAT_LONGFORMER_FOLD", fold)
    g = torch.Generator().manual_seed(46)
    glob = torch.randperm(S, generator=g)[:n_glob].sort().values.numpy()
    spec = PatternSpec.longformer(left, right, glob)
    for dtype in (torch.bfloat16, torch.float16):
        q, k, v = seeded_qkv(47, B, S, H, 64, dtype)
        got = run(spec, q, k, v)
        assert nat.last_kernel() == "umma_longformer"
        check_close(got, oracle_out(q, k, v, spec), dtype)


# ---- index sets, recovered from the kernels themselves -----------------------------------------

def _attended_sets(spec, S, dtype, D):
    """q = 0 gives uniform weights; V = identity rows make output[i, j] > 0 exactly
    for the keys row i attended."""
    q = torch.zeros(1, S, 1, D, dtype=dtype)
    k = torch.zeros(1, S, 1, D, dtype=dtype)
    v = torch.zeros(1, S, 1, D, dtype=dtype)
    v[0, torch.arange(S), 0, torch.arange(S)] = 1.0
    out = run(spec, q, k, v)[0, :, 0, :S].float().cpu().numpy()
    return [np.nonzero(out[i] > 0)[0].astype(np.int64) for i in range(S)], out


@pytest.mark.parametrize("dtype,D", [(torch.float32, 48), (torch.bfloat16, 64)])
def test_index_sets_bit_exact(dtype, D, oracle):
    S = 48
    rp, ci = band_random_block_layout(S // 8, 2, 1, seed=1)
    rp64, ci64 = tridiagonal_block_layout(64, 64)
    specs = [PatternSpec.sliding_window(3), PatternSpec.causal_window(5), PatternSpec.causal_window(4, dilation=3),
             PatternSpec(left=0, right=7), PatternSpec.block_sparse(8, rp, ci, causal=True),
             PatternSpec.block_sparse(64, rp64, ci64, causal=True),
             PatternSpec.longformer(2, 3, [5, 40, 17]), PatternSpec.sliding_window(500)]
    for spec in specs:
        sets, out = _attended_sets(spec, S, dtype, D)
        for i in range(S):
            want = oracle.rowset(to_oracle(spec), S, i)
            assert np.array_equal(sets[i], want), (spec, i)
            assert np.array_equal(spec.rowset(S, i), want)
            if len(want):  # uniform weights: every attended key carries 1/n
                assert abs(out[i, want[0]] - 1.0 / len(want)) < (1e-6 if dtype == torch.float32 else 4e-3)


# ---- reference extension behaviour ---------------------------------------------------------------

def test_extension_call_contract():
    q, k, v = (t.to(DEV) for t in seeded_qkv(51, 2, 33, 2, 16))
    # window 0 = self only: output equals V (tests/python/test_cuda_sparse_kernel_launch.py W=0)
    assert torch.allclose(ext.forward(q, k, v, 0), v, atol=1e-6)
    # window beyond S clamps to dense
    dense = ext.dense_forward(q, k, v, False)
    assert torch.allclose(ext.forward(q, k, v, 10_000), dense, atol=1e-6)
    np.testing.assert_allclose(dense.cpu().numpy(), mt.pytorch_dense_attention(q.cpu(), k.cpu(), v.cpu()).numpy(),
                               rtol=1e-4, atol=1e-5)
    causal = ext.dense_forward(q, k, v, True)
    np.testing.assert_allclose(causal.cpu().numpy(),
                               mt.pytorch_dense_attention(q.cpu(), k.cpu(), v.cpu(), True).numpy(), rtol=1e-4, atol=1e-5)
    # non-contiguous input raises RuntimeError (tests/integration/test_cuda_extensive.py:196-204)
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.forward(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), 4)
    with pytest.raises(RuntimeError, match="same shape"):
        ext.forward(q, k[:, :5].contiguous(), v, 4)
    with pytest.raises(RuntimeError):
        ext.forward(q, k.double(), v, 4)
    # inputs are never written
    q0 = q.clone()
    ext.forward(q, k, v, 4)
    assert torch.equal(q, q0)


def test_module_surface_on_gpu():
    q, k, v = (t.to(DEV) for t in seeded_qkv(52, 2, 40, 4, 32))
    attn = mt.MACoreAttention(sparse=True, window_size=8, fallback_training=False).eval()
    want = oracle_out(q.cpu(), k.cpu(), v.cpu(), PatternSpec.sliding_window(8))
    check_close(attn(q, k, v), want, torch.float32)
    # non-contiguous inputs are made contiguous by the bridge (test_cuda_extensive.py:95-115)
    qt = q.transpose(1, 2).contiguous().transpose(1, 2)
    check_close(attn(qt, k, v), want, torch.float32)
    # 16-bit inputs keep their dtype and now run natively (test_cuda_extensive.py:118-136)
    for dt in (torch.bfloat16, torch.float16):
        y = attn(q.to(dt), k.to(dt), v.to(dt))
        assert y.dtype == dt
        assert (y.float().cpu() - torch.from_numpy(want)).abs().max() < 3e-2
    # [B,S,D] layer, eval mode
    layer = mt.SparseAttention(window_size=3).eval()
    x = torch.randn(2, 50, 24, device=DEV)
    y = layer(x, x, x)
    want3 = oracle_out(x.cpu().unsqueeze(2), x.cpu().unsqueeze(2), x.cpu().unsqueeze(2), PatternSpec.sliding_window(3))
    check_close(y.unsqueeze(2), want3, torch.float32)
    # backward through the native forward (tests/python/test_cuda_backward.py)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    attn(qg, kg, vg).square().sum().backward()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    mt.pytorch_sparse_attention(qr, kr, vr, 8).square().sum().backward()
    for a, b in ((qg, qr), (kg, kr), (vg, vr)):
        assert torch.allclose(a.grad, b.grad, atol=2e-3)


# ---- host-buffer entry point ------------------------------------------------------------------------

@pytest.mark.parametrize("spec", [PatternSpec.causal_window(64), PatternSpec.sliding_window(30),
                                  PatternSpec.causal_window(8, dilation=2)], ids=["causal64", "pm30", "dil2"])
def test_host_entry_point_equals_device_entry_point(spec):
    # long enough for several pipeline chunks (an eighth of a batch item each: 2.5 MB)
    q, k, v = seeded_qkv(61, 2, 20000, 8, 64, torch.bfloat16)
    qp, kp, vp = (t.pin_memory() for t in (q, k, v))
    got = ext.forward_host(qp, kp, vp, spec)
    want = run(spec, q, k, v).cpu()
    assert torch.equal(got, want)


@pytest.mark.parametrize("spec", [PatternSpec.causal_window(11), PatternSpec.sliding_window(5),
                                  PatternSpec.causal_window(64), PatternSpec(left=3, right=70)],
                         ids=["causal11", "pm5", "causal64", "l3r70"])
def test_host_entry_point_never_reads_rows_that_have_not_landed(spec):
    """The tiled kernels stage whole groups of keys; the rows of a group that lie in a chunk whose copy has not
    been waited for must read as zeros, not as whatever the staging memory held.  The staging buffer is filled
    with NaN patterns first: a single stale row under a zero weight would turn an output row into NaN."""
    q, k, v = seeded_qkv(64, 1, 24000, 8, 64, torch.bfloat16)
    qp, kp, vp = (t.pin_memory() for t in (q, k, v))
    s = spec.device_struct(DEV)
    nbytes = nat.lib.mat_sparse_attn_host_staging_bytes(1, 24000, 8, 64, nat.MAT_BF16, s)
    want = run(spec, q, k, v).cpu()
    for _ in range(3):   # the race, if present, is a matter of timing: a few tries
        staging = ext._workspace(torch.device(DEV), nbytes)
        staging.view(torch.int16).fill_(0x7FC0)        # bf16 NaN everywhere
        torch.cuda.synchronize()
        got = ext.forward_host(qp, kp, vp, spec)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)


def test_host_entry_point_general_patterns_and_module():
    S = 1024
    rp, ci = band_random_block_layout(S // 64, 4, 2, seed=2)
    for spec, dtype in [(PatternSpec.block_sparse(64, rp, ci, causal=True), torch.bfloat16),
                        (PatternSpec.longformer(8, 8, [3, 500]), torch.float32)]:
        q, k, v = seeded_qkv(62, 1, S, 2, 64, dtype)
        check_close(ext.forward_host(q, k, v, spec), oracle_out(q, k, v, spec), dtype)
    # CPU tensors through the module: computed on the GPU, returned on the CPU
    q, k, v = seeded_qkv(63, 1, 64, 2, 16)
    attn = mt.MACoreAttention(sparse=True, window_size=4).eval()
    y = attn(q, k, v)
    assert y.device.type == "cpu"
    check_close(y, oracle_out(q, k, v, PatternSpec.sliding_window(4)), torch.float32)


# ---- the full-size configurations: size-independent properties ---------------------------------------------------

def test_cfg2_full_size_properties():
    B, S, H, D = 1, 65536, 8, 64
    spec = PatternSpec.causal_window(64)
    q, k, v = (t.to(DEV) for t in seeded_qkv(2, B, S, H, D, torch.bfloat16, scale=0.5))
    out = ext.forward_pattern(q, k, v, spec)
    assert nat.last_kernel() == "umma_band"
    assert torch.isfinite(out.float()).all()
    # (a) linear in V: doubling V doubles the output exactly (power of two)
    assert torch.equal(ext.forward_pattern(q, k, v * 2, spec), out * 2)
    # (b) constant V rows come back unchanged (weights sum to one)
    vc = torch.full_like(v, 0.75)
    assert (ext.forward_pattern(q, k, vc, spec).float() - 0.75).abs().max() <= 0.75 * 2 ** -7
    # (c) deterministic
    assert torch.equal(ext.forward_pattern(q, k, v, spec), out)
    # (d) sampled row blocks against the oracle, each with its 63-row halo
    for a in (0, 64, 4096 - 32, 32768, S - 128):
        lo = max(0, a - 63)
        sl = spec.shifted(a - lo)
        want = oracle_out(q[:, a:a + 128].cpu(), k[:, lo:a + 128].cpu(), v[:, lo:a + 128].cpu(), sl)
        check_close(out[:, a:a + 128], want, torch.bfloat16)


def test_device_status_word_is_clear():
    torch.cuda.synchronize()
    assert nat.device_status() == 0


# ---- backward kernels (next row after the forward) -----------------------------------------------------

@pytest.mark.parametrize("B,S,H,D", [(2, 33, 2, 16), (1, 7, 1, 5), (2, 65, 3, 32), (1, 128, 2, 64)])
@pytest.mark.parametrize("W", [0, 1, 4, 8, 200])
def test_backward_matches_autograd_of_reference_oracle(B, S, H, D, W):
    """tests/python/test_cuda_backward.py:75-101 and test_cuda_extensive.py:168-193 compare the extension's
    backward with autograd through the python oracle at 2e-3."""
    q, k, v = (t.to(DEV) for t in seeded_qkv(81, B, S, H, D))
    go = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(82)).to(DEV)
    dq, dk, dv = ext.backward(q, k, v, go, W)
    assert nat.last_kernel() == ("bwd_f32_mma" if D % 4 == 0 else "bwd_window")   # multiples of 4: tensor cores
    qr, kr, vr = (t.detach().cpu().double().requires_grad_(True) for t in (q, k, v))
    mt.pytorch_sparse_attention(qr, kr, vr, W).backward(go.cpu().double())
    for got, ref in ((dq, qr), (dk, kr), (dv, vr)):
        assert (got.cpu().double() - ref.grad).abs().max() < 2e-5 * max(1.0, float(ref.grad.abs().max()))


@pytest.mark.parametrize("D", [8, 16, 32, 40, 48, 64, 80, 96, 128, 256, 512])
@pytest.mark.parametrize("B,S,H,left,right,dil", [
    (1, 512, 2, 63, 0, 1), (2, 200, 3, 32, 32, 1), (1, 33, 1, 8, 8, 1), (1, 130, 2, 10, 3, 1), (1, 70, 1, 40, 41, 1),
    (1, 300, 2, 64, 64, 1), (1, 256, 2, 15, 0, 2), (2, 96, 1, 5, 5, 3), (1, 1000, 2, 1000, 1000, 1), (1, 1000, 1, 1000, 0, 1),
    (1, 700, 2, 300, 100, 1),
])
@pytest.mark.parametrize("walk", ["default", "chunks", "recompute"])
def test_fp32_backward_on_tensor_cores(monkeypatch, walk, B, S, H, left, right, dil, D):
    """The fp32 backward as three TF32 products per product (head widths 32 and 64): against autograd in fp64
    through a dense masked softmax at the fp32 kernels' bar (2e-5 of the gradient's scale), windows narrow, wide,
    dilated, dense and causal dense, ragged lengths; and against the warp-level fp32 kernels.  Narrow windows
    default to the walk in which every warp takes its own column range; MAT_BWD_F32_WALK=chunks keeps them on
    the 64-column chunks the wide ones use.  Head widths 128 and 256 (one head of width model_dim is what the
    reference's layer passes) run the same passes 64 columns at a time."""
    if walk != "default":   # ("recompute": one-pass walks of a 64-wide head on the kernel that recomputes S and dP)
        if D > 64 or (walk == "recompute" and (D != 64 or left + right + 16 > 144)):
            pytest.skip("no such variant for this shape")
        monkeypatch.setenv("MAT_BWD_F32_WALK", walk)
    spec = PatternSpec(left=left, right=right, dilation=dil)
    q, k, v = seeded_qkv(87, B, S, H, D, torch.float32)
    go = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(88))
    args = tuple(t.to(DEV) for t in (q, k, v, go))
    got = ext.backward_pattern(*args, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "bwd_f32_mma" and nat.device_status() == 0
    ref = [t.double().requires_grad_(True) for t in (q, k, v)]
    masked_dense_attention(*ref, left, right, dil).backward(go.double())
    for name, a, r in zip(("dQ", "dK", "dV"), got, ref):
        err = float((a.cpu().double() - r.grad).abs().max())
        assert err <= 2e-5 * max(1.0, float(r.grad.abs().max())), f"{name} vs fp64 autograd: {err}"
    monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
    want = ext.backward_pattern(*args, spec)
    assert nat.last_kernel() == "bwd_window"
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert float((a - b).abs().max()) <= 2e-5 * max(1.0, float(b.abs().max())), name
    monkeypatch.delenv("MAT_BWD_KERNEL")
    again = ext.backward_pattern(*args, spec)
    for a, b in zip(got, again):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [8, 40, 144, 192, 256, 512])
@pytest.mark.parametrize("B,S,H,left,right,dil", [
    (1, 512, 2, 63, 0, 1), (2, 200, 2, 32, 32, 1), (1, 33, 1, 8, 8, 1), (1, 70, 1, 40, 41, 1), (1, 300, 2, 64, 64, 1),
    (1, 256, 1, 15, 0, 2), (1, 130, 1, 0, 100, 1),
])
def test_16bit_backward_for_wide_heads(monkeypatch, dtype, D, B, S, H, left, right, dil):
    """The 16-bit backward for one wide head (192 to 512 columns; the reference's layer passes D = model_dim) with a
    window of at most 144 taps: the tensor-core passes with the head dimension 64 columns at a time, against autograd
    in fp64 through a dense masked softmax on the same rounded inputs and against the one-warp-per-row kernels."""
    spec = PatternSpec(left=left, right=right, dilation=dil)
    q, k, v = seeded_qkv(91, B, S, H, D, dtype)
    go = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(92)).to(dtype)
    args = tuple(t.to(DEV) for t in (q, k, v, go))
    got = ext.backward_pattern(*args, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "bwd_d_mma" and nat.device_status() == 0
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    ref = [t.double().requires_grad_(True) for t in (q, k, v)]
    masked_dense_attention(*ref, left, right, dil).backward(go.double())
    for name, a, r in zip(("dQ", "dK", "dV"), got, ref):
        err = float((a.cpu().double() - r.grad).abs().max())
        assert err <= tol * max(1.0, float(r.grad.abs().max())), f"{name} vs fp64 autograd: {err}"
    if S // dil >= 200:   # (a window clamps to the sequence, so a short sequence makes every window narrow)
        # walks of more than two passes keep their sums in fp32 copies of the outputs' shape (the workspace)
        for wl, wr in ((100, 100), (S, S)):
            wide = PatternSpec(left=wl, right=wr, dilation=dil)
            gw = ext.backward_pattern(*args, wide)
            assert nat.last_kernel() == "bwd_d_mma" and nat.device_status() == 0
            refw = [t.double().requires_grad_(True) for t in (q, k, v)]
            masked_dense_attention(*refw, wl, wr, dil).backward(go.double())
            for name, a, r in zip(("dQ", "dK", "dV"), gw, refw):
                err = float((a.cpu().double() - r.grad).abs().max())
                assert err <= tol * max(1.0, float(r.grad.abs().max())), f"wide window {name} vs fp64 autograd: {err}"
    monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
    want = ext.backward_pattern(*args, spec)
    assert nat.last_kernel() == "bwd_window"
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert float((a.float() - b.float()).abs().max()) <= tol * max(1.0, float(b.float().abs().max())), name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [16, 32, 96, 128])
@pytest.mark.parametrize("B,S,H,left,right,dil", [
    (1, 512, 2, 63, 0, 1), (2, 200, 3, 32, 32, 1), (1, 33, 1, 8, 8, 1), (1, 70, 1, 40, 41, 1), (1, 300, 2, 64, 64, 1),
    (1, 256, 2, 15, 0, 2), (1, 600, 2, 600, 600, 1), (1, 600, 1, 600, 0, 1),
])
@pytest.mark.parametrize("walk", ["default", "chunks", "whole"])
def test_16bit_backward_for_other_head_widths(monkeypatch, walk, dtype, D, B, S, H, left, right, dil):
    """The 16-bit backward for head widths that are multiples of 16 up to 128 other than 64 (the reference's
    kernel takes any width: src/cuda/sparse_attention_kernel.cu:265-346) on the warp-level tensor-core kernels:
    against autograd in fp64 through a dense masked softmax on the same rounded inputs, and against the
    one-warp-per-row kernels.  Narrow windows default to the walk in which every warp takes its own column range;
    MAT_BWD_D_WALK=chunks keeps them on the 64-column chunks the wide ones use."""
    if walk != "default":   # ("whole": a head of 128 columns in one piece where the default takes it 64 columns at a time)
        if walk == "whole" and (D != 128 or not 80 < left + right + 16 <= 144):
            pytest.skip("no such variant for this shape")
        monkeypatch.setenv("MAT_BWD_D_WALK", walk)
    spec = PatternSpec(left=left, right=right, dilation=dil)
    q, k, v = seeded_qkv(89, B, S, H, D, dtype)
    go = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(90)).to(dtype)
    args = tuple(t.to(DEV) for t in (q, k, v, go))
    got = ext.backward_pattern(*args, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "bwd_d_mma" and nat.device_status() == 0
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    ref = [t.double().requires_grad_(True) for t in (q, k, v)]
    masked_dense_attention(*ref, left, right, dil).backward(go.double())
    for name, a, r in zip(("dQ", "dK", "dV"), got, ref):
        err = float((a.cpu().double() - r.grad).abs().max())
        assert err <= tol * max(1.0, float(r.grad.abs().max())), f"{name} vs fp64 autograd: {err}"
    monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
    want = ext.backward_pattern(*args, spec)
    assert nat.last_kernel() == "bwd_window"
    for name, a, b in zip(("dQ", "dK", "dV"), got, want):
        assert float((a.float() - b.float()).abs().max()) <= tol * max(1.0, float(b.float().abs().max())), name


@pytest.mark.parametrize("causal", [False, True])
def test_dense_backward_and_custom_windows(causal):
    q, k, v = (t.to(DEV) for t in seeded_qkv(83, 2, 40, 2, 24))
    go = torch.randn(2, 40, 2, 24, generator=torch.Generator().manual_seed(84)).to(DEV)
    dq, dk, dv = ext.dense_backward(q, k, v, go, causal)
    qr, kr, vr = (t.detach().cpu().double().requires_grad_(True) for t in (q, k, v))
    mt.pytorch_dense_attention(qr, kr, vr, causal).backward(go.cpu().double())
    for got, ref in ((dq, qr), (dk, kr), (dv, vr)):
        assert (got.cpu().double() - ref.grad).abs().max() < 2e-5 * max(1.0, float(ref.grad.abs().max()))
    # a dilated causal window through the module (bf16): gradients flow and match the fp32 kernels loosely
    spec = PatternSpec.causal_window(8, dilation=2)
    attn = mt.MACoreAttention(sparse=True, window_size=8, pattern=spec, fallback_training=False)
    qb, kb, vb = (t.to(torch.bfloat16).requires_grad_(True) for t in seeded_qkv(85, 1, 64, 2, 64))
    qb, kb, vb = (t.detach().to(DEV).requires_grad_(True) for t in (qb, kb, vb))
    attn(qb, kb, vb).float().square().sum().backward()
    q32, k32, v32 = (t.detach().float().requires_grad_(True) for t in (qb, kb, vb))
    attn(q32, k32, v32).square().sum().backward()
    for a16, a32 in ((qb, q32), (kb, k32), (vb, v32)):
        assert torch.isfinite(a16.grad.float()).all()
        assert (a16.grad.float() - a32.grad).abs().max() < 0.06 * max(1.0, float(a32.grad.abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,left,right,dil", [
    (1, 512, 2, 63, 0, 1),      # 64 causal taps: the headline window
    (2, 200, 3, 32, 32, 1),     # two-sided, ragged last tile
    (1, 33, 1, 8, 8, 1),        # shorter than one tile
    (1, 130, 2, 10, 3, 1),      # lopsided
    (1, 257, 1, 0, 0, 1),       # self only
    (1, 64, 2, 0, 64, 1),       # looking ahead only
    (1, 384, 2, 63, 0, 2),      # dilated causal taps i - 2k (the order-book model's window)
    (1, 96, 1, 5, 5, 3),        # dilated, two-sided
    (1, 30, 2, 200, 200, 1),    # reaches past both ends: clamps to the sequence
    (1, 512, 2, 64, 64, 1),     # the reference's default window_size=64 (+-64): the two-sweep rows pass
    (1, 300, 2, 127, 0, 1),     # 128 causal taps, ragged last tile
    (2, 200, 1, 100, 20, 1),    # lopsided, wide
    (1, 256, 2, 64, 64, 2),     # wide and dilated
    (1, 70, 1, 40, 41, 1),      # just past 64 taps on a sequence barely longer than a tile
    (1, 512, 2, 512, 512, 1),   # dense (the reference's dense_backward): the band streamed in 64-column chunks
    (1, 300, 2, 300, 0, 1),     # causal dense, ragged last tile
    (2, 200, 1, 150, 20, 1),    # wide and lopsided
    (1, 1024, 1, 200, 0, 1),    # 201 causal taps: chunks skipped on both sides of the band
    (1, 512, 2, 100, 100, 2),   # wide, two-sided and dilated
    (1, 129, 1, 65, 64, 1),     # one tap past the resident-band kernels
])
def test_tensor_core_backward_matches_fp64_autograd_and_fp32_math_kernels(monkeypatch, dtype, B, S, H, left, right, dil):
    """The mma backward (16-bit, D = 64; band resident in shared memory up to 128 taps between the two sides,
    streamed beyond) held to an independent reference: autograd in fp64 through a dense masked softmax on the
    same 16-bit-rounded inputs (the bar of tests/python/test_cuda_backward.py:75-101 and
    tests/integration/test_cuda_extensive.py:168-193, at the 16-bit tolerance).  The warp-level kernels,
    which compute in fp32 from the same inputs, are a second, tighter comparison."""
    spec = PatternSpec(left=left, right=right, dilation=dil)
    q, k, v = seeded_qkv(91, B, S, H, 64, dtype)
    go = torch.randn(B, S, H, 64, generator=torch.Generator().manual_seed(92)).to(dtype)
    qd, kd, vd, god = (t.to(DEV) for t in (q, k, v, go))
    got = ext.backward_pattern(qd, kd, vd, god, spec)
    torch.cuda.synchronize()
    taps = min(left, S // dil - 1) + min(right, S // dil - 1)
    assert nat.last_kernel() == ("bwd_window_mma" if taps <= 128 else "bwd_stream_mma")
    tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
    # (1) fp64 autograd through the dense masked reference
    ref = [t.double().requires_grad_(True) for t in (q, k, v)]
    masked_dense_attention(*ref, left, right, dil).backward(go.double())
    for name, a, r in zip(("dQ", "dK", "dV"), got, ref):
        a = a.cpu().double()
        assert torch.isfinite(a).all(), name
        err = float((a - r.grad).abs().max())
        assert err <= tol * max(1.0, float(r.grad.abs().max())), f"{name} vs fp64 autograd: {err}"
    # (2) the fp32-math warp-level kernels
    monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
    want = ext.backward_pattern(qd, kd, vd, god, spec)
    torch.cuda.synchronize()
    assert nat.last_kernel() == "bwd_window"
    for name, a, b, r in zip(("dQ", "dK", "dV"), got, want, ref):
        a, b = a.float(), b.float()
        err = float((a - b).abs().max())
        assert err <= tol * max(1.0, float(b.abs().max())), f"{name}: {err}"
        # and those kernels against the same fp64 reference, at the rounding of their 16-bit outputs
        errw = float((b.cpu().double() - r.grad).abs().max())
        assert errw <= (2 ** -7 if dtype == torch.bfloat16 else 2 ** -10) * max(1.0, float(r.grad.abs().max())), name
    # deterministic: a second run gives the same bits
    monkeypatch.delenv("MAT_BWD_KERNEL")
    again = ext.backward_pattern(qd, kd, vd, god, spec)
    for a, b in zip(got, again):
        assert torch.equal(a, b)


def _general_backward_cases():
    rp, ci = band_random_block_layout(5, 2, 2, seed=3)            # 5 blocks of 64: band of 2 + 2 random earlier ones
    rp32, ci32 = band_random_block_layout(9, 3, 1, seed=4)        # 9 blocks of 32
    full_rp, full_ci = np.arange(0, 17, 4), np.tile(np.arange(4), 4)   # every block: dense through a layout
    return [
        ("block64-causal", PatternSpec.block_sparse(64, rp, ci, causal=True), 320),
        ("block64-ragged", PatternSpec.block_sparse(64, rp, ci, causal=True), 300),      # the last block is partly filled
        ("block32", PatternSpec.block_sparse(32, rp32, ci32, causal=False), 288),
        ("block64-dense", PatternSpec.block_sparse(64, full_rp, full_ci, causal=False), 256),
        ("longformer", PatternSpec.longformer(8, 8, [0, 17, 100, 199]), 200),
        ("longformer-lopsided", PatternSpec.longformer(20, 3, [5, 6, 7, 150]), 211),
        ("longformer-no-globals", PatternSpec.longformer(4, 0, []), 70),
        ("longformer-cfg4-like", PatternSpec.longformer(64, 64, list(range(3, 600, 19))), 600),   # 32 globals, several tiles
        ("longformer-70-globals", PatternSpec.longformer(5, 5, list(range(0, 140, 2))), 150),     # more than one chunk holds
    ]


@pytest.mark.parametrize("name,spec,S", _general_backward_cases(), ids=[c[0] for c in _general_backward_cases()])
@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 64), (torch.float16, 64), (torch.float32, 40)])
def test_backward_of_block_layouts_and_longformer_against_fp64_autograd(monkeypatch, name, spec, S, dtype, D):
    """dQ, dK, dV of block layouts and of the Longformer pattern (the reference's interface has no backward for
    them: src/csrc/attention_interface.hpp:14-52) against autograd in fp64 through a dense softmax masked with
    the pattern's own index sets; and through the autograd function of the module."""
    B, H = 2, 2
    q, k, v = seeded_qkv(97, B, S, H, D, dtype)
    go = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(98)).to(dtype)
    got = ext.backward_pattern(q.to(DEV), k.to(DEV), v.to(DEV), go.to(DEV), spec)
    torch.cuda.synchronize()
    # block layouts whose blocks are multiples of 64 run on the streamed tensor-core kernels (16-bit, D = 64)
    # and so does the Longformer pattern with 1 to 64 global positions (none: a plain window)
    n_glob = len(spec.global_idx) if spec.kind == 2 else 0
    sixteen = dtype != torch.float32 and D == 64
    on_mma = sixteen and ((spec.kind == 1 and spec.block % 64 == 0) or (spec.kind == 2 and n_glob <= 64))
    want_kernel = "bwd_general"
    if on_mma:
        want_kernel = "bwd_block_mma" if spec.kind == 1 else ("bwd_longformer_mma" if n_glob else "bwd_window_mma")
    assert nat.last_kernel() == want_kernel and nat.device_status() == 0
    keep = pattern_mask(spec, S)
    ref = [t.double().requires_grad_(True) for t in (q, k, v)]
    masked_attention_with(*ref, keep).backward(go.double())
    # fp32 math with 16-bit outputs rounded once; the tensor-core kernels also round P and dS to the input type
    tol = 1e-5 if dtype == torch.float32 else (2e-2 if dtype == torch.bfloat16 else 5e-3) if on_mma else 2 ** -7
    for nm, a, r in zip(("dQ", "dK", "dV"), got, ref):
        a = a.cpu().double()
        assert torch.isfinite(a).all(), nm
        err = float((a - r.grad).abs().max())
        assert err <= tol * max(1.0, float(r.grad.abs().max())), f"{name} {nm}: {err}"
    # the same gradients through torch.autograd and the module's function (forward on the native kernels too)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = mt.MACoreAttentionFunction.apply(qd, kd, vd, True, 0, False, spec)
    out.backward(go.to(DEV))
    for a, b in zip(got, (qd.grad, kd.grad, vd.grad)):
        assert torch.equal(a, b)
    if on_mma:   # and the fp32-math kernels on the same inputs
        monkeypatch.setenv("MAT_BWD_KERNEL", "warp")
        want = ext.backward_pattern(q.to(DEV), k.to(DEV), v.to(DEV), go.to(DEV), spec)
        assert nat.last_kernel() == "bwd_general"
        for nm, a, b in zip(("dQ", "dK", "dV"), got, want):
            err = float((a.float() - b.float()).abs().max())
            assert err <= tol * max(1.0, float(b.float().abs().max())), f"{name} {nm} vs warp-level: {err}"


def test_backward_of_unaligned_tensors_stays_on_warp_kernels():
    """Tensors that do not start on a 16-byte boundary cannot be moved by TMA: the call still works."""
    flat = [torch.randn(1 * 128 * 2 * 64 + 4, generator=torch.Generator().manual_seed(95 + i)).to(torch.bfloat16).to(DEV)
            for i in range(4)]
    q, k, v, go = (f[4:].view(1, 128, 2, 64) for f in flat)          # 8 bytes past an aligned address
    got = ext.backward_pattern(q, k, v, go, PatternSpec.causal_window(16))
    assert nat.last_kernel() == "bwd_window"
    want = ext.backward_pattern(q.clone(), k.clone(), v.clone(), go.clone(), PatternSpec.causal_window(16))
    assert nat.last_kernel() == "bwd_window_mma"
    for a, b in zip(got, want):
        assert (a.float() - b.float()).abs().max() <= 2e-2 * max(1.0, float(b.float().abs().max()))


def test_tensor_core_backward_against_fp64_autograd():
    """Same bar as the fp32 kernels' test, at the 16-bit tolerance: autograd in fp64 through the reference's
    python oracle (src/layers/ma_core_bridge.py:224-247) on the bf16-rounded inputs."""
    q, k, v = seeded_qkv(93, 2, 192, 2, 64, torch.bfloat16)
    go = torch.randn(2, 192, 2, 64, generator=torch.Generator().manual_seed(94)).to(torch.bfloat16)
    dq, dk, dv = ext.backward(q.to(DEV), k.to(DEV), v.to(DEV), go.to(DEV), 16)
    assert nat.last_kernel() == "bwd_window_mma"
    qr, kr, vr = (t.double().requires_grad_(True) for t in (q, k, v))
    mt.pytorch_sparse_attention(qr, kr, vr, 16).backward(go.double())
    for got, ref in ((dq, qr), (dk, kr), (dv, vr)):
        assert (got.cpu().double() - ref.grad).abs().max() < 2e-2 * max(1.0, float(ref.grad.abs().max()))


def test_block_layout_on_warp_level_kernel_too(monkeypatch):
    """MAT_BLOCK_KERNEL=mma keeps block layouts on the warp-level ring kernel (debugging aid);
    both kernels must agree with the oracle."""
    S, block = 512, 64
    rp, ci = band_random_block_layout(S // block, 4, 2, seed=9)
    spec = PatternSpec.block_sparse(block, rp, ci, causal=True)
    q, k, v = seeded_qkv(34, 1, S, 2, 64, torch.bfloat16)
    want = oracle_out(q, k, v, spec)
    monkeypatch.setenv("MAT_BLOCK_KERNEL", "mma")
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "mma_block"
    check_close(got, want, torch.bfloat16)
    monkeypatch.delenv("MAT_BLOCK_KERNEL")
    got = run(spec, q, k, v)
    assert nat.last_kernel() == "umma_block"
    check_close(got, want, torch.bfloat16)


@pytest.mark.parametrize("tiles", ["1", "2"])
def test_tcgen05_tiles_per_cta(monkeypatch, tiles):
    """The tcgen05 pipeline with one 128-row tile per CTA and with two tiles sharing the K/V stages
    (MAT_UMMA_TILES overrides the size-based choice): block layouts whose four 64-row halves hold
    different blocks, ragged ends, block edges of 64, 128 and 256, dense and causal dense."""
    monkeypatch.setenv("MAT_UMMA_TILES", tiles)
    for S, block, seed in [(1024, 64, 5), (832, 64, 6), (1280, 128, 7), (1536, 256, 8)]:
        rp, ci = band_random_block_layout((S + block - 1) // block, 3, 2, seed=seed)
        spec = PatternSpec.block_sparse(block, rp, ci, causal=True)
        for dtype in (torch.bfloat16, torch.float16):
            q, k, v = seeded_qkv(40 + seed, 1, S, 2, 64, dtype)
            got = run(spec, q, k, v)
            assert nat.last_kernel() == "umma_block"
            check_close(got, oracle_out(q, k, v, spec), dtype)
    spec = PatternSpec.block_sparse(64, [0, 1, 1, 3, 4, 4, 6], [0, 0, 2, 1, 0, 5])   # empty rows among the four halves
    q, k, v = seeded_qkv(49, 1, 384, 1, 64, torch.bfloat16)
    got = run(spec, q, k, v)
    assert torch.count_nonzero(got[:, 64:128]) == 0 and torch.count_nonzero(got[:, 256:320]) == 0
    check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)
    for S, causal in [(1024, False), (896, True), (1000, True), (384, False)]:
        q, k, v = seeded_qkv(50, 1, S, 2, 64, torch.bfloat16)
        got = ext.dense_forward(q.to(DEV), k.to(DEV), v.to(DEV), causal)
        assert nat.last_kernel() == "umma_dense"
        check_close(got, oracle_out(q, k, v, PatternSpec(left=S, right=0 if causal else S)), torch.bfloat16)


def test_random_windows_and_offsets_fuzz():
    """Seeded sweep over window shapes, dilations, lengths and shard offsets on the tiled kernel."""
    rng = np.random.default_rng(77)
    for _ in range(40):
        dil = int(rng.choice([1, 1, 2, 3]))
        left, right = int(rng.integers(0, 90)), int(rng.integers(0, 90))
        if rng.random() < 0.4:
            right = 0
        Sq = int(rng.integers(1, 12)) * 16 * dil
        off = int(rng.integers(0, 6)) * dil * int(rng.choice([1, 16]))
        tail = int(rng.integers(0, 5)) * dil
        spec = PatternSpec(left=left, right=right, dilation=dil).shifted(off)
        q, k, v = seeded_qkv(int(rng.integers(1 << 30)), 1, Sq, 2, 64, torch.bfloat16, Skv=Sq + off + tail)
        got = run(spec, q, k, v)
        assert nat.last_kernel() == expected_window_kernel(spec, Sq + off + tail), (left, right, dil, Sq, off, tail)
        check_close(got, oracle_out(q, k, v, spec), torch.bfloat16)


def test_longformer_over_sequence_shards_building_blocks():
    """Longformer with the sequence cut into 4 shards, emulated on one GPU: the per-shard window +
    global-key pass (halo rows read from the neighbour shards' tensors), the partials of all global
    queries over each shard's keys, and the merge by the shard that owns a token; the two
    all-gathers are a torch.cat here.  Must equal the unsharded oracle."""
    from ma_transformer_b200 import longformer_sharded as ls
    g = torch.Generator().manual_seed(5)
    S, P, H = 2048, 4, 3
    glob = torch.randperm(S, generator=g)[:20].sort().values
    spec = PatternSpec.longformer(40, 24, glob.numpy())
    q, k, v = seeded_qkv(91, 2, S, H, 64, torch.bfloat16)
    want = oracle_out(q, k, v, spec)
    rows = S // P
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    chunks = [tuple(t[:, r * rows:(r + 1) * rows].contiguous() for t in (qd, kd, vd)) for r in range(P)]
    gd = glob.to(DEV)
    qg, kg, vg = (t[:, gd].contiguous() for t in (qd, kd, vd))                      # collective 1
    partials = torch.stack([ls.global_rows_partial(qg, c[1], c[2]) for c in chunks])    # collective 2
    for r in range(P):
        cq, ck, cv = chunks[r]
        g_pos = (gd - r * rows).contiguous()
        out = ls.shard_pass1(cq, ck, cv, 40, 24, kg, vg, g_pos,
                             chunks[r - 1][1:] if r > 0 else None, chunks[r + 1][1:] if r < P - 1 else None)
        own = ((glob >= r * rows) & (glob < (r + 1) * rows)).nonzero().flatten()
        if len(own):
            ls.global_rows_merge(partials, out, g_pos, int(own[0]), len(own))
        torch.cuda.synchronize()
        check_close(out, want[:, r * rows:(r + 1) * rows], torch.bfloat16)
    assert nat.device_status() == 0
