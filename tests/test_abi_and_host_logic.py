"""CPU-side checks of the shipped library: it loads, exports every symbol the
header declares, its host index sets equal the oracle's bit for bit, and the
python surface validates arguments as the reference does."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import ma_transformer_b200 as mt
from ma_transformer_b200 import _native as nat
from ma_transformer_b200.patterns import PatternSpec, band_random_block_layout, tridiagonal_block_layout
from helpers import to_oracle

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    text = (ROOT / "include" / "mat_sparse_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(mat_[a-z_0-9]+)\s*\(", text))
    assert declared, "no declarations parsed"
    lib = C.CDLL(str(nat.LIB_PATH))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(nat.EXPORTS)
    assert lib.mat_version() >= 100


def _random_specs(rng):
    for _ in range(40):
        S = int(rng.integers(1, 70))
        kind = int(rng.integers(0, 3))
        if kind == 0:
            yield S, PatternSpec(left=int(rng.integers(0, 12)), right=int(rng.integers(0, 12)),
                                 dilation=int(rng.integers(1, 4)))
        elif kind == 1:
            block = int(rng.choice([1, 3, 4, 8, 16]))
            nb = (S + block - 1) // block
            rp, ci = [0], []
            for r in range(nb):
                ci += sorted(rng.choice(nb, size=int(rng.integers(0, min(nb, 4) + 1)), replace=False).tolist())
                rp.append(len(ci))
            yield S, PatternSpec.block_sparse(block, rp, ci, causal=bool(rng.integers(0, 2)))
        else:
            ng = int(rng.integers(0, min(S, 5) + 1))
            yield S, PatternSpec.longformer(int(rng.integers(0, 6)), int(rng.integers(0, 6)),
                                            rng.choice(S, size=ng, replace=False))


def test_host_rowsets_match_oracle_bit_exact(oracle):
    rng = np.random.default_rng(2024)
    for S, spec in _random_specs(rng):
        opat = to_oracle(spec)
        total = 0
        for i in range(S):
            mine = spec.rowset(S, i)
            ref = oracle.rowset(opat, S, i)
            assert mine.dtype == np.int64 and np.array_equal(mine, ref), (spec, i)
            total += len(mine)
        assert spec.nnz(S) == total == oracle.pattern_nnz(opat, S)


def test_host_rowsets_with_shard_offset(oracle):
    spec = PatternSpec.causal_window(5, dilation=2).shifted(8)
    for i in range(10):
        assert np.array_equal(spec.rowset(30, i), oracle.rowset(to_oracle(spec), 30, i))
    assert spec.rowset(30, 0).tolist() == [0, 2, 4, 6, 8]


def test_reference_pattern_counts():
    assert PatternSpec.sliding_window(4).nnz(4) == 16     # tests/python/test_tensor_functionality.py:173-179
    assert PatternSpec.sliding_window(10).nnz(4) == 16
    assert PatternSpec.sliding_window(2).nnz(12) == 54
    rp, ci = tridiagonal_block_layout(12, 4)
    assert PatternSpec.block_sparse(4, rp, ci).nnz(12) == 112
    assert PatternSpec.longformer(2, 2, [0, 1]).nnz(12) == 88


def test_band_random_layout_shape():
    rp, ci = band_random_block_layout(256, band=4, n_random=2, seed=0)
    assert rp[-1] == 1521      # 1018 band + 503 random entries for 256 block rows
    for r in range(256):
        row = ci[rp[r]:rp[r + 1]]
        assert len(set(row.tolist())) == len(row) and row.max() <= r
        assert set(range(max(0, r - 3), r + 1)) <= set(row.tolist())


def test_pattern_statistics_and_estimates():
    """Pattern tooling of the reference (get_pattern_statistics, tests/python/test_tensor_functionality.py:181-202;
    attention_utils::estimate_flops / estimate_memory_usage, src/csrc/sparse_attention.cpp:312-357) from the
    closed-form patterns."""
    from ma_transformer_b200.patterns import (estimate_flops, estimate_memory_usage, pattern_flops,
                                               pattern_statistics)
    stats = pattern_statistics(PatternSpec.sliding_window(3), 16)
    assert isinstance(stats, str)
    for key in ("Pattern Statistics", "Total elements", "Non-zero elements", "Sparsity ratio"):
        assert key in stats
    lines = stats.split("\n")
    total = int([l for l in lines if "Total elements" in l][0].split(": ")[1])
    nonzero = int([l for l in lines if "Non-zero elements" in l][0].split(": ")[1])
    assert total == 256 and nonzero == 16 * 7 - 2 * (1 + 2 + 3)       # +-3 window clipped at both ends
    assert "60.937500%" in stats                                       # std::to_string of the float ratio
    # the reference's conventions on the long-sequence shape: w keys per row, one matmul
    assert estimate_flops("sliding_window", 1, 65536, 8, 64, window_size=64) == 4294967296
    assert estimate_memory_usage("sliding_window", 1, 65536, 8, window_size=64) == 67108864
    assert estimate_flops("full", 2, 128, 4, 64) == 2 * 4 * 128 * 128 * 64 * 2
    assert estimate_flops("block_sparse", 1, 200, 2, 64, block_size=64) == 2 * 4 * 3 * 64 * 64 * 64
    assert estimate_flops("big_bird", 1, 100, 1, 8) == 100 * 100 * 8
    assert estimate_memory_usage("causal", 1, 100, 2) == 2 * 100 * 100 * 2
    # what a pattern really costs: both products over its (query, key) pairs
    assert pattern_flops(PatternSpec.causal_window(64), 1, 65536, 8, 64) == 4 * 8 * 64 * (65536 * 64 - 63 * 64 // 2)


def test_bigbird_and_random_block_layouts():
    """BIG_BIRD and RANDOM_SPARSE of the reference's pattern vocabulary (src/csrc/attention_types.hpp:26-56),
    as seeded block layouts."""
    from ma_transformer_b200.patterns import bigbird_block_layout, random_block_layout
    nb = 12
    rp, ci = bigbird_block_layout(nb, window_blocks=3, n_global_blocks=2, n_random_blocks=2, seed=3)
    assert rp[0] == 0 and len(rp) == nb + 1 and rp[-1] == len(ci)
    for r in range(nb):
        cols = ci[rp[r]:rp[r + 1]].tolist()
        assert cols == sorted(set(cols)) and all(0 <= c < nb for c in cols)
        if r < 2:
            assert cols == list(range(nb))                      # global rows see everything
        else:
            assert {0, 1} <= set(cols)                          # global columns
            assert {c for c in (r - 1, r, r + 1) if c < nb} <= set(cols)
            assert len(cols) == len({0, 1} | {c for c in (r - 1, r, r + 1) if c < nb}) + 2
    again = bigbird_block_layout(nb, 3, 2, 2, seed=3)
    assert np.array_equal(again[0], rp) and np.array_equal(again[1], ci)          # seeded: reproducible
    rp, ci = random_block_layout(16, 0.25, seed=4)
    for r in range(16):
        cols = ci[rp[r]:rp[r + 1]].tolist()
        assert len(cols) == 4 and r in cols and cols == sorted(set(cols))
    spec = PatternSpec.block_sparse(8, rp, ci)
    assert spec.nnz(16 * 8) == 16 * 4 * 64
    with pytest.raises(ValueError):
        random_block_layout(4, 1.5)


def test_malformed_patterns_are_rejected():
    with pytest.raises(ValueError):
        PatternSpec(left=-1)
    with pytest.raises(ValueError):
        PatternSpec(dilation=0)
    with pytest.raises(ValueError):
        PatternSpec.block_sparse(4, [0, 2], [1, 1])       # repeated column
    with pytest.raises(ValueError):
        PatternSpec.block_sparse(4, [0, 3], [0, 1])       # row pointers past the end
    s = nat.MatPatternSpec()
    s.kind = 9
    n = C.c_int64()
    assert nat.lib.mat_pattern_nnz(C.byref(s), 4, 4, C.byref(n)) != 0
    assert b"pattern kind" in nat.lib.mat_last_error()


def test_global_positions_outside_the_sequence_are_refused_on_the_host():
    """The list of global positions is read on the device, where nothing can refuse it, so the python
    surface checks it before any launch (no GPU involved: the check is host arithmetic)."""
    spec = PatternSpec.longformer(2, 2, [3, 64])
    with pytest.raises(RuntimeError, match=r"\[0, S\)"):
        spec.check_against(64)
    spec.check_against(65)                       # in range: silent
    PatternSpec.longformer(2, 2, []).check_against(1)
    PatternSpec.causal_window(8).check_against(4)
    with pytest.raises(ValueError):
        PatternSpec.longformer(2, 2, [-1, 3])     # negative positions never pass the constructor
    # host tensors through forward_host are refused before the library is entered
    q = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="outside the sequence"):
        mt.sparse_attention_cuda.forward_host(q, q, q, spec)


def test_module_validation_matches_reference_messages():
    # src/layers/ma_core_bridge.py:272-277, 297-314
    with pytest.raises(ValueError):
        mt.MACoreAttention(sparse=True, window_size=0)
    with pytest.raises(TypeError):
        mt.MACoreAttention(sparse=True, window_size=2.5)
    attn = mt.MACoreAttention(sparse=True, window_size=4).eval()
    with pytest.raises(ValueError, match="shape"):
        attn(torch.randn(2, 8, 16), torch.randn(2, 8, 16), torch.randn(2, 8, 16))
    with pytest.raises(ValueError) as ei:
        attn(torch.randn(1, 8, 2, 4), torch.randn(1, 9, 2, 4), torch.randn(1, 9, 2, 4))
    assert any(w in str(ei.value).lower() for w in ("sequence", "length", "mismatch", "size"))
    with pytest.raises(ValueError):
        attn(torch.randn(1, 0, 2, 4), torch.randn(1, 0, 2, 4), torch.randn(1, 0, 2, 4))
    with pytest.raises(ValueError):
        mt.create_attention_layer("nope")
    with pytest.raises(ValueError):
        mt.SparseAttention(window_size=0)
    assert isinstance(mt.create_attention_layer("auto", window_size=3), mt.MACoreAttention)


def test_extension_surface_rejects_cpu_tensors_like_the_reference():
    # sparse_attention_kernel.cu:427: TORCH_CHECK -> RuntimeError
    q = torch.randn(1, 4, 1, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        mt.sparse_attention_cuda.forward(q, q, q, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        mt.sparse_attention_cuda.dense_forward(q, q, q)
    import inspect
    sig = inspect.signature(mt.sparse_attention_cuda.forward)
    assert list(sig.parameters) == ["query", "key", "value", "window_size"]
    assert sig.parameters["window_size"].default == 64
    assert list(inspect.signature(mt.sparse_attention_cuda.backward).parameters) == \
        ["query", "key", "value", "grad_out", "window_size"]


def test_training_mode_uses_differentiable_path_on_cpu():
    attn = mt.MACoreAttention(sparse=True, window_size=2)   # fresh module: training, fallback_training
    q = torch.randn(1, 9, 2, 4, requires_grad=True)
    y = attn(q, q, q)
    y.sum().backward()
    assert q.grad is not None and torch.isfinite(q.grad).all()


def test_torch_oracle_functions_match_oracle(oracle):
    g = torch.Generator().manual_seed(3)
    q, k, v = [torch.randn(2, 21, 3, 8, generator=g) for _ in range(3)]
    for w in (0, 1, 5, 30):
        want = oracle.sparse_attention(q.numpy(), k.numpy(), v.numpy(), oracle.OraclePattern.symmetric(w))
        np.testing.assert_allclose(mt.pytorch_sparse_attention(q, k, v, w).numpy(), want, rtol=1e-5, atol=1e-6)
    want = oracle.sparse_attention(q.numpy(), k.numpy(), v.numpy(), oracle.OraclePattern(left=21, right=0))
    np.testing.assert_allclose(mt.pytorch_dense_attention(q, k, v, True).numpy(), want, rtol=1e-5, atol=1e-6)


def test_transposed_block_layout_round_trip():
    """The layout the backward's dK / dV pass walks: for every key block the ascending query blocks that hold it.
    Transposing twice gives the layout back; entries are the same (row, column) pairs."""
    from ma_transformer_b200.patterns import PatternSpec, band_random_block_layout
    rp, ci = band_random_block_layout(17, 3, 2, seed=11)
    spec = PatternSpec.block_sparse(64, rp, ci, causal=True)
    t_rp, t_ci = spec.transposed_layout()
    assert t_rp.dtype == np.int32 and t_ci.dtype == np.int32 and t_rp[-1] == len(ci) and len(t_rp) == len(rp)
    pairs = {(r, int(c)) for r in range(len(rp) - 1) for c in ci[rp[r]:rp[r + 1]]}
    t_pairs = {(int(r), c) for c in range(len(t_rp) - 1) for r in t_ci[t_rp[c]:t_rp[c + 1]]}
    assert pairs == t_pairs
    for c in range(len(t_rp) - 1):
        assert list(t_ci[t_rp[c]:t_rp[c + 1]]) == sorted(t_ci[t_rp[c]:t_rp[c + 1]])
    back = PatternSpec.block_sparse(64, t_rp, t_ci).transposed_layout()
    assert np.array_equal(back[0], spec.blk_rowptr) and np.array_equal(back[1], spec.blk_colidx)
