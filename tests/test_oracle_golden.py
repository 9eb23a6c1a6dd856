"""Pins the CPU oracle: bit-exact against the outputs of the compiled reference
engine stored in tests/golden (and against the engine itself when oracle/_ref is
present), within the reference's own test tolerance of its python oracle, and on
the pattern counts the reference's tests hold."""
import numpy as np
import pytest

from helpers import to_oracle
from ma_transformer_b200.patterns import PatternSpec, tridiagonal_block_layout


def _cases(golden):
    for n, (seed, B, S, H, D, W) in enumerate(golden["meta"].tolist()):
        tag = f"{seed}_{B}_{S}_{H}_{D}"
        yield n, W, golden[f"q_{tag}"], golden[f"k_{tag}"], golden[f"v_{tag}"]


def test_oracle_bit_exact_vs_reference_cpp(golden, oracle):
    for n, W, q, k, v in _cases(golden):
        got = oracle.sparse_attention(q, k, v, oracle.OraclePattern.symmetric(W))
        assert np.array_equal(got, golden[f"ref_cpp{n}"]), f"case {n} differs from ma_core.compute_sparse_attention"


def test_oracle_vs_reference_python_oracle(golden, oracle):
    # tolerance of tests/integration/test_cpu_parity.py:26-43 in the reference
    for n, W, q, k, v in _cases(golden):
        got = oracle.sparse_attention(q, k, v, oracle.OraclePattern.symmetric(W))
        np.testing.assert_allclose(got, golden[f"ref_torch{n}"], rtol=1e-5, atol=1e-6)


def test_oracle_vs_live_reference_engine(oracle):
    if oracle.reference_module() is None:
        pytest.skip("oracle/_ref not built in this environment")
    rng = np.random.default_rng(5)
    for (B, S, H, D, W) in [(1, 64, 4, 64, 32), (2, 50, 3, 24, 7), (1, 9, 1, 3, 100)]:
        q, k, v = [rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3)]
        assert np.array_equal(oracle.sparse_attention(q, k, v, oracle.OraclePattern.symmetric(W)),
                              oracle.reference_sparse_attention(q, k, v, W))


def test_pattern_counts_pinned_by_reference(golden, oracle):
    # ma_core.create_sliding_window_pattern(S, w).nnz(), tests/python/test_tensor_functionality.py:173-200
    for (S, w), nnz in zip(golden["pattern_cases"].tolist(), golden["pattern_nnz"].tolist()):
        assert oracle.pattern_nnz(oracle.OraclePattern.symmetric(w), S) == nnz
    # anchors read from the reference's generators (sparse_attention.cpp:181-259)
    assert oracle.pattern_nnz(oracle.OraclePattern.symmetric(2), 12) == 54
    rp, ci = tridiagonal_block_layout(12, 4)
    assert oracle.pattern_nnz(oracle.OraclePattern.block_csr(4, rp, ci), 12) == 112
    # Longformer S=12, w=2, globals {0,1}: 102 COO entries in the reference, 88 distinct
    assert oracle.pattern_nnz(oracle.OraclePattern.longformer(2, 2, [0, 1]), 12) == 88


def test_rowsets_by_hand(oracle):
    P = oracle.OraclePattern
    assert oracle.rowset(P.causal_taps(4), 20, 9).tolist() == [6, 7, 8, 9]
    assert oracle.rowset(P.causal_taps(4, 2), 20, 9).tolist() == [3, 5, 7, 9]
    assert oracle.rowset(P.causal_taps(4, 2), 20, 2).tolist() == [0, 2]
    assert oracle.rowset(P.symmetric(0), 5, 3).tolist() == [3]
    assert oracle.rowset(P.longformer(1, 1, [7, 3]), 10, 5).tolist() == [3, 4, 5, 6, 7]
    assert oracle.rowset(P.longformer(1, 1, [7, 3]), 10, 7).tolist() == list(range(10))
    blk = P.block_csr(4, [0, 1, 3], [0, 0, 1], causal=True)
    assert oracle.rowset(blk, 8, 5).tolist() == [0, 1, 2, 3, 4, 5]
    shifted = P.causal_taps(3)
    shifted.q_offset = 2
    assert oracle.rowset(shifted, 10, 0).tolist() == [0, 1, 2]


def test_oracle_generalised_patterns_reduce_to_reference(oracle):
    """Each generalised key set collapses to the reference's +-w set on the
    overlapping special case, so their arithmetic is pinned through it."""
    rng = np.random.default_rng(11)
    B, S, H, D, w = 1, 24, 2, 8, 3
    q, k, v = [rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3)]
    want = oracle.sparse_attention(q, k, v, oracle.OraclePattern.symmetric(w))
    # Longformer without globals
    assert np.array_equal(oracle.sparse_attention(q, k, v, oracle.OraclePattern.longformer(w, w, [])), want)
    # dilation 1
    assert np.array_equal(oracle.sparse_attention(q, k, v, oracle.OraclePattern(oracle.WINDOW, left=w, right=w, dilation=1)), want)
    # block size 1, band layout |r-c| <= w
    rp, ci = [0], []
    for r in range(S):
        ci += [c for c in range(S) if abs(r - c) <= w]
        rp.append(len(ci))
    assert np.array_equal(oracle.sparse_attention(q, k, v, oracle.OraclePattern.block_csr(1, rp, ci)), want)
    # a sharded view: rows 8..15 with a halo of w rows either side equal the same rows of the full run
    sh = oracle.OraclePattern.symmetric(w)
    sh.q_offset = w
    part = oracle.sparse_attention(q[:, 8:16], k[:, 8 - w:16 + w], v[:, 8 - w:16 + w], sh)
    assert np.array_equal(part, want[:, 8:16])
