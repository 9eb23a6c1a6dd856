"""Shared helpers of the parity tests: seeded inputs, tolerances, pattern pairs."""
import numpy as np
import torch

from oracle import oracle as O
from ma_transformer_b200.patterns import PatternSpec, WINDOW, BLOCK, LONGFORMER

# tolerances of the parity bar
FP32_REL = 1e-5     # max|gpu - oracle| / max|oracle|
BF16_ABS = 2e-2     # max|gpu - oracle| with the oracle fed the bf16-rounded inputs in fp32
F16_ABS = 5e-3


def to_oracle(spec: PatternSpec) -> O.OraclePattern:
    """The oracle's own description of the same key set (built field by field)."""
    return O.OraclePattern(kind={WINDOW: O.WINDOW, BLOCK: O.BLOCK, LONGFORMER: O.LONGFORMER}[spec.kind],
                           left=spec.left, right=spec.right, dilation=spec.dilation, causal=spec.causal,
                           block=spec.block, blk_rowptr=spec.blk_rowptr, blk_colidx=spec.blk_colidx,
                           global_idx=spec.global_idx, q_offset=spec.q_offset)


def seeded_qkv(seed, B, Sq, H, D, dtype=torch.float32, Skv=None, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    Skv = Sq if Skv is None else Skv
    q = (torch.randn(B, Sq, H, D, generator=g) * scale).to(dtype)
    k = (torch.randn(B, Skv, H, D, generator=g) * scale).to(dtype)
    v = (torch.randn(B, Skv, H, D, generator=g) * scale).to(dtype)
    return q, k, v


def oracle_out(q, k, v, spec, scale=0.0):
    """fp32 oracle on the exact values the GPU sees (16-bit inputs upcast)."""
    return O.sparse_attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), to_oracle(spec), scale)


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def check_close(got: torch.Tensor, want: np.ndarray, dtype):
    got = got.float().cpu().numpy()
    assert np.isfinite(got).all()
    if dtype == torch.float32:
        e = rel_err(got, want)
        assert e <= FP32_REL, f"fp32 rel-err {e:.3e} > {FP32_REL}"
    else:
        tol = BF16_ABS if dtype == torch.bfloat16 else F16_ABS
        e = float(np.abs(got - want).max())
        assert e <= tol, f"max-abs {e:.3e} > {tol}"


def expected_window_kernel(spec: PatternSpec, Skv: int) -> str:
    """Which kernel family the library picks for a 16-bit, D = 64 window call it can tile (the routing
    of run_problem): dense and windows of more than 128 taps on tcgen05 when the sequence is long
    enough and the shard offset is a multiple of 64, the warp-level tiled kernel otherwise."""
    left, right = min(spec.left, Skv - 1), min(spec.right, Skv - 1)
    if spec.dilation != 1 or spec.q_offset % 64 or Skv < 256:
        return "mma_window"
    if left >= Skv - 1 and (right >= Skv - 1 or right == 0):
        return "umma_dense"
    return "umma_window" if left + right > 128 else "mma_window"
