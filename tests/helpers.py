"""Shared helpers of the parity tests: seeded inputs, tolerances, pattern pairs."""
import math

import numpy as np
import torch
import torch.nn.functional as F

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


def expected_window_kernel(spec: PatternSpec, Skv: int, neighbours: bool = False) -> str:
    """Which kernel family the library picks for a 16-bit, D = 64 window call it can tile (the routing
    of run_problem): dense and windows of more than 128 taps on the tcgen05 walk when the sequence is long
    enough and the shard offset is a multiple of 64; windows of at most 128 taps on the persistent
    tcgen05 band kernel; the warp-level tiled kernel otherwise.  ``neighbours``: the call reads halo rows
    from neighbouring shards' tensors (only the band and the warp-level kernels do)."""
    dil = spec.dilation
    left, right = min(spec.left, Skv - 1), min(spec.right, Skv - 1)
    if dil == 1 and spec.q_offset % 64 == 0 and Skv >= 256 and not neighbours:
        if left >= Skv - 1 and (right >= Skv - 1 or right == 0):
            return "umma_dense"
        if left + right > 128:
            return "umma_window"
    skv1 = Skv // dil
    reach = 2 * skv1 if neighbours else skv1           # taps clamp to the keys that exist (own rows plus a neighbour's)
    l1, r1 = min(spec.left, reach), min(spec.right, reach)
    cl = (spec.q_offset // dil - l1) % 16
    if cl + l1 + r1 <= 128:
        return "umma_band"
    return "mma_window"


def orderbook_reference_forward(model, ticks: torch.Tensor) -> torch.Tensor:
    """The order-book transformer (ma_transformer_b200.layers.orderbook_model) in plain fp32 torch with a dense masked attention: the
    numerics reference of the model tests (small sequences only)."""
    spec = model.pattern
    x = model.embed(ticks) * math.sqrt(model.d_model)
    S = x.shape[1]
    i = torch.arange(S, device=x.device)
    d = i[:, None] - i[None, :]                      # query - key
    keep = (d >= 0) & (d <= spec.left * spec.dilation) & (d % spec.dilation == 0)
    for blk in model.blocks:
        B, _, Dm = x.shape
        y = blk.norm1(x)
        q, k, v = blk.qkv_proj(y).view(B, S, 3, blk.n_heads, blk.head_dim).unbind(2)
        s = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(blk.head_dim)
        s = s.masked_fill(~keep, float("-inf"))
        a = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), v).reshape(B, S, Dm)
        x = x + blk.out_proj(a)
        x = x + blk.ff2(F.gelu(blk.ff1(blk.norm2(x))))
    return model.head(model.norm(x[:, -1]))


def masked_dense_attention(q, k, v, left, right, dilation=1):
    """Window attention { p + t*dilation : -left <= t <= right } as a dense masked softmax in the
    tensors' own dtype (use float64 inputs for an autograd reference): independent of every kernel
    and of the banded torch implementation."""
    S = q.shape[1]
    i = torch.arange(S, device=q.device)
    d = i[None, :] - i[:, None]                       # key - query
    keep = (d % dilation == 0) & (d >= -left * dilation) & (d <= right * dilation)
    s = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~keep, float("-inf"))
    return torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), v)


def pattern_mask(spec, S):
    """[S, S] boolean: entry (i, j) is set iff query row i of the pattern attends key j.  Built row by row from
    the library's host index sets (mat_pattern_rowset), which are pinned to the oracle bit for bit and share no
    code with the backward kernels."""
    keep = torch.zeros(S, S, dtype=torch.bool)
    for i in range(S):
        keep[i, torch.from_numpy(spec.rowset(S, i))] = True
    return keep


def masked_attention_with(q, k, v, keep):
    """Dense masked softmax attention over an explicit [S, S] mask, in the tensors' own dtype."""
    s = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~keep.to(q.device), float("-inf"))
    return torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), v)
