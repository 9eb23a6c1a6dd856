"""Regenerates tests/golden/reference_window.npz from the reference itself.

Run in a container that holds the reference tree (``--ref``, or $MAT_REFERENCE_DIR) and
the compiled reference engine (``make -C oracle`` builds oracle/_ref):

    python tests/golden/make_golden.py --ref <path to the ma-transformer checkout>

For every case the file stores the seeded inputs (once per seed and shape,
under ``q_<seed>_<B>_<S>_<H>_<D>``) and two outputs of the
reference: ``ref_cpp`` from the compiled C++ engine
(``ma_core.compute_sparse_attention``, src/csrc/ma_core.cpp:160-246) and
``ref_torch`` from the reference's python test oracle
(``pytorch_sparse_attention``, src/layers/ma_core_bridge.py:224-247).
The cases are the shapes, seeds and windows the reference's own tests use:
  tests/python/test_cpu_attention_cpp.py:42-56          seed 1
  tests/integration/test_cpu_parity.py:26-43            seed 42
  tests/integration/test_cuda_parity.py:42-57           seed 0
  tests/integration/test_cuda_extensive.py:52-74        seed 321
  tests/python/test_cuda_sparse_kernel_launch.py:13-30  seed 123
It also stores the pattern counts the reference's tests pin
(tests/python/test_tensor_functionality.py:173-200).
"""
import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def main() -> None:
    ap = argparse.ArgumentParser()
    import os
    ap.add_argument("--ref", default=os.environ.get("MAT_REFERENCE_DIR", str(ROOT.parent / "reference")))
    args = ap.parse_args()
    sys.path.insert(0, str(ROOT / "oracle" / "_ref"))
    sys.path.insert(0, args.ref)
    import ma_core  # the compiled reference engine
    from src.layers.ma_core_bridge import pytorch_sparse_attention, pytorch_to_ma_core

    cases = []  # (seed, B, S, H, D, W)
    cases += [(1, 1, 10, 2, 4, 2)]
    cases += [(42, b, s, h, d, w) for (b, s, h, d) in [(1, 8, 2, 4), (2, 20, 2, 8)] for w in (1, 2, 4)]
    cases += [(0, b, s, h, d, w) for (b, s, h, d) in [(1, 32, 2, 16), (2, 64, 4, 32)] for w in (1, 4, 8)]
    cases += [(321, b, s, h, d, w) for (b, s, h, d) in [(1, 7, 2, 5), (2, 16, 4, 8), (2, 33, 1, 13)]
              for w in (0, 1, 2, 4, 8, 64)]
    cases += [(123, 2, s, 2, 16, w) for s in (1, 17, 33, 64, 127) for w in (0, 1, 4, 8)]

    out = {}
    meta = []
    for n, (seed, B, S, H, D, W) in enumerate(cases):
        torch.manual_seed(seed)
        q = torch.randn(B, S, H, D)
        k = torch.randn(B, S, H, D)
        v = torch.randn(B, S, H, D)
        ref_torch = pytorch_sparse_attention(q, k, v, window_size=W)
        mc = ma_core.compute_sparse_attention(pytorch_to_ma_core(q), pytorch_to_ma_core(k),
                                              pytorch_to_ma_core(v), W)
        ref_cpp = np.asarray(mc.to_numpy())
        # inputs depend on (seed, shape) only: store them once per group
        tag = f"{seed}_{B}_{S}_{H}_{D}"
        out[f"q_{tag}"], out[f"k_{tag}"], out[f"v_{tag}"] = q.numpy(), k.numpy(), v.numpy()
        out[f"ref_cpp{n}"], out[f"ref_torch{n}"] = ref_cpp, ref_torch.numpy()
        meta.append((seed, B, S, H, D, W))
    out["meta"] = np.asarray(meta, dtype=np.int64)

    # pattern counts through the compiled reference generator (ma_core.cpp:34-48)
    pats = [(4, 4), (4, 10), (16, 3), (12, 2), (1, 0), (33, 8)]
    out["pattern_cases"] = np.asarray(pats, dtype=np.int64)
    out["pattern_nnz"] = np.asarray(
        [ma_core.create_sliding_window_pattern(s, w).nnz() for s, w in pats], dtype=np.int64)
    np.savez_compressed(HERE / "reference_window.npz", **out)
    print(f"wrote {len(cases)} cases to {HERE / 'reference_window.npz'}")


if __name__ == "__main__":
    main()
