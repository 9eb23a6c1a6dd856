"""numpy front end of the CPU oracle (liboracle.so).  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module; it is the checker used by
the tests, by the smoke check and by the CPU-baseline leg of the benchmark.
The arithmetic is the C restatement of ma-transformer's
``ma_core::compute_sparse_attention`` (src/csrc/ma_core.cpp:160-246); see the
header of sparse_attn_oracle.c for the line-by-line mapping.

``reference_module()`` returns the *unmodified* reference engine (python module
``ma_core`` compiled from the reference's own three sources into oracle/_ref/)
when that build is present, else None.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os
import subprocess
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB: Optional[C.CDLL] = None

WINDOW, BLOCK, LONGFORMER = 0, 1, 2


class _Spec(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("causal", C.c_int32),
        ("left", C.c_int64), ("right", C.c_int64), ("dilation", C.c_int64),
        ("block", C.c_int64), ("n_qblocks", C.c_int64),
        ("blk_rowptr", C.POINTER(C.c_int32)), ("blk_colidx", C.POINTER(C.c_int32)),
        ("n_global", C.c_int64), ("global_idx", C.POINTER(C.c_int64)),
        ("q_offset", C.c_int64),
    ]


def build() -> Path:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    subprocess.run(["make", "-C", str(_HERE), "-s"], check=True)
    return _HERE / "liboracle.so"


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        so = _HERE / "liboracle.so"
        if not so.exists():
            build()
        L = C.CDLL(str(so))
        L.oracle_rowset.restype = C.c_int64
        L.oracle_rowset.argtypes = [C.POINTER(_Spec), C.c_int64, C.c_int64, C.c_void_p, C.c_int64]
        L.oracle_pattern_nnz.restype = C.c_int64
        L.oracle_pattern_nnz.argtypes = [C.POINTER(_Spec), C.c_int64, C.c_int64]
        L.oracle_sparse_attn_fwd_f32.restype = C.c_int
        L.oracle_sparse_attn_fwd_f32.argtypes = [C.c_void_p] * 4 + [C.c_int64] * 6 + [
            C.POINTER(_Spec), C.c_float, C.c_int]
        L.oracle_num_threads.restype = C.c_int
        _LIB = L
    return _LIB


@dataclass
class OraclePattern:
    """Key-set description understood by the oracle (independent of the product's)."""
    kind: int = WINDOW
    left: int = 0
    right: int = 0
    dilation: int = 1
    causal: bool = False
    block: int = 0
    blk_rowptr: Optional[np.ndarray] = None
    blk_colidx: Optional[np.ndarray] = None
    global_idx: Optional[np.ndarray] = None
    q_offset: int = 0
    _keep: list = field(default_factory=list, repr=False)

    # -- constructors named after the configurations they describe ---------
    @staticmethod
    def symmetric(w: int) -> "OraclePattern":
        """The reference's own key set [i-w, i+w] (ma_core.cpp:197-198)."""
        return OraclePattern(WINDOW, left=w, right=w)

    @staticmethod
    def causal_taps(w: int, dilation: int = 1) -> "OraclePattern":
        """w taps ending at the query: i-(w-1)*dil, ..., i-dil, i."""
        return OraclePattern(WINDOW, left=w - 1, right=0, dilation=dilation)

    @staticmethod
    def block_csr(block: int, rowptr: Sequence[int], colidx: Sequence[int],
                  causal: bool = False) -> "OraclePattern":
        return OraclePattern(BLOCK, block=block, causal=causal,
                             blk_rowptr=np.ascontiguousarray(rowptr, dtype=np.int32),
                             blk_colidx=np.ascontiguousarray(colidx, dtype=np.int32))

    @staticmethod
    def longformer(left: int, right: int, global_idx: Sequence[int]) -> "OraclePattern":
        return OraclePattern(LONGFORMER, left=left, right=right,
                             global_idx=np.ascontiguousarray(global_idx, dtype=np.int64))

    def c_struct(self) -> _Spec:
        s = _Spec()
        s.kind, s.causal = int(self.kind), int(bool(self.causal))
        s.left, s.right, s.dilation = int(self.left), int(self.right), int(self.dilation)
        s.block, s.q_offset = int(self.block), int(self.q_offset)
        if self.blk_rowptr is not None:
            rp = np.ascontiguousarray(self.blk_rowptr, dtype=np.int32)
            ci = np.ascontiguousarray(self.blk_colidx, dtype=np.int32)
            self._keep = [rp, ci]
            s.n_qblocks = len(rp) - 1
            s.blk_rowptr = rp.ctypes.data_as(C.POINTER(C.c_int32))
            s.blk_colidx = ci.ctypes.data_as(C.POINTER(C.c_int32))
        if self.global_idx is not None and len(self.global_idx):
            g = np.ascontiguousarray(self.global_idx, dtype=np.int64)
            self._keep.append(g)
            s.n_global = len(g)
            s.global_idx = g.ctypes.data_as(C.POINTER(C.c_int64))
        return s


def rowset(pat: OraclePattern, s_kv: int, i: int) -> np.ndarray:
    """Sorted unique key positions of query row ``i`` as int64."""
    sp = pat.c_struct()
    cap = 2 * s_kv + int(sp.n_global) + 8
    out = np.empty(cap, dtype=np.int64)
    n = lib().oracle_rowset(C.byref(sp), s_kv, i, out.ctypes.data, cap)
    if n < 0:
        raise ValueError("malformed pattern description")
    return out[:n].copy()


def pattern_nnz(pat: OraclePattern, s_q: int, s_kv: Optional[int] = None) -> int:
    sp = pat.c_struct()
    n = lib().oracle_pattern_nnz(C.byref(sp), s_q, s_kv if s_kv is not None else s_q)
    if n < 0:
        raise ValueError("malformed pattern description")
    return int(n)


def sparse_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, pat: OraclePattern,
                     scale: float = 0.0, threads: int = 0) -> np.ndarray:
    """fp32 forward over [B,S,H,D] arrays.  ``scale`` 0 means 1/sqrt(D)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("expected [B,S,H,D] arrays")
    B, Sq, H, D = q.shape
    Skv, Dv = k.shape[1], v.shape[3]
    if k.shape != (B, Skv, H, D) or v.shape[:3] != (B, Skv, H):
        raise ValueError("q/k/v shapes disagree")
    o = np.empty((B, Sq, H, Dv), dtype=np.float32)
    sp = pat.c_struct()
    rc = lib().oracle_sparse_attn_fwd_f32(q.ctypes.data, k.ctypes.data, v.ctypes.data,
                                          o.ctypes.data, B, Sq, Skv, H, D, Dv,
                                          C.byref(sp), float(scale), int(threads))
    if rc != 0:
        raise RuntimeError("oracle forward failed (malformed pattern or out of memory)")
    return o


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def reference_module():
    """The reference's own compiled CPU engine (module ``ma_core``), or None."""
    ref_dir = _HERE / "_ref"
    hits = sorted(ref_dir.glob("ma_core*.so")) if ref_dir.is_dir() else []
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("ma_core", hits[0])
    try:
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)  # type: ignore[union-attr]
    except Exception:
        return None
    return mod


def reference_sparse_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, w: int) -> np.ndarray:
    """Run the compiled reference engine (key set [i-w, i+w]) on fp32 arrays."""
    m = reference_module()
    if m is None:
        raise RuntimeError("oracle/_ref is not built")
    ts = []
    for a in (q, k, v):
        a = np.ascontiguousarray(a, dtype=np.float32)
        t = m.create_tensor(list(a.shape))
        t.copy_from_numpy(a)
        ts.append(t)
    return np.asarray(m.compute_sparse_attention(ts[0], ts[1], ts[2], int(w)).to_numpy())
