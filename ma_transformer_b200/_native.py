"""ctypes binding of libmat_sparse_attn.so (declared in include/mat_sparse_attn.h).

The library is the only compute path of this package: if it is missing or does
not load, importing this module raises, and nothing falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libmat_sparse_attn.so"

MAT_OK = 0
MAT_F32, MAT_BF16, MAT_F16 = 0, 1, 2
MAT_WINDOW, MAT_BLOCK, MAT_LONGFORMER = 0, 1, 2

# every symbol include/mat_sparse_attn.h declares
EXPORTS = (
    "mat_version", "mat_last_error", "mat_last_kernel", "mat_device_status",
    "mat_sparse_attn_fwd", "mat_sparse_attn_fwd_strided", "mat_sparse_attn_workspace_bytes", "mat_sparse_attn_fwd_window",
    "mat_sparse_attn_fwd_host", "mat_sparse_attn_host_staging_bytes", "mat_sparse_attn_fwd_sharded",
    "mat_pattern_rowset", "mat_pattern_nnz", "mat_enable_peer_access",
    "mat_ipc_export", "mat_ipc_open", "mat_ipc_close", "mat_sparse_attn_fwd_longformer_noalloc",
    "mat_sparse_attn_bwd", "mat_sparse_attn_bwd_workspace_bytes", "mat_sparse_attn_bwd_general", "mat_sparse_attn_bwd_general_workspace_bytes",
    "mat_longformer_shard_fwd", "mat_global_rows_partial_layout", "mat_global_rows_partial", "mat_global_rows_merge",
)


class MatPatternSpec(C.Structure):
    """struct mat_pattern_spec"""
    _fields_ = [
        ("kind", C.c_int32), ("causal", C.c_int32),
        ("left", C.c_int64), ("right", C.c_int64), ("dilation", C.c_int64),
        ("block", C.c_int64), ("n_qblocks", C.c_int64),
        ("blk_rowptr", C.c_void_p), ("blk_colidx", C.c_void_p),
        ("n_global", C.c_int64), ("global_idx", C.c_void_p),
        ("q_offset", C.c_int64),
    ]


class NativeError(RuntimeError):
    """A libmat_sparse_attn call returned an error code (RuntimeError, as the
    reference extension's TORCH_CHECK failures are)."""


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python ma_transformer_b200/build_native.py` "
            "(there is no CPU fallback)")
    lib = C.CDLL(str(LIB_PATH))
    i64, vp, sz = C.c_int64, C.c_void_p, C.c_size_t
    spec_p = C.POINTER(MatPatternSpec)
    lib.mat_version.restype = C.c_int
    lib.mat_last_error.restype = C.c_char_p
    lib.mat_last_kernel.restype = C.c_char_p
    lib.mat_device_status.restype = C.c_int
    lib.mat_device_status.argtypes = [C.POINTER(C.c_int)]
    lib.mat_sparse_attn_fwd.restype = C.c_int
    lib.mat_sparse_attn_fwd.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, C.c_int, spec_p,
                                        C.c_float, vp, sz, vp]
    lib.mat_sparse_attn_fwd_strided.restype = C.c_int
    lib.mat_sparse_attn_fwd_strided.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, C.c_int, spec_p,
                                                C.c_float, i64, i64, i64, i64, vp]
    lib.mat_sparse_attn_workspace_bytes.restype = sz
    lib.mat_sparse_attn_workspace_bytes.argtypes = [i64, i64, i64, i64, i64, C.c_int, spec_p]
    lib.mat_sparse_attn_fwd_window.restype = C.c_int
    lib.mat_sparse_attn_fwd_window.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, C.c_int, i64, vp]
    lib.mat_sparse_attn_fwd_sharded.restype = C.c_int
    lib.mat_sparse_attn_fwd_sharded.argtypes = [vp, vp, vp, vp, vp, vp, i64, vp, vp, i64, i64, i64, i64, i64,
                                                C.c_int, spec_p, C.c_float, vp]
    lib.mat_sparse_attn_fwd_longformer_noalloc.restype = C.c_int
    lib.mat_sparse_attn_fwd_longformer_noalloc.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, C.c_int, spec_p,
                                                           C.c_float, vp]
    lib.mat_sparse_attn_bwd.restype = C.c_int
    lib.mat_sparse_attn_bwd.argtypes = [vp] * 7 + [i64, i64, i64, i64, C.c_int, spec_p, C.c_float, vp, sz, vp]
    lib.mat_sparse_attn_bwd_general.restype = C.c_int
    lib.mat_sparse_attn_bwd_general.argtypes = [vp] * 7 + [i64, i64, i64, i64, C.c_int, spec_p, vp, vp, C.c_float, vp, sz, vp]
    lib.mat_sparse_attn_bwd_general_workspace_bytes.restype = sz
    lib.mat_sparse_attn_bwd_general_workspace_bytes.argtypes = [i64, i64, i64, i64, C.c_int, spec_p]
    lib.mat_sparse_attn_bwd_workspace_bytes.restype = sz
    lib.mat_sparse_attn_bwd_workspace_bytes.argtypes = [i64, i64, i64]
    lib.mat_longformer_shard_fwd.restype = C.c_int
    lib.mat_longformer_shard_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i64, vp, vp, i64, vp, vp, vp, i64,
                                             i64, i64, i64, i64, C.c_int, i64, i64, C.c_float, vp]
    lib.mat_global_rows_partial_layout.restype = sz
    lib.mat_global_rows_partial_layout.argtypes = [i64, i64, i64, i64, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.mat_global_rows_partial.restype = C.c_int
    lib.mat_global_rows_partial.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, C.c_int, C.c_float, vp]
    lib.mat_global_rows_merge.restype = C.c_int
    lib.mat_global_rows_merge.argtypes = [vp, i64, i64, vp, vp, i64, i64, i64, i64, i64, C.c_int32, C.c_int32,
                                          C.c_int, C.c_float, vp]
    lib.mat_enable_peer_access.restype = C.c_int
    lib.mat_enable_peer_access.argtypes = [C.c_int, C.c_int]
    lib.mat_ipc_export.restype = C.c_int
    lib.mat_ipc_export.argtypes = [vp, vp, C.POINTER(i64)]
    lib.mat_ipc_open.restype = C.c_int
    lib.mat_ipc_open.argtypes = [vp, C.c_int, C.POINTER(vp)]
    lib.mat_ipc_close.restype = C.c_int
    lib.mat_ipc_close.argtypes = [vp, C.c_int]
    lib.mat_sparse_attn_fwd_host.restype = C.c_int
    lib.mat_sparse_attn_fwd_host.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, C.c_int, spec_p,
                                             C.c_float, vp, sz, C.c_int]
    lib.mat_sparse_attn_host_staging_bytes.restype = sz
    lib.mat_sparse_attn_host_staging_bytes.argtypes = [i64, i64, i64, i64, C.c_int, spec_p]
    lib.mat_pattern_rowset.restype = C.c_int
    lib.mat_pattern_rowset.argtypes = [spec_p, i64, i64, vp, i64, C.POINTER(i64)]
    lib.mat_pattern_nnz.restype = C.c_int
    lib.mat_pattern_nnz.argtypes = [spec_p, i64, i64, C.POINTER(i64)]
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != MAT_OK:
        raise NativeError(lib.mat_last_error().decode("utf-8", "replace") or f"error code {rc}")


def last_kernel() -> str:
    return lib.mat_last_kernel().decode()


def device_status() -> int:
    out = C.c_int(0)
    check(lib.mat_device_status(C.byref(out)))
    return out.value
