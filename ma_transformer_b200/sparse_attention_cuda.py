"""Drop-in for the reference's torch extension module ``sparse_attention_cuda``
(src/cuda/sparse_attention_kernel.cu:501-510): same function names, keyword
names, argument meaning and error type, served by libmat_sparse_attn through
its C ABI.  Additions: ``forward_pattern`` (causal / dilated / block-sparse /
Longformer key sets) and ``forward_host`` (host tensors in, host tensor out).

Differences from the reference extension, all relaxations:
  * bf16 and fp16 inputs run natively (the reference accepts fp32 only,
    sparse_attention_kernel.cu:428-429, and its bridge sends 16-bit inputs to a
    python loop, src/layers/ma_core_bridge.py:77-79);
There is no CPU fallback: CPU tensors raise RuntimeError here exactly as in the
reference ("Inputs must be CUDA tensors"); use ``forward_host`` for those.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch

from . import _native as nat
from .patterns import PatternSpec, WINDOW, BLOCK

_DTYPES = {torch.float32: nat.MAT_F32, torch.bfloat16: nat.MAT_BF16, torch.float16: nat.MAT_F16}
_workspaces: Dict[tuple, torch.Tensor] = {}


def _check_inputs(*tensors: torch.Tensor) -> None:
    # the reference's five TORCH_CHECKs (sparse_attention_kernel.cu:427-432)
    if not all(t.is_cuda for t in tensors):
        raise RuntimeError("Inputs must be CUDA tensors")
    dt = tensors[0].dtype
    if dt not in _DTYPES or any(t.dtype != dt for t in tensors):
        raise RuntimeError("Only float32, bfloat16 and float16 are supported in CUDA path "
                           "(all inputs of one dtype)")
    if not all(t.is_contiguous() for t in tensors):
        raise RuntimeError("Inputs must be contiguous")
    if any(t.dim() != 4 for t in tensors):
        raise RuntimeError("Expected shape [B, S, H, D]")
    if any(t.device != tensors[0].device for t in tensors):
        raise RuntimeError("Inputs must be on the same device")


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch buffer of at least ``nbytes`` for work on torch's current stream of ``device``.

    One buffer per (device, stream): calls issued on one stream reuse it in stream order, calls on
    different streams get different buffers and cannot race.  A buffer that has to grow is replaced;
    the old one goes back to torch's allocator on the stream that used it, which orders its reuse
    behind the kernels still reading it.
    """
    device = torch.device(device)
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        with torch.cuda.device(device):
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def forward_pattern(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    spec: PatternSpec, scale: Optional[float] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sparse-attention forward for any ``PatternSpec``.

    query: [B, S_q, H, D]; key, value: [B, S_kv, H, D] with
    S_kv >= S_q + spec.q_offset (a sequence shard passes its halo rows in key and
    value).  Asynchronous on torch's current stream; returns [B, S_q, H, D] in the
    inputs' dtype.
    """
    _check_inputs(query, key, value)
    if key.shape != value.shape or query.shape[0] != key.shape[0] or query.shape[2:] != key.shape[2:]:
        raise RuntimeError("Q,K,V must have same shape (key/value may only differ from query in length)")
    B, Sq, H, D = query.shape
    Skv = key.shape[1]
    spec.check_against(Skv)
    if out is None:
        out = torch.empty_like(query)
    else:
        _check_inputs(out)
        if out.shape != query.shape or out.dtype != query.dtype:
            raise RuntimeError("out must match query in shape and dtype")
    dt = _DTYPES[query.dtype]
    with torch.cuda.device(query.device):
        s = spec.device_struct(query.device)
        ws_bytes = nat.lib.mat_sparse_attn_workspace_bytes(B, Sq, Skv, H, D, dt, C.byref(s))
        ws = _workspace(query.device, ws_bytes) if ws_bytes else None
        stream = torch.cuda.current_stream(query.device).cuda_stream
        nat.check(nat.lib.mat_sparse_attn_fwd(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), B, Sq, Skv, H, D, dt,
            C.byref(s), float(scale) if scale else 0.0,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            C.c_void_p(stream)))
    return out


def _token_stride(t: torch.Tensor) -> Optional[int]:
    """Elements between consecutive tokens of a [B, S, H, D] tensor whose heads and head columns are packed
    and whose batch items follow each other (a view of a fused projection output), or None."""
    B, S, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D:
        return None
    ts = t.stride(1)
    if ts < H * D or ts % 8 or (B > 1 and t.stride(0) != S * ts):
        return None
    return int(ts)


def forward_strided(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, spec: PatternSpec,
                    scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``forward_pattern`` for tensors whose tokens are not packed: views of one fused projection output
    [B, S, 3, H, D] (``qkv[:, :, 0]`` and so on) go to the kernels as they are, without the copy that
    ``.contiguous()`` would make.  Heads and head columns must be packed; window patterns of at most 128 taps,
    16-bit dtypes, D = 64.  ``out`` defaults to a packed tensor."""
    for t in (query, key, value):
        if not t.is_cuda:
            raise RuntimeError("Inputs must be CUDA tensors")
        if t.dim() != 4:
            raise RuntimeError("Expected shape [B, S, H, D]")
    if query.dtype not in _DTYPES or key.dtype != query.dtype or value.dtype != query.dtype:
        raise RuntimeError("Only float32, bfloat16 and float16 are supported in CUDA path (all inputs of one dtype)")
    if key.shape != value.shape or query.shape[0] != key.shape[0] or query.shape[2:] != key.shape[2:]:
        raise RuntimeError("Q,K,V must have same shape (key/value may only differ from query in length)")
    B, Sq, H, D = query.shape
    Skv = key.shape[1]
    spec.check_against(Skv)
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=query.dtype, device=query.device)
    strides = [_token_stride(t) for t in (query, key, value, out)]
    if any(s is None for s in strides):
        raise RuntimeError("Inputs must be contiguous, or views with packed heads and a uniform token stride "
                           "that is a multiple of 8 elements")
    with torch.cuda.device(query.device):
        s = spec.device_struct(query.device)
        stream = torch.cuda.current_stream(query.device).cuda_stream
        nat.check(nat.lib.mat_sparse_attn_fwd_strided(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), B, Sq, Skv, H, D,
            _DTYPES[query.dtype], C.byref(s), float(scale) if scale else 0.0, *strides, C.c_void_p(stream)))
    return out


def forward_sharded(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, spec: PatternSpec,
                    prev_kv=None, next_kv=None, scale: Optional[float] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Forward of one sequence shard [B, S, H, 64]; ``prev_kv`` / ``next_kv`` are
    ``(key, value)`` pairs of the neighbouring shards, usually tensors that live on
    another GPU and are mapped into this process (see ``sharded.PeerHaloAttention``).
    The edge tiles read the halo rows from them inside the kernel."""
    _check_inputs(query, key, value)
    if not (query.shape == key.shape == value.shape):
        raise RuntimeError("Q,K,V must have same shape")
    B, S, H, D = query.shape
    if out is None:
        out = torch.empty_like(query)

    def side(kv):
        if kv is None:
            return None, None, 0
        k, v = kv
        if k.dtype != query.dtype or v.dtype != query.dtype or not (k.is_contiguous() and v.is_contiguous()):
            raise RuntimeError("neighbour tensors must be contiguous and of the query's dtype")
        if k.shape != v.shape or k.dim() != 4 or k.shape[0] != B or tuple(k.shape[2:]) != (H, D):
            raise RuntimeError("neighbour tensors must be [B, S_neighbour, H, D]")
        return k.data_ptr(), v.data_ptr(), k.shape[1]

    kp, vp, sp = side(prev_kv)
    kn, vn, sn = side(next_kv)
    with torch.cuda.device(query.device):
        s = spec.device_struct(query.device)
        stream = torch.cuda.current_stream(query.device).cuda_stream
        nat.check(nat.lib.mat_sparse_attn_fwd_sharded(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), kp, vp, sp, kn, vn, sn,
            B, S, H, D, _DTYPES[query.dtype], C.byref(s), float(scale) if scale else 0.0, C.c_void_p(stream)))
    return out


def forward_longformer_noalloc(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                               spec: PatternSpec, out: torch.Tensor,
                               scale: Optional[float] = None) -> torch.Tensor:
    """Longformer forward for callers that may not allocate device memory while they
    run (an inference server whose arena already owns all of HBM, a latency-critical
    loop that cannot take the device-wide stall of an allocation).  ``out`` must be
    supplied; this function and the library call below it allocate nothing on the
    device, and the scratch of the global-row pass is a fixed 4 MiB array inside the
    library.  16-bit inputs, D = 64; B*H*ceil64(globals)*264 bytes must fit in 4 MiB
    (RuntimeError otherwise: use ``forward_pattern``).  All calls on a device share
    that array, so calls that overlap on the GPU race: keep them on one stream.  The
    first call on a device resolves the array's address; make it before any stream
    capture.  ``spec`` must already have been used on this device, or be given
    device arrays before the no-allocation phase starts (its global positions are
    uploaded once, on first use)."""
    _check_inputs(query, key, value, out)
    if not (query.shape == key.shape == value.shape == out.shape):
        raise RuntimeError("Q,K,V and out must have same shape")
    B, S, H, D = query.shape
    spec.check_against(S)
    with torch.cuda.device(query.device):
        s = spec.device_struct(query.device)
        stream = torch.cuda.current_stream(query.device).cuda_stream
        nat.check(nat.lib.mat_sparse_attn_fwd_longformer_noalloc(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), B, S, H, D,
            _DTYPES[query.dtype], C.byref(s), float(scale) if scale else 0.0, C.c_void_p(stream)))
    return out


def forward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
            window_size: int = 64) -> torch.Tensor:
    """Sparse attention forward (CUDA): keys [i-window_size, i+window_size].

    Same call as the reference's ``sparse_attention_cuda.forward``
    (sparse_attention_kernel.cu:423-458); ``window_size`` 0 is legal (a query
    attends to itself only) and values beyond S clamp.
    """
    _check_inputs(query, key, value)
    if query.shape != key.shape or key.shape != value.shape:
        raise RuntimeError("Q,K,V must have same shape")
    B, S, H, D = query.shape
    out = torch.empty_like(query)
    with torch.cuda.device(query.device):
        stream = torch.cuda.current_stream(query.device).cuda_stream
        nat.check(nat.lib.mat_sparse_attn_fwd_window(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), B, S, H, D,
            _DTYPES[query.dtype], int(window_size), C.c_void_p(stream)))
    return out


def dense_forward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                  use_causal_mask: bool = False) -> torch.Tensor:
    """Dense attention forward (CUDA), the call of sparse_attention_kernel.cu:348-382,
    expressed as the window that covers the whole sequence (left = S, right = S or
    0 when causal) and run by the same kernels."""
    _check_inputs(query, key, value)
    if query.shape != key.shape or key.shape != value.shape:
        raise RuntimeError("Q,K,V must have same shape")
    S = query.shape[1]
    spec = PatternSpec(WINDOW, left=S, right=0 if use_causal_mask else S)
    return forward_pattern(query, key, value, spec)


def forward_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, spec: PatternSpec,
                 scale: Optional[float] = None, device: int = 0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Forward for HOST tensors: copies in, computes on ``cuda:device``, copies out.

    The counterpart of handing CPU tensors to the reference's CPU engine
    (src/layers/ma_core_bridge.py:102-112).  Pinned tensors make the copies
    asynchronous and let them overlap the compute; the call returns when ``out``
    is complete.
    """
    for t in (query, key, value):
        if t.is_cuda:
            raise RuntimeError("forward_host expects CPU tensors")
        if t.dim() != 4:
            raise RuntimeError("Expected shape [B, S, H, D]")
        if not t.is_contiguous():
            raise RuntimeError("Inputs must be contiguous")
    if query.shape != key.shape or key.shape != value.shape:
        raise RuntimeError("Q,K,V must have same shape")
    if query.dtype not in _DTYPES or key.dtype != query.dtype or value.dtype != query.dtype:
        raise RuntimeError("Only float32, bfloat16 and float16 are supported")
    B, S, H, D = query.shape
    spec.check_against(S)
    dt = _DTYPES[query.dtype]
    dev = torch.device("cuda", device)
    if out is None:
        out = torch.empty_like(query)
    with torch.cuda.device(dev):
        s = spec.device_struct(dev)
        nbytes = nat.lib.mat_sparse_attn_host_staging_bytes(B, S, H, D, dt, C.byref(s))
        staging = _workspace(dev, nbytes)
        torch.cuda.current_stream(dev).synchronize()  # staging may still be in use by earlier work
        nat.check(nat.lib.mat_sparse_attn_fwd_host(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), B, S, H, D, dt,
            C.byref(s), float(scale) if scale else 0.0, staging.data_ptr(), staging.numel(), device))
    return out


def backward_pattern(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, grad_out: torch.Tensor,
                     spec: PatternSpec, scale: Optional[float] = None) -> List[torch.Tensor]:
    """[dQ, dK, dV] of any pattern by the library's backward kernels: deterministic, no atomics.  Window
    patterns (sliding, causal, dilated, dense-as-window) with 16-bit inputs and D = 64 run on tensor-core
    kernels; block layouts and the Longformer pattern on the warp-level kernels with fp32 math."""
    _check_inputs(query, key, value, grad_out)
    if not (query.shape == key.shape == value.shape == grad_out.shape):
        raise RuntimeError("All tensors must have same shape")
    B, S, H, D = query.shape
    dq, dk, dv = torch.empty_like(query), torch.empty_like(key), torch.empty_like(value)
    with torch.cuda.device(query.device):
        s = spec.device_struct(query.device)
        ws = _workspace(query.device, nat.lib.mat_sparse_attn_bwd_general_workspace_bytes(
            B, S, H, D, _DTYPES[query.dtype], C.byref(s)))
        stream = torch.cuda.current_stream(query.device).cuda_stream
        t_rp = t_ci = None
        if spec.kind == BLOCK:   # the dK / dV pass walks the transposed layout
            t_rp, t_ci = spec.device_transposed_layout(query.device)
        nat.check(nat.lib.mat_sparse_attn_bwd_general(
            query.data_ptr(), key.data_ptr(), value.data_ptr(), grad_out.data_ptr(), dq.data_ptr(), dk.data_ptr(),
            dv.data_ptr(), B, S, H, D, _DTYPES[query.dtype], C.byref(s),
            t_rp.data_ptr() if t_rp is not None else None, t_ci.data_ptr() if t_ci is not None else None,
            float(scale) if scale else 0.0, ws.data_ptr(), ws.numel(), C.c_void_p(stream)))
    return [dq, dk, dv]


def backward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, grad_out: torch.Tensor,
             window_size: int = 64) -> List[torch.Tensor]:
    """Sparse attention backward (CUDA) -> [dQ, dK, dV]; the call of
    sparse_attention_kernel.cu:460-497 (keys [i-window_size, i+window_size])."""
    return backward_pattern(query, key, value, grad_out, PatternSpec.sliding_window(int(window_size)))


def dense_backward(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                   grad_out: torch.Tensor, use_causal_mask: bool = False) -> List[torch.Tensor]:
    """Dense attention backward (CUDA) -> [dQ, dK, dV]; the call of
    sparse_attention_kernel.cu:384-421, as the window that covers the sequence."""
    S = query.shape[1] if query.dim() == 4 else 0
    return backward_pattern(query, key, value, grad_out,
                            PatternSpec(WINDOW, left=S, right=0 if use_causal_mask else S))
