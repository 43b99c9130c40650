"""``tfcc::blas::matmul`` on the B200 backend.

Shape rules, the empty-tensor short cut and the error cases follow
tfcc/core/operations/tfcc_blas.cpp:26-96; strides and batch count follow
tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-186.
"""
from __future__ import annotations

import torch

from . import exceptions
from ._lib import ACTIVATIONS, PATHS, PRECISIONS, check, lib
from .session import get_session


def _result_shape(a, b):
    if a.dim() < 2 or b.dim() < 2:
        raise exceptions.InvalidArgumentError("matmul require tensors with two or more dimensions")
    if a.dim() != b.dim() and a.dim() != 2 and b.dim() != 2:
        raise exceptions.InvalidArgumentError("shape invalid")
    if a.shape[-1] != b.shape[-2]:
        raise exceptions.InvalidArgumentError("shape invalid")
    if a.dim() == b.dim() and tuple(a.shape[:-2]) != tuple(b.shape[:-2]):
        raise exceptions.InvalidArgumentError("shape invalid")
    lead = list(a.shape[:-2]) if a.dim() > b.dim() or a.dim() == b.dim() else list(b.shape[:-2])
    return lead + [a.shape[-2], b.shape[-1]]


def _check_operand(t, name):
    if not isinstance(t, torch.Tensor):
        raise exceptions.InvalidArgumentError(f"{name} must be a tensor")
    if t.dtype != torch.float32:
        # the reference's CPU backend implements float only
        # (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:35-39)
        raise exceptions.NotImplementedError(f"matmul is implemented for float32, got {t.dtype}")
    if not t.is_cuda:
        raise exceptions.InvalidArgumentError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise exceptions.InvalidArgumentError(f"{name} must be contiguous row-major")


def matmul(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None = None, *,
           precision: str = "fp32", path: str = "auto", activation: str | None = None) -> torch.Tensor:
    """``a . b`` (+ ``c`` broadcast over rows).  Batched when either operand has rank > 2;
    a rank-2 operand is shared by every batch entry.  Asynchronous on the current stream.
    ``activation="gelu"`` applies the erf GELU to the result inside the GEMM epilogue."""
    for t, nm in ((a, "a"), (b, "b")) + (((c, "c"),) if c is not None else ()):
        if not isinstance(t, torch.Tensor):
            raise exceptions.InvalidArgumentError(f"{nm} must be a tensor")
    shape = _result_shape(a, b)
    if c is not None and (c.dim() != 1 or c.numel() != b.shape[-1]):
        raise exceptions.InvalidArgumentError("shape invalid")
    _check_operand(a, "a")
    _check_operand(b, "b")
    if c is not None:
        _check_operand(c, "c")
    if a.device != b.device or (c is not None and c.device != a.device):
        raise exceptions.InvalidArgumentError("operands live on different devices")
    result = torch.empty(shape, dtype=torch.float32, device=a.device)
    if a.numel() == 0 or b.numel() == 0:
        return result  # uninitialised, as in the reference
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    stride_a, stride_b, stride_c = m * k, n * k, m * n
    if a.dim() != b.dim():
        stride_a = 0 if a.dim() == 2 else stride_a
        stride_b = 0 if b.dim() == 2 else stride_b
    batch = result.numel() // (m * n)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        ws_bytes = lib.tfccb200_sgemm_workspace(m, n, k, batch, PRECISIONS[precision])
        ws_ptr, ws_len = sess.workspace(ws_bytes)
        st = lib.tfccb200_sgemm_act(
            sess.stream_ptr, a.data_ptr(), stride_a, b.data_ptr(), stride_b, result.data_ptr(),
            stride_c, c.data_ptr() if c is not None else None, m, n, k, batch,
            PRECISIONS[precision], PATHS[path], ACTIVATIONS[activation], ws_ptr, ws_len,
            sess.status_ptr)
    check(st)
    return result


def matmul_host(a, b, c=None, *, precision: str = "fp32"):
    """Host-buffer round trip: numpy float32 arrays in, numpy array out (synchronous).
    Uploads the operands, multiplies on the current CUDA device and downloads the product."""
    import numpy as np

    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    shape = _result_shape(ta, tb)
    out = np.empty(shape, dtype=np.float32)
    if a.size == 0 or b.size == 0:
        return out
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    stride_a, stride_b, stride_c = m * k, n * k, m * n
    if a.ndim != b.ndim:
        stride_a = 0 if a.ndim == 2 else stride_a
        stride_b = 0 if b.ndim == 2 else stride_b
    batch = out.size // (m * n)
    bias_ptr = None
    if c is not None:
        c = np.ascontiguousarray(c, dtype=np.float32)
        if c.ndim != 1 or c.size != n:
            raise exceptions.InvalidArgumentError("shape invalid")
        bias_ptr = c.ctypes.data
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.tfccb200_sgemm_host(stream, a.ctypes.data, stride_a, b.ctypes.data, stride_b,
                                 out.ctypes.data, stride_c, bias_ptr, m, n, k, batch,
                                 PRECISIONS[precision])
    check(st)
    return out
