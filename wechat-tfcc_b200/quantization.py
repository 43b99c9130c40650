"""Quantized matmul and its integer sums on the B200 backend.

Mirrors the free functions ``tfcc::mkl::quantization::matmul`` and
``reduce_sum`` (tfcc/mkl/operations/tfcc_mklquantization.h:39-51): same
arguments, same checks and messages (tfcc_mklquantization.cpp:75-118,
:284-289), same results.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import exceptions
from ._lib import PATHS, check, lib
from .session import get_session

_REDUCE = {torch.uint8: "tfccb200_reduce_sum_u8", torch.int8: "tfccb200_reduce_sum_s8",
           torch.int16: "tfccb200_reduce_sum_s16"}


_TYPE_IDS = {torch.int8: 0, torch.uint8: 1, torch.int16: 2, torch.uint16: 3, torch.int32: 4,
             torch.uint32: 5}


def _scalar(t, name, device):
    """A (min or max) range tensor: one float32 element, rank 1, on the operand's device."""
    if not isinstance(t, torch.Tensor) or t.numel() != 1 or t.dim() != 1:
        raise exceptions.InvalidArgumentError(f"invalid {name}")
    if t.dtype != torch.float32 or t.device != device or not t.is_contiguous():
        raise exceptions.InvalidArgumentError(f"invalid {name}: expected float32 on {device}")
    return t


def quantize(a: torch.Tensor, dtype, min_value=None, max_value=None):
    """``tfcc::quantization::quantize<T>``: with no range, ``(q, min, max)`` where the range is
    reduced from ``a`` on the device; with ``min_value`` / ``max_value`` (one-element device
    tensors), just ``q``.  No host synchronisation either way."""
    if not isinstance(a, torch.Tensor) or a.numel() == 0:
        raise exceptions.InvalidArgumentError("invalid tensor")
    if dtype not in _TYPE_IDS:
        raise exceptions.NotImplementedError(f"quantize is not implemented for {dtype}")
    _dev(a, "a", torch.float32)
    sess = get_session(a.device)
    out = torch.empty(a.shape, dtype=dtype, device=a.device)
    with torch.cuda.device(a.device):
        if min_value is None and max_value is None:
            rng = torch.empty(2, dtype=torch.float32, device=a.device)
            check(lib.tfccb200_minmax_f32(sess.stream_ptr, a.data_ptr(), a.numel(), rng.data_ptr()))
            mn, mx = rng[0:1], rng[1:2]
            check(lib.tfccb200_quantize_f32(sess.stream_ptr, a.data_ptr(), a.numel(), mn.data_ptr(),
                                            mx.data_ptr(), out.data_ptr(), _TYPE_IDS[dtype]))
            return out, mn, mx
        mn = _scalar(min_value, "minValue", a.device)
        mx = _scalar(max_value, "maxValue", a.device)
        check(lib.tfccb200_quantize_f32(sess.stream_ptr, a.data_ptr(), a.numel(), mn.data_ptr(),
                                        mx.data_ptr(), out.data_ptr(), _TYPE_IDS[dtype]))
    return out


def quantize_with_row_sums(a: torch.Tensor, dtype, min_value=None, max_value=None):
    """``quantize`` and ``reduce_sum(q, row=True)`` in one pass over ``a`` (rank >= 2):
    ``(q, row_sums)`` for a given range, ``(q, min, max, row_sums)`` when the range is reduced
    from ``a`` here.  Same values as the two separate calls."""
    if not isinstance(a, torch.Tensor) or a.numel() == 0 or a.dim() < 2:
        raise exceptions.InvalidArgumentError("invalid tensor")
    if dtype not in _REDUCE:
        raise exceptions.NotImplementedError(f"row sums exist for int8/uint8/int16, got {dtype}")
    _dev(a, "a", torch.float32)
    sess = get_session(a.device)
    cols = a.shape[-1]
    rows = a.numel() // cols
    out = torch.empty(a.shape, dtype=dtype, device=a.device)
    sums = torch.empty(a.shape[:-1], dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        given = min_value is not None or max_value is not None
        if given:
            mn = _scalar(min_value, "minValue", a.device)
            mx = _scalar(max_value, "maxValue", a.device)
        else:
            rng = torch.empty(2, dtype=torch.float32, device=a.device)
            check(lib.tfccb200_minmax_f32(sess.stream_ptr, a.data_ptr(), a.numel(), rng.data_ptr()))
            mn, mx = rng[0:1], rng[1:2]
        check(lib.tfccb200_quantize_rowsum_f32(sess.stream_ptr, a.data_ptr(), rows, cols,
                                               mn.data_ptr(), mx.data_ptr(), out.data_ptr(),
                                               _TYPE_IDS[dtype], sums.data_ptr()))
    return (out, sums) if given else (out, mn, mx, sums)


def dequantize(a: torch.Tensor, min_value, max_value) -> torch.Tensor:
    """``tfcc::quantization::dequantize``: float32 values of a quantized tensor."""
    if not isinstance(a, torch.Tensor) or a.numel() == 0:
        raise exceptions.InvalidArgumentError("invalid tensor")
    if a.dtype not in _TYPE_IDS:
        raise exceptions.NotImplementedError(f"dequantize is not implemented for {a.dtype}")
    _dev(a, "a")
    mn = _scalar(min_value, "minValue", a.device)
    mx = _scalar(max_value, "maxValue", a.device)
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_dequantize_f32(sess.stream_ptr, a.data_ptr(), _TYPE_IDS[a.dtype],
                                          a.numel(), mn.data_ptr(), mx.data_ptr(), out.data_ptr()))
    return out


def requantize(a: torch.Tensor, min_input, max_input, min_output, max_output, dtype) -> torch.Tensor:
    """``tfcc::quantization::requantize<T>``: quantized ``a`` re-expressed in ``dtype`` over the
    output range."""
    if not isinstance(a, torch.Tensor) or a.numel() == 0:
        raise exceptions.InvalidArgumentError("invalid tensor")
    if a.dtype not in _TYPE_IDS or dtype not in _TYPE_IDS:
        raise exceptions.NotImplementedError("requantize is implemented for 8/16/32-bit integers")
    _dev(a, "a")
    r = [_scalar(t, n, a.device) for t, n in ((min_input, "minInput"), (max_input, "maxInput"),
                                              (min_output, "minOutput"), (max_output, "maxOutput"))]
    out = torch.empty(a.shape, dtype=dtype, device=a.device)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_requantize(sess.stream_ptr, a.data_ptr(), _TYPE_IDS[a.dtype], a.numel(),
                                      r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr(),
                                      r[3].data_ptr(), out.data_ptr(), _TYPE_IDS[dtype]))
    return out


def _dev(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
        raise exceptions.InvalidArgumentError(f"invalid tensor {name}")
    if dtype is not None and t.dtype != dtype:
        raise exceptions.InvalidArgumentError(f"invalid tensor {name}: expected {dtype}")


def reduce_sum(a: torch.Tensor, row: bool) -> torch.Tensor:
    """int32 sums over the last dimension (``row``) or the second-to-last (not ``row``)."""
    if not isinstance(a, torch.Tensor) or a.numel() == 0 or a.dim() < 2:
        raise exceptions.InvalidArgumentError("invalid input tensor a")
    if a.dtype not in _REDUCE:
        raise exceptions.NotImplementedError(f"reduce_sum is implemented for int8/uint8/int16, got {a.dtype}")
    _dev(a, "a")
    r, c = a.shape[-2], a.shape[-1]
    batch = a.numel() // (r * c)
    shape = list(a.shape[:-2]) + [r if row else c]
    out = torch.empty(shape, dtype=torch.int32, device=a.device)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        st = getattr(lib, _REDUCE[a.dtype])(sess.stream_ptr, a.data_ptr(), batch, r, c,
                                           1 if row else 0, out.data_ptr())
    check(st)
    return out


def matmul_params(min_a: float, max_a: float, min_b: float, max_b: float):
    """(offA, offB, minC, maxC) exactly as the reference derives them on the host."""
    oa, ob = C.c_int32(), C.c_int32()
    mn, mx = C.c_float(), C.c_float()
    check(lib.tfccb200_quantized_matmul_params(min_a, max_a, min_b, max_b, C.byref(oa),
                                               C.byref(ob), C.byref(mn), C.byref(mx)))
    return oa.value, ob.value, mn.value, mx.value


def matmul(a, reduce_sum_a, min_a, max_a, b, reduce_sum_b, min_b, max_b, *, path: str = "auto"):
    """Returns ``(C int32, minC float[1], maxC float[1])``.

    ``min_*`` / ``max_*`` are one-element float tensors as in the reference.  When all four
    live on the operands' device the zero-point offsets and the result range are derived
    there by a prologue kernel and nothing returns to the host; ranges given as CPU tensors
    are read on the host instead.
    """
    if not isinstance(a, torch.Tensor) or a.numel() == 0 or a.dim() < 2:
        raise exceptions.InvalidArgumentError("invalid input tensor a")
    if reduce_sum_a.numel() == 0:
        raise exceptions.InvalidArgumentError("invalid tensor reduceSumA")
    for t, nm in ((min_a, "minA"), (max_a, "maxA")):
        if t.numel() != 1 or t.dim() != 1:
            raise exceptions.InvalidArgumentError(f"invalid tensor {nm}")
    if not isinstance(b, torch.Tensor) or b.numel() == 0 or b.dim() < 2:
        raise exceptions.InvalidArgumentError("invalid input tensor b")
    if reduce_sum_b.numel() == 0:
        raise exceptions.InvalidArgumentError("invalid tensor reduceSumB")
    for t, nm in ((min_b, "minB"), (max_b, "maxB")):
        if t.numel() != 1 or t.dim() != 1:
            raise exceptions.InvalidArgumentError(f"invalid tensor {nm}")
    if a.shape[-1] != b.shape[-2]:
        raise exceptions.InvalidArgumentError("tensor a and b don't match")
    if a.dim() != b.dim() and a.dim() != 2 and b.dim() != 2:
        raise exceptions.InvalidArgumentError("tensor a and b don't match")
    if a.shape[-2] != reduce_sum_a.shape[-1]:
        raise exceptions.InvalidArgumentError("tensor a and reduceSumA don't match")
    if b.shape[-1] != reduce_sum_b.shape[-1]:
        raise exceptions.InvalidArgumentError("tensor b and reduceSumB don't match")
    if a.dim() == b.dim() and tuple(a.shape[:-2]) != tuple(b.shape[:-2]):
        raise exceptions.InvalidArgumentError("tensor a and b don't match")
    _dev(a, "a", torch.uint8)
    _dev(b, "b", torch.int8)
    _dev(reduce_sum_a, "reduceSumA", torch.int32)
    _dev(reduce_sum_b, "reduceSumB", torch.int32)

    lead = list(a.shape[:-2]) if a.dim() >= b.dim() else list(b.shape[:-2])
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    result = torch.empty(lead + [m, n], dtype=torch.int32, device=a.device)
    batch = result.numel() // (m * n)
    stride_rs_a = 0 if reduce_sum_a.dim() == 1 else m
    stride_rs_b = 0 if reduce_sum_b.dim() == 1 else n
    stride_a = 0 if a.dim() == 2 else m * k
    stride_b = 0 if b.dim() == 2 else k * n
    sess = get_session(a.device)
    ranges = (min_a, max_a, min_b, max_b)
    if all(t.device == a.device and t.dtype == torch.float32 and t.is_contiguous() for t in ranges):
        out_range = torch.empty(2, dtype=torch.float32, device=a.device)
        offsets = torch.empty(2, dtype=torch.int32, device=a.device)
        with torch.cuda.device(a.device):
            st = lib.tfccb200_qgemm_u8s8s32_dev(
                sess.stream_ptr, a.data_ptr(), stride_a, reduce_sum_a.data_ptr(), stride_rs_a,
                min_a.data_ptr(), max_a.data_ptr(), b.data_ptr(), stride_b, reduce_sum_b.data_ptr(),
                stride_rs_b, min_b.data_ptr(), max_b.data_ptr(), result.data_ptr(), m * n,
                out_range.data_ptr(), out_range.data_ptr() + 4, offsets.data_ptr(), m, n, k, batch,
                PATHS[path], sess.status_ptr)
        check(st)
        return result, out_range[0:1], out_range[1:2]
    off_a, off_b, min_c, max_c = matmul_params(float(min_a.item()), float(max_a.item()),
                                               float(min_b.item()), float(max_b.item()))
    with torch.cuda.device(a.device):
        st = lib.tfccb200_qgemm_u8s8s32_ex(
            sess.stream_ptr, a.data_ptr(), stride_a, reduce_sum_a.data_ptr(), stride_rs_a, off_a,
            b.data_ptr(), stride_b, reduce_sum_b.data_ptr(), stride_rs_b, off_b,
            result.data_ptr(), m * n, m, n, k, batch, PATHS[path], sess.status_ptr)
    check(st)
    min_r = torch.tensor([min_c], dtype=torch.float32, device=a.device)
    max_r = torch.tensor([max_c], dtype=torch.float32, device=a.device)
    return result, min_r, max_r


def matmul_host(a, b, min_a, max_a, min_b, max_b):
    """Host-buffer round trip of reduce_sum(a,row), reduce_sum(b,col) and matmul:
    numpy uint8 / int8 in, ``(int32 array, minC, maxC)`` out (synchronous)."""
    import numpy as np

    a = np.ascontiguousarray(a, dtype=np.uint8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    if a.ndim < 2 or b.ndim < 2 or a.shape[-1] != b.shape[-2]:
        raise exceptions.InvalidArgumentError("tensor a and b don't match")
    if a.ndim != b.ndim and a.ndim != 2 and b.ndim != 2:
        raise exceptions.InvalidArgumentError("tensor a and b don't match")
    lead = list(a.shape[:-2]) if a.ndim >= b.ndim else list(b.shape[:-2])
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    out = np.empty(lead + [m, n], dtype=np.int32)
    batch = out.size // (m * n)
    stride_a = 0 if a.ndim == 2 else m * k
    stride_b = 0 if b.ndim == 2 else k * n
    mn, mx = C.c_float(), C.c_float()
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.tfccb200_qgemm_u8s8s32_host(stream, a.ctypes.data, stride_a, b.ctypes.data, stride_b,
                                         float(min_a), float(max_a), float(min_b), float(max_b),
                                         out.ctypes.data, m * n, C.byref(mn), C.byref(mx), m, n,
                                         k, batch)
    check(st)
    return out, mn.value, mx.value
