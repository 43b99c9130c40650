"""TEST INFRASTRUCTURE -- CPU oracle of the TFCC matmul hot path.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product never does.

What it restates, and from where (paths relative to the reference tree):

* ``blas_matmul``        shape rules of ``tfcc::blas::matmul``
                         (tfcc/core/operations/tfcc_blas.cpp:26-96) and the batch /
                         broadcast strides of ``MKLBlasInterface<float>::matmul``
                         (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-186).  The
                         arithmetic itself is a third-party dependency that is not in
                         the reference tree -- oneDNN v1.8.1 ``dnnl::matmul``
                         (pinned in build.sh:19-23) -- so the oracle computes the
                         mathematically exact product in float64 and, as the stand-in
                         for "the reference's fp32 result", numpy's float32 GEMM.
* ``is_similar``         the reference's comparison predicate
                         (tfcc/core/utils/tfcc_debugutils.cpp:102-127).
* ``quantized_*``        scale / offset math (tfcc/core/utils/tfcc_quantizationutils.h),
                         quantize / dequantize
                         (tfcc/mkl/kernel/tfcc_mklquantizationkernel.hpp:21-46),
                         ``reduce_sum`` and the quantized ``matmul``
                         (tfcc/mkl/operations/tfcc_mklquantization.cpp), in numpy
                         (int64, wrapped to int32) and through the C port / the
                         reference's own compiled AVX2 kernel when built.

Parity pin: fp32 -- pinned to the reference's own tolerance only (its tests compare
with ``is_similar`` against numpy, tfcc/test/blas.cpp:34-61); int8 -- pinned exactly
by the reference's known-answer tests (tfcc/test/quantization.cpp:105-218) and by
the reference kernel compiled from its sources into ``oracle/_ref``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "liboracle_port.so"
REF_LIB = HERE / "_ref" / "libtfcc_ref_qmatmul.so"
_REF_COLMAJOR = "_ZN4tfcc28_MKLQuantizationMatmulAVX25623quantizedMatmulColMajorEjPKajPKhjjjjPij"
_REF_N1 = "_ZN4tfcc28_MKLQuantizationMatmulAVX25617quantizedMatmulN1EPKhPKiiPKaiijjPi"


class OracleError(ValueError):
    """Argument rejected by the restated reference checks (InvalidArgumentError)."""


# --------------------------------------------------------------------------- build / load
def build(ref_root: str | None = None) -> None:
    """Compile the C port, and the reference kernel when the reference tree is present."""
    subprocess.run(["make", "-s", "-C", str(HERE), "port"], check=True)
    ref_root = ref_root or os.environ.get("TFCC_REF_ROOT", "/root/reference")
    if Path(ref_root, "tfcc/mkl/kernel/tfcc_mklquantizationmatmul.avx256.cpp").exists():
        subprocess.run(["make", "-s", "-C", str(HERE), "ref", f"TFCC_REF_ROOT={ref_root}"],
                       check=True)


_port = None
_ref = None


def port_lib():
    global _port
    if _port is None:
        if not PORT_LIB.exists():
            build()
        _port = C.CDLL(str(PORT_LIB))
    return _port


def ref_lib():
    """The reference's compiled int8 kernel, or None when it was not built."""
    global _ref
    if _ref is None and REF_LIB.exists():
        _ref = C.CDLL(str(REF_LIB))
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------------------- fp32 matmul
def matmul_result_shape(sa, sb, sc=None):
    """Result shape, or OracleError, per tfcc_blas.cpp:27-45 (and :61-82 with a bias)."""
    sa, sb = tuple(sa), tuple(sb)
    if len(sa) < 2 or len(sb) < 2:
        raise OracleError("matmul require tensors with two or more dimensions")
    if len(sa) != len(sb) and len(sa) != 2 and len(sb) != 2:
        raise OracleError("shape invalid")
    if sa[-1] != sb[-2]:
        raise OracleError("shape invalid")
    if sc is not None and (len(sc) != 1 or sc[0] != sb[-1]):
        raise OracleError("shape invalid")
    if len(sa) == len(sb) and sa[:-2] != sb[:-2]:
        raise OracleError("shape invalid")
    lead = sa[:-2] if len(sa) >= len(sb) else sb[:-2]
    return tuple(lead) + (sa[-2], sb[-1])


def blas_matmul(a, b, c=None, dtype=np.float64):
    """``a . b (+ c)`` with the reference's batching.  ``dtype=float64`` gives the exact
    product of the float32 inputs rounded nowhere (ground truth); ``dtype=float32`` gives a
    float32 BLAS product, the stand-in for the reference's own fp32 output."""
    a = np.asarray(a)
    b = np.asarray(b)
    shape = matmul_result_shape(a.shape, b.shape, None if c is None else np.asarray(c).shape)
    if a.size == 0 or b.size == 0:
        return np.zeros(shape, dtype=dtype)
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    batch = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    a3 = a.reshape(-1, m, k).astype(dtype, copy=False)
    b3 = b.reshape(-1, k, n).astype(dtype, copy=False)
    out = np.empty((batch, m, n), dtype=dtype)
    for i in range(batch):  # stride 0 for a rank-2 operand next to a batched one
        ai = a3[i if a3.shape[0] > 1 else 0]
        bi = b3[i if b3.shape[0] > 1 else 0]
        np.matmul(ai, bi, out=out[i])
    if c is not None:
        out += np.asarray(c).astype(dtype, copy=False)
    return out.reshape(shape)


def host_cores() -> int:
    """Cores this process may run on."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def set_cpu_threads(n: int) -> int:
    """Make every CPU arm of the oracle use ``n`` threads, whatever the environment says
    (launchers such as torch.distributed.run export OMP_NUM_THREADS=1): torch's intra-op pool
    (MKL sgemm / oneDNN), numpy's BLAS, and the OpenMP runtime of the C port and of the
    reference kernel in oracle/_ref.  The reference states its thread count the same way
    (``omp_set_num_threads(4)``, tfcc/test/environment.cpp:40).  Returns ``n``."""
    n = max(1, int(n))
    try:
        import torch
        torch.set_num_threads(n)
    except Exception:
        pass
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    try:
        C.CDLL("libgomp.so.1").omp_set_num_threads(C.c_int(n))
    except Exception:
        pass
    return n


def blas_matmul_mkl(a, b, c=None):
    """``a . b (+ c)`` in float32 by torch's CPU matmul (MKL sgemm / oneDNN, the vendor
    libraries the reference's "MKL" backend wraps; its pinned oneDNN v1.8.1 is not buildable
    here).  Batching and the rank-2 broadcast are torch's, which agree with
    tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-186 for every shape the rules admit.
    Returns a numpy float32 array.  This is the timed stand-in for the reference's fp32 path."""
    import torch
    ta = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    tb = torch.from_numpy(np.ascontiguousarray(b, dtype=np.float32))
    matmul_result_shape(ta.shape, tb.shape, None if c is None else np.asarray(c).shape)
    out = torch.matmul(ta, tb)
    if c is not None:
        out += torch.from_numpy(np.ascontiguousarray(c, dtype=np.float32))
    return out.numpy()


def is_similar(a, b) -> bool:
    """tfcc::is_similar: integers exact; floats |a-b| < 1e-3*|a+b| or |a-b| < 1e-5."""
    a = np.asarray(a)
    b = np.asarray(b)
    if a.shape != b.shape:
        return False
    if np.issubdtype(a.dtype, np.integer) and np.issubdtype(b.dtype, np.integer):
        return bool(np.array_equal(a.astype(np.int64), b.astype(np.int64)))
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    d = np.abs(a - b)
    return bool(np.all((d < 1e-3 * np.abs(a + b)) | (d < 1e-5)))


def normwise_rel_error(x, truth) -> float:
    truth = np.asarray(truth, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    den = np.linalg.norm(truth.ravel())
    return float(np.linalg.norm((x - truth).ravel()) / den) if den > 0 else float(
        np.linalg.norm((x - truth).ravel()))


# --------------------------------------------------------------------------- quantization
_LIMITS = {np.uint8: (0, 255), np.int8: (-128, 127), np.uint16: (0, 65535),
           np.int16: (-32768, 32767), np.int32: (-2**31, 2**31 - 1), np.uint32: (0, 2**32 - 1)}


def _c_round(x: float) -> int:
    """C ``round``: half away from zero."""
    import math
    return int(math.floor(abs(x) + 0.5)) * (1 if x >= 0 else -1)


def quantized_scale_info(min_value, max_value, bits=8):
    """get_quantized_scale_info<T> (tfcc_quantizationutils.h:45-56)."""
    min_value = float(np.float32(min_value))
    max_value = float(np.float32(max_value))
    step_cnt = 1 << bits
    range_adjust = step_cnt / (step_cnt - 1.0)
    rng = float(np.float32(max_value) - np.float32(min_value)) * range_adjust
    range_scale = step_cnt / rng
    return range_scale, _c_round(min_value * range_scale)


def matmul_params(min_a, max_a, min_b, max_b):
    """(offA, offB, minC, maxC) as tfcc_mklquantization.cpp:181-193 computes them."""
    _, oa = quantized_scale_info(min_a, max_a)
    _, ob = quantized_scale_info(min_b, max_b)
    oa -= 0
    ob -= -128
    f = np.float32
    a_level = (f(max_a) - f(min_a)) / f(255)
    b_level = (f(max_b) - f(min_b)) / f(255)
    c_level = f(a_level * b_level)
    return int(oa), int(ob), float(f(c_level * f(-2**31))), float(f(c_level * f(2**31 - 1)))


def _quantize_values(real, scale, offset, dtype):
    """quantize_one over an array of doubles (tfcc_quantizationutils.h:72-79)."""
    lo, hi = _LIMITS[dtype]
    x = np.asarray(real, dtype=np.float64) * scale
    r = np.sign(x) * np.floor(np.abs(x) + 0.5)  # C round()
    q = r.astype(np.int64) - offset + lo
    return np.clip(q, lo, hi).astype(dtype)


def quantize(a, dtype, min_value=None, max_value=None):
    """MKLQuantizationInterface<T>::quantize: with no range, (q, min, max) with the range
    reduced from `a`; with a range, (q, min, max) for that range
    (tfcc/mkl/interfaces/tfcc_mklquantizationinterface.cpp:47-69,150-240,
     kernel/tfcc_mklquantizationkernel.hpp:23-33)."""
    a = np.asarray(a, dtype=np.float32)
    lo, hi = _LIMITS[dtype]
    if min_value is None:
        mn, mx = float(a.min()), float(a.max())
    else:
        mn, mx = float(np.float32(min_value)), float(np.float32(max_value))
    if mn >= mx:
        return np.full(a.shape, lo, dtype=dtype), mn, mx
    scale, offset = quantized_scale_info(mn, mx, bits=np.dtype(dtype).itemsize * 8)
    return _quantize_values(a.astype(np.float64), scale, offset, dtype), mn, mx


def requantize(a, min_in, max_in, min_out, max_out, dtype):
    """_requantize_helper<TO,TI> (tfcc_mklquantizationinterface.cpp:71-147) with
    _MKLRequantizationKernel (kernel/tfcc_mklquantizationkernel.hpp:48-64)."""
    a = np.asarray(a)
    lo_o, _ = _LIMITS[dtype]
    f = lambda v: float(np.float32(v))
    min_in, max_in, min_out, max_out = f(min_in), f(max_in), f(min_out), f(max_out)
    if min_out >= max_out:
        return np.full(a.shape, lo_o, dtype=dtype)
    bits_i = a.dtype.itemsize * 8
    step = float(2 ** bits_i)
    rng = float(np.float32(max_in) - np.float32(min_in)) * (step / (step - 1.0))
    in_scale = rng / step
    out_scale, out_offset = quantized_scale_info(min_out, max_out, bits=np.dtype(dtype).itemsize * 8)
    if min_in >= max_in:
        return np.full(a.shape, _quantize_values(np.array([min_in]), out_scale, out_offset, dtype)[0],
                       dtype=dtype)
    lo_i, _ = _LIMITS[a.dtype.type]
    real = min_in + (a.astype(np.float64) - lo_i) * in_scale
    return _quantize_values(real, out_scale, out_offset, dtype)


def dequantize(a, min_value, max_value):
    """kernel/tfcc_mklquantizationkernel.hpp:35-45 with get_dequantized_scale_info
    (tfcc_quantizationutils.h:58-70)."""
    a = np.asarray(a)
    if float(np.float32(min_value)) >= float(np.float32(max_value)):
        return np.full(a.shape, np.float32(min_value), dtype=np.float32)
    lo, _ = _LIMITS[a.dtype.type]
    bits = a.dtype.itemsize * 8
    step_cnt = float(2 ** bits)
    range_adjust = step_cnt / (step_cnt - 1.0)
    rng = float(np.float32(max_value) - np.float32(min_value)) * range_adjust
    scale = rng / step_cnt
    return (float(np.float32(min_value)) + (a.astype(np.float64) - lo) * scale).astype(np.float32)


def reduce_sum(a, row: bool):
    """tfcc::mkl::quantization::reduce_sum (tfcc_mklquantization.cpp:284-318)."""
    a = np.asarray(a)
    if a.size == 0 or a.ndim < 2:
        raise OracleError("invalid input tensor a")
    return a.astype(np.int64).sum(axis=-1 if row else -2).astype(np.int32)


def _check_qmatmul(a, rs_a, b, rs_b):
    if a.size == 0 or a.ndim < 2:
        raise OracleError("invalid input tensor a")
    if rs_a.size == 0:
        raise OracleError("invalid tensor reduceSumA")
    if b.size == 0 or b.ndim < 2:
        raise OracleError("invalid input tensor b")
    if rs_b.size == 0:
        raise OracleError("invalid tensor reduceSumB")
    if a.shape[-1] != b.shape[-2]:
        raise OracleError("tensor a and b don't match")
    if a.ndim != b.ndim and a.ndim != 2 and b.ndim != 2:
        raise OracleError("tensor a and b don't match")
    if a.shape[-2] != rs_a.shape[-1]:
        raise OracleError("tensor a and reduceSumA don't match")
    if b.shape[-1] != rs_b.shape[-1]:
        raise OracleError("tensor b and reduceSumB don't match")
    if a.ndim == b.ndim and a.shape[:-2] != b.shape[:-2]:
        raise OracleError("tensor a and b don't match")


def _fold(a, rs_a, b, rs_b):
    """Shapes, strides and the single-B batch fold of tfcc_mklquantization.cpp:120-145."""
    lead = a.shape[:-2] if a.ndim >= b.ndim else b.shape[:-2]
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    shape = tuple(lead) + (m, n)
    batch = int(np.prod(lead)) if lead else 1
    srs_a = 0 if rs_a.ndim == 1 else m
    srs_b = 0 if rs_b.ndim == 1 else n
    sa = 0 if a.ndim == 2 else m * k
    sb = 0 if b.ndim == 2 else k * n
    if b.size == k * n:
        m *= batch
        srs_a *= batch
        sa *= batch
        batch = 1
    return shape, batch, m, n, k, sa, sb, srs_a, srs_b


def quantized_matmul(a, rs_a, min_a, max_a, b, rs_b, min_b, max_b, impl="numpy"):
    """tfcc::mkl::quantization::matmul -> (C int32, minC, maxC).

    impl: "numpy" (int64 einsum wrapped to int32), "port" (the C restatement) or "ref"
    (offset matrix from the C port, accumulation by the reference's compiled kernel called
    with the reference's own argument order, tfcc_mklquantization.cpp:199-201).
    """
    a = np.ascontiguousarray(a, dtype=np.uint8)
    b = np.ascontiguousarray(b, dtype=np.int8)
    rs_a = np.ascontiguousarray(rs_a, dtype=np.int32)
    rs_b = np.ascontiguousarray(rs_b, dtype=np.int32)
    _check_qmatmul(a, rs_a, b, rs_b)
    off_a, off_b, min_c, max_c = matmul_params(min_a, max_a, min_b, max_b)
    shape, batch, m, n, k, sa, sb, srs_a, srs_b = _fold(a, rs_a, b, rs_b)
    if impl == "numpy":
        a3 = a.reshape(-1, a.shape[-2], k).astype(np.int64)
        b3 = b.reshape(-1, k, n).astype(np.int64)
        nb = max(a3.shape[0], b3.shape[0])
        ra = np.broadcast_to(rs_a.reshape(-1, a.shape[-2]).astype(np.int64), (a3.shape[0] if rs_a.ndim > 1 else 1, a.shape[-2]))
        rb = rs_b.reshape(-1, n).astype(np.int64)
        out = np.empty((nb, a.shape[-2], n), dtype=np.int64)
        for i in range(nb):
            ai = a3[i if a3.shape[0] > 1 else 0]
            bi = b3[i if b3.shape[0] > 1 else 0]
            rai = ra[i if ra.shape[0] > 1 else 0]
            rbi = rb[i if rb.shape[0] > 1 else 0]
            out[i] = ai @ bi + off_a * off_b * k + rai[:, None] * off_b + rbi[None, :] * off_a
        c = (out & 0xFFFFFFFF).astype(np.uint32).view(np.int32).reshape(shape)
        return c, min_c, max_c
    lib = port_lib()
    c = np.zeros(shape, dtype=np.int32)
    u, i32 = C.c_uint, C.c_int32
    if impl == "port":
        lib.oracle_qmatmul(u(batch), _p(a), u(sa), _p(rs_a), u(srs_a), i32(off_a), _p(b), u(sb),
                           _p(rs_b), u(srs_b), i32(off_b), u(m), u(n), u(k), _p(c))
        return c, min_c, max_c
    if impl == "ref":
        ref = ref_lib()
        if ref is None:
            raise RuntimeError("oracle/_ref is not built")
        if n == 1 and batch == 1:
            getattr(ref, _REF_N1)(_p(a), _p(rs_a), i32(off_a), _p(b), i32(int(rs_b.ravel()[0])),
                                  i32(off_b), u(m), u(k), _p(c))
            return c, min_c, max_c
        lib.oracle_create_offset_matrix(u(batch), _p(rs_a), u(m), u(srs_a), _p(rs_b), u(n),
                                        u(srs_b), i32(off_a), i32(off_b), i32(k), _p(c), u(m * n))
        getattr(ref, _REF_COLMAJOR)(u(batch), _p(b), u(sb), _p(a), u(sa), u(n), u(m), u(k), _p(c),
                                    u(m * n))
        return c, min_c, max_c
    raise ValueError(impl)


def quantized_dense(a, b, impl="numpy"):
    """quantize -> reduce_sum -> matmul -> dequantize on float inputs: the helper of the
    reference's known-answer tests (tfcc/test/quantization.cpp:105-121)."""
    qa, min_a, max_a = quantize(a, np.uint8)
    qb, min_b, max_b = quantize(b, np.int8)
    ra = reduce_sum(qa, True)
    rb = reduce_sum(qb, False)
    qc, min_c, max_c = quantized_matmul(qa, ra, min_a, max_a, qb, rb, min_b, max_b, impl=impl)
    return dequantize(qc, min_c, max_c)


# --------------------------------------------------------------------------- attention / FFN glue
def softmax_v2(a, scale=1.0):
    """_MKLActivationKernel::softmaxV2 on float32 rows
    (tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:138-155), after an optional pre-scale."""
    a = (np.asarray(a, dtype=np.float32) * np.float32(scale)).astype(np.float32)
    e = np.exp(a - a.max(axis=-1, keepdims=True)).astype(np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def attention(q, k, v, heads, scale=None):
    """The operator sequence of one attention block as the reference graph runs it, in
    float32: split heads (transpose to [batch, head, seq, dim],
    tfcc/cuda/interfaces/tfcc_cudabasicinterface.cu:83-100), ``q . k^T`` (blas matmul), scale
    and softmaxV2, ``. v``, merge heads.  Matmuls accumulate in float64 and round once, the
    exact-product oracle of ``blas_matmul``.  Inputs and output ``[batch, seq, heads*dim]``."""
    q, k, v = (np.asarray(t, dtype=np.float32) for t in (q, k, v))
    b, s, w = q.shape
    d = w // heads
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    sp = lambda t: t.reshape(b, s, heads, d).transpose(0, 2, 1, 3)
    scores = blas_matmul(sp(q), np.ascontiguousarray(sp(k).transpose(0, 1, 3, 2))).astype(np.float32)
    p = softmax_v2(scores, scale)
    o = blas_matmul(p, np.ascontiguousarray(sp(v))).astype(np.float32)
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(b, s, w)


def gelu_accurate(a):
    """_MKLActivationKernel::geluAccurate (:214-220): erf in float, outer products in double."""
    from scipy.special import erf
    a = np.asarray(a, dtype=np.float32)
    e = (np.float32(1.0) + erf(a / np.float32(1.4142135623730951)).astype(np.float32)).astype(np.float32)
    return (0.5 * a.astype(np.float64) * e.astype(np.float64)).astype(np.float32)


def layer_normalize(a, gamma, beta, eps=1e-5, residual=None):
    """_mkl_layer_normalize (tfcc/mkl/interfaces/tfcc_mklnormalizationinterface.cpp:29-62),
    float32 throughout, on x (+ residual)."""
    a = np.asarray(a, dtype=np.float32)
    if residual is not None:
        a = (a + np.asarray(residual, dtype=np.float32)).astype(np.float32)
    n = np.float32(a.shape[-1])
    mean = (a.sum(axis=-1, keepdims=True, dtype=np.float32) / n).astype(np.float32)
    d = (a - mean).astype(np.float32)
    var = ((d * d).sum(axis=-1, keepdims=True, dtype=np.float32) / n).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(var + np.float32(eps))).astype(np.float32)
    return (d * (inv * np.asarray(gamma, np.float32)) + np.asarray(beta, np.float32)).astype(np.float32)


def sgemm_f64acc_c(a, b, bias=None):
    """The C port's double-accumulating fp32 GEMM on rank-2 operands (float32 result)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), dtype=np.float32)
    bp = _p(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
    port_lib().oracle_sgemm_f64acc(C.c_uint(1), _p(a), C.c_uint(0), _p(b), C.c_uint(0), bp,
                                   C.c_uint(m), C.c_uint(n), C.c_uint(k), _p(c), None)
    return c
