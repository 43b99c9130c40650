"""The operators between the matmuls of an attention / feed-forward block, on the B200
backend: row softmax with a fused pre-scale, erf GELU, layer normalisation with a fused
residual add, and the two permutations attention needs.  Formulas are the reference's
(tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:138-155,214-220,
tfcc/mkl/interfaces/tfcc_mklnormalizationinterface.cpp:29-62)."""
from __future__ import annotations

import torch

from . import exceptions
from ._lib import check, lib
from .session import get_session


def _f32(t, name):
    if not isinstance(t, torch.Tensor) or t.numel() == 0:
        raise exceptions.InvalidArgumentError(f"invalid tensor {name}")
    if t.dtype != torch.float32:
        raise exceptions.NotImplementedError(f"{name}: implemented for float32, got {t.dtype}")
    if not t.is_cuda or not t.is_contiguous():
        raise exceptions.InvalidArgumentError(f"{name} must be a contiguous CUDA tensor")


def softmax(a: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """softmax(scale * a) over the last dimension."""
    _f32(a, "a")
    cols = a.shape[-1]
    out = torch.empty_like(a)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_softmax_f32(sess.stream_ptr, a.data_ptr(), a.numel() // cols, cols,
                                       float(scale), out.data_ptr()))
    return out


def gelu(a: torch.Tensor) -> torch.Tensor:
    """erf-form GELU (the reference's gelu_accurate)."""
    _f32(a, "a")
    out = torch.empty_like(a)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_gelu_f32(sess.stream_ptr, a.data_ptr(), a.numel(), out.data_ptr()))
    return out


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-5,
               residual: torch.Tensor | None = None) -> torch.Tensor:
    """Layer normalisation of ``x`` (+ ``residual``) over the last dimension."""
    _f32(x, "x")
    _f32(gamma, "gamma")
    _f32(beta, "beta")
    cols = x.shape[-1]
    if gamma.numel() != cols or beta.numel() != cols:
        raise exceptions.InvalidArgumentError("gamma / beta do not match the last dimension")
    if residual is not None:
        _f32(residual, "residual")
        if residual.shape != x.shape:
            raise exceptions.InvalidArgumentError("residual does not match x")
    out = torch.empty_like(x)
    sess = get_session(x.device)
    with torch.cuda.device(x.device):
        check(lib.tfccb200_layer_norm_f32(
            sess.stream_ptr, x.data_ptr(), residual.data_ptr() if residual is not None else None,
            gamma.data_ptr(), beta.data_ptr(), float(eps), x.numel() // cols, cols, out.data_ptr()))
    return out


def permute_0213(a: torch.Tensor) -> torch.Tensor:
    """[d0,d1,d2,d3] -> [d0,d2,d1,d3], materialised (splitting / merging attention heads)."""
    _f32(a, "a")
    if a.dim() != 4:
        raise exceptions.InvalidArgumentError("permute_0213 takes a rank-4 tensor")
    d0, d1, d2, d3 = a.shape
    out = torch.empty((d0, d2, d1, d3), dtype=torch.float32, device=a.device)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_permute_0213_f32(sess.stream_ptr, a.data_ptr(), d0, d1, d2, d3,
                                            out.data_ptr()))
    return out


def transpose_last2(a: torch.Tensor) -> torch.Tensor:
    """[..., r, c] -> [..., c, r], materialised (K transposed for Q.K^T)."""
    _f32(a, "a")
    if a.dim() < 2:
        raise exceptions.InvalidArgumentError("transpose_last2 needs rank >= 2")
    r, c = a.shape[-2], a.shape[-1]
    out = torch.empty(tuple(a.shape[:-2]) + (c, r), dtype=torch.float32, device=a.device)
    sess = get_session(a.device)
    with torch.cuda.device(a.device):
        check(lib.tfccb200_transpose_last2_f32(sess.stream_ptr, a.data_ptr(), a.numel() // (r * c),
                                               r, c, out.data_ptr()))
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int,
              scale: float | None = None) -> torch.Tensor:
    """``softmax(scale * Q K^T) V`` per head, in one kernel.

    ``q``, ``k``, ``v`` are ``[batch, seq, heads*dim]`` tensors as the projections produce
    them; they may be column slices of one packed ``[batch, seq, 3*heads*dim]`` tensor (their
    last dimension must be contiguous and all three must share the row pitch).  Returns
    ``[batch, seq, heads*dim]``.  ``scale`` defaults to ``1/sqrt(dim)``.  Shapes outside the
    fused kernel's range (seq > 128, dim not 32 or 64) raise InvalidArgumentError; compose
    ``permute_0213`` / ``transpose_last2`` / ``blas.matmul`` / ``softmax`` for those.
    """
    for t, nm in ((q, "q"), (k, "k"), (v, "v")):
        if not isinstance(t, torch.Tensor) or t.dim() != 3 or t.numel() == 0:
            raise exceptions.InvalidArgumentError(f"invalid tensor {nm}")
        if t.dtype != torch.float32:
            raise exceptions.NotImplementedError(f"{nm}: implemented for float32, got {t.dtype}")
        if not t.is_cuda or t.stride(2) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
            raise exceptions.InvalidArgumentError(f"{nm}: rows must be contiguous and batches dense")
    if q.shape != k.shape or q.shape != v.shape or q.shape[2] % heads != 0:
        raise exceptions.InvalidArgumentError("shape invalid")
    if not (q.stride(1) == k.stride(1) == v.stride(1)):
        raise exceptions.InvalidArgumentError("q, k and v must share one row pitch")
    batch, seq, width = q.shape
    dim = width // heads
    if scale is None:
        scale = 1.0 / float(dim) ** 0.5
    out = torch.empty((batch, seq, width), dtype=torch.float32, device=q.device)
    sess = get_session(q.device)
    with torch.cuda.device(q.device):
        check(lib.tfccb200_attention_f32(sess.stream_ptr, q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                         out.data_ptr(), batch, seq, heads, dim, q.stride(1), width,
                                         float(scale), sess.status_ptr))
    return out


def pack_qkv(wq, bq, wk, bk, wv, bv):
    """One ``[K, 3*N]`` weight and one ``[3*N]`` bias from the three projection weights of an
    attention block: a one-time preparation when the constants are loaded (the reference's
    Constant preprocess hook, tfcc/core/framework/tfcc_constant.cpp:70-106), after which
    ``x . Wqkv + bqkv`` is one launch and ``attention`` reads its three slices in place."""
    for t in (wq, bq, wk, bk, wv, bv):
        _f32(t, "weight")
    return torch.cat([wq, wk, wv], dim=1).contiguous(), torch.cat([bq, bk, bv]).contiguous()
