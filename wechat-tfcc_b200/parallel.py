"""Multi-GPU shim for one box: one process per GPU over ``torch.distributed``.

The reference has no multi-device operator; its only scheme is independent
replicas, one Device per GPU (tfcc/core/utils/tfcc_initializer.cpp:50-66).  Two
partitionings of the matmul path are added here:

* batch split -- a batched matmul is cut into contiguous batch ranges, one per
  rank, with no communication; results stay sharded.
* N split -- B (the weight) is column-sharded, A is replicated, every rank
  computes ``C[:, shard]`` and one all-gather leaves the full row-major C on
  every rank.

The local products run on this package's CUDA kernels.  ``matmul_fn`` and
``interleave_fn`` exist so that the host-side logic (ranges, gather order,
layout) can be exercised by CPU ranks in tests with a stand-in product.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import blas, exceptions
from ._lib import check, lib
from .session import get_session


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous range of ``total`` items owned by ``rank``: sizes differ by at most one,
    larger shards first."""
    if world <= 0 or not 0 <= rank < world:
        raise exceptions.InvalidArgumentError("invalid rank / world size")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def batch_split_matmul(a, b, c=None, *, rank=None, world=None, matmul_fn=None):
    """This rank's slice of a batched matmul: ``(result_slice, (start, stop))`` over the
    leading batch dimension.  A rank-2 operand is shared by all ranks.  No communication."""
    matmul_fn = matmul_fn or blas.matmul
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    batched = a if a.dim() > 2 else b
    if batched.dim() <= 2:
        raise exceptions.InvalidArgumentError("batch split needs a batched operand")
    start, stop = shard_range(batched.shape[0], world, rank)
    a_loc = a[start:stop] if a.dim() > 2 else a
    b_loc = b[start:stop] if b.dim() > 2 else b
    out = matmul_fn(a_loc, b_loc, c) if c is not None else matmul_fn(a_loc, b_loc)
    return out, (start, stop)


def interleave_panels(staging: torch.Tensor, out: torch.Tensor) -> None:
    """``out[m, g*ns + j] = staging[g, m, j]``: rank-major column panels into row-major C."""
    g, m, ns = staging.shape
    sess = get_session(staging.device)
    with torch.cuda.device(staging.device):
        st = lib.tfccb200_interleave_panels_f32(sess.stream_ptr, staging.data_ptr(),
                                                out.data_ptr(), m, ns, g)
    check(st)


def nsplit_matmul(a, b_shard, bias_shard=None, *, group=None, matmul_fn=None,
                  interleave_fn=None, staging=None, out=None):
    """Full ``C = A . B`` on every rank from column shards of B.

    ``b_shard`` is ``B[:, rank*N/G:(rank+1)*N/G]`` stored contiguously as ``[K, N/G]``; all
    shards have the same width.  Returns row-major ``[M, N]``.
    """
    matmul_fn = matmul_fn or blas.matmul
    interleave_fn = interleave_fn or interleave_panels
    world = dist.get_world_size(group)
    if a.dim() != 2 or b_shard.dim() != 2:
        raise exceptions.InvalidArgumentError("N split takes rank-2 operands")
    m, ns = a.shape[0], b_shard.shape[1]
    c_local = matmul_fn(a, b_shard, bias_shard) if bias_shard is not None else matmul_fn(a, b_shard)
    if world == 1:
        return c_local
    if staging is None:
        staging = torch.empty((world, m, ns), dtype=c_local.dtype, device=c_local.device)
    if out is None:
        out = torch.empty((m, world * ns), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(staging.view(-1), c_local.view(-1), group=group)
    interleave_fn(staging, out)
    return out
