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

import ctypes as C
import os

from . import blas, exceptions
from ._lib import BARRIER_FN, PRECISIONS, check, lib
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


class FusedNSplit:
    """N-split matmul whose all-gather happens inside the GEMM epilogue.

    Every rank owns full row-major ``C [M, N]`` buffers that its peers can address (symmetric
    memory, or CUDA IPC handles when that is unavailable).  ``matmul`` runs the tensor-core
    GEMM on this rank's column shard of B and stores each finished tile into the matching
    columns of every rank's C with ordinary 128-byte-line stores over NVLink (or one multimem
    store through the switch), overlapping the transfer with the remaining tiles; a cross-rank
    barrier then closes the step.  ``dtype=torch.int32`` plans the same for the quantized
    matmul (``qmatmul``).

    Result buffers.  Every lane alternates between two C buffers, so a call never writes the
    buffer its predecessor returned: the result of a call may be read by work enqueued before
    the next call of this object on the same rank, with no extra barrier.

    ``in_flight=2`` keeps two products in flight: calls alternate between two lanes, each with
    its own stream, C buffers, scratch and barrier channel, and each limited to half of the
    SMs.  The last tiles of one product are then pushed while the other product is still
    multiplying, which hides the burst of NVLink traffic at the end of a product (every GPU
    finishes its last tiles at the same moment and every GPU receives from all the others).
    ``in_flight=3`` and more add lanes without making the products narrower: two products
    multiply side by side and the CTAs of a third take over the SMs of whichever finishes,
    while that one's last tiles cross NVLink and its barrier runs -- no half of the chip waits
    for a barrier.  Measured on eight GPUs (8192^3): 1358 / 1533 / 1674 / 1757 TFLOP/s with one
    to four lanes, 1440 with six.
    Use ``matmul(..., wait=False)`` and ``join()`` to get the overlap.
    """

    def __init__(self, m: int, n_total: int, device, group=None, *, in_flight: int = 1,
                 dtype=torch.float32, multicast=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        if n_total % self.world != 0:
            raise exceptions.InvalidArgumentError("N must divide evenly over the ranks")
        if in_flight not in range(1, 9):
            raise exceptions.InvalidArgumentError("in_flight is 1 to 8")
        if dtype not in (torch.float32, torch.int32):
            raise exceptions.InvalidArgumentError("C is float32 (matmul) or int32 (qmatmul)")
        self.m, self.n_total, self.ns = m, n_total, n_total // self.world
        self.dtype = dtype
        self.in_flight = in_flight
        self.how = None
        self._keep = []
        self._calls = 0
        # NVLink multicast stores: by default for float32 results from four ranks on.  The int32
        # result of the quantized product is small and bound by what a rank RECEIVES, and a
        # multicast store also sends the rank its own tiles back through the switch (measured
        # on four GPUs, 4096^3: 102 us with peer stores against 118 us with multicast; the
        # 8192^3 fp32 product: 888 against 926 TFLOP/s), so it keeps plain peer stores.
        if multicast is None:
            default = "1" if (self.world >= 4 and dtype == torch.float32) else "0"
            want_mc = os.environ.get("TFCCB200_MULTICAST", default) != "0"
        else:
            want_mc = bool(multicast)
        # buffers[lane][slot] -> (tensor, ctypes array of every rank's pointer, multicast ptr, handle)
        self.buffers = [[self._shared((m, n_total), dtype, want_mc) for _slot in range(2)]
                        for _lane in range(in_flight)]
        self.handle = self.buffers[0][0][3]
        self.c = self.buffers[0][0][0]
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._streams = ([torch.cuda.Stream(self.device) for _ in range(in_flight)]
                         if in_flight >= 2 else [None])
        self._done = [None] * in_flight
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._max_ctas = (sms // 2) & ~1 if in_flight >= 2 else 0
        self._host = None

    # ---- peer-addressable buffers ------------------------------------------------------------
    def _shared(self, shape, dtype, want_mc):
        """A tensor every rank can address: (tensor, pointers by rank, multicast ptr or None,
        symmetric-memory handle or None)."""
        try:
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty(shape, dtype=dtype, device=self.device)
            handle = symm_mem.rendezvous(t, group=self.group)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            how = "symmetric memory"
            # NVLink multicast alias (0 when the fabric has no NVLS): one store reaches every
            # rank, so a GPU sends its shard once instead of world - 1 times.  With two ranks the
            # plain peer store is as cheap, so multicast is the default from four ranks on;
            # TFCCB200_MULTICAST=0/1 overrides.
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
            mc_ptr = None
            if mc and want_mc:
                mc_ptr = mc + (t.data_ptr() - ptrs[self.rank])
                how = "symmetric memory, NVLink multicast stores"
        except Exception as exc:  # fall back to classic CUDA IPC handles
            self._symm_error = repr(exc)
            handle, mc_ptr = None, None
            t = torch.empty(shape, dtype=dtype, device=self.device)
            ptrs = self._exchange_ipc(t)
            how = "CUDA IPC handles"
        self.how = how
        return t, (C.c_void_p * self.world)(*ptrs), mc_ptr, handle

    def _exchange_ipc(self, t):
        storage = t.untyped_storage()
        handle = storage._share_cuda_()
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (handle, t.storage_offset()), group=self.group)
        ptrs = []
        for r, (h, off) in enumerate(gathered):
            if r == self.rank:
                ptrs.append(t.data_ptr())
                continue
            st = torch.UntypedStorage._new_shared_cuda(*h)
            peer = torch.empty(0, dtype=t.dtype, device=st.device).set_(st, off, t.shape, t.stride())
            self._keep.append(peer)  # keeps the mapping alive
            ptrs.append(peer.data_ptr())
        return ptrs

    def barrier(self, channel: int = 0):
        """All ranks' kernels issued so far on the current streams have completed."""
        if self.handle is not None and hasattr(self.handle, "barrier"):
            self.handle.barrier(channel=channel)
        else:
            dist.all_reduce(self._flag, group=self.group)

    # ---- the product -------------------------------------------------------------------------
    def _next(self):
        lane = self._calls % self.in_flight
        slot = (self._calls // self.in_flight) % 2
        self._calls += 1
        return lane, self.buffers[lane][slot]

    def _run(self, launch, wait):
        """Run ``launch(buffer)`` plus the closing barrier on the next lane."""
        lane, buf = self._next()
        stream = self._streams[lane]
        if stream is None:
            with torch.cuda.device(self.device):
                launch(buf)
                self.barrier(0)
            return buf[0]
        cur = torch.cuda.current_stream(self.device)
        stream.wait_event(cur.record_event())   # operands, and readers of older results
        with torch.cuda.device(self.device), torch.cuda.stream(stream):
            launch(buf)
            self.barrier(lane)
            self._done[lane] = stream.record_event()
        if wait:
            cur.wait_event(self._done[lane])
        return buf[0]

    def join(self):
        """The current stream waits for every product issued so far."""
        cur = torch.cuda.current_stream(self.device)
        for ev in self._done:
            if ev is not None:
                cur.wait_event(ev)

    def matmul(self, a, b_shard, bias_shard=None, *, precision: str = "fp32", wait: bool = True,
               destinations=None):
        """``destinations``: ranks whose C is written (default all); for measurements."""
        if self.dtype != torch.float32:
            raise exceptions.InvalidArgumentError("this plan holds an int32 C: use qmatmul")
        if a.dim() != 2 or b_shard.dim() != 2 or a.shape[1] != b_shard.shape[0]:
            raise exceptions.InvalidArgumentError("shape invalid")
        if a.shape[0] != self.m or b_shard.shape[1] != self.ns:
            raise exceptions.InvalidArgumentError("operands do not match the planned C")
        for t in (a, b_shard) + ((bias_shard,) if bias_shard is not None else ()):
            if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
                raise exceptions.InvalidArgumentError("operands must be contiguous float32 CUDA tensors")
        k = a.shape[1]

        def launch(buf):
            _t, ptrs, mc_ptr, _h = buf
            if destinations is not None:
                ptrs = (C.c_void_p * self.world)(*[ptrs[r] if (r in destinations or r == self.rank)
                                                   else None for r in range(self.world)])
                mc_ptr = None
            sess = get_session(self.device)
            ws_bytes = lib.tfccb200_sgemm_workspace(self.m, self.ns, k, 1, PRECISIONS[precision])
            ws_ptr, ws_len = sess.workspace(ws_bytes) if ws_bytes else (None, 0)
            check(lib.tfccb200_sgemm_nsplit_push_ex(
                sess.stream_ptr, a.data_ptr(), b_shard.data_ptr(), ptrs, self.world, self.rank,
                bias_shard.data_ptr() if bias_shard is not None else None, self.m, self.ns, k,
                PRECISIONS[precision], mc_ptr, ws_ptr, ws_len, self._max_ctas, sess.status_ptr))

        return self._run(launch, wait)

    def qmatmul(self, a, rs_a, off_a: int, b_shard, rs_b_shard, off_b: int, *, wait: bool = True):
        """Quantized u8 x s8 -> s32 product with the zero-point correction, column shards of B
        (and of its column sums) per rank, tiles stored into every rank's int32 C."""
        if self.dtype != torch.int32:
            raise exceptions.InvalidArgumentError("this plan holds a float32 C: use matmul")
        if a.dim() != 2 or b_shard.dim() != 2 or a.shape[1] != b_shard.shape[0]:
            raise exceptions.InvalidArgumentError("tensor a and b don't match")
        if a.shape[0] != self.m or b_shard.shape[1] != self.ns:
            raise exceptions.InvalidArgumentError("operands do not match the planned C")
        if rs_a.numel() != self.m or rs_b_shard.numel() != self.ns:
            raise exceptions.InvalidArgumentError("tensor a and reduceSumA don't match")
        for t, dt in ((a, torch.uint8), (b_shard, torch.int8), (rs_a, torch.int32),
                      (rs_b_shard, torch.int32)):
            if t.dtype != dt or not t.is_cuda or not t.is_contiguous():
                raise exceptions.InvalidArgumentError("operands must be contiguous CUDA tensors of "
                                                      "uint8 / int8 / int32")
        k = a.shape[1]

        def launch(buf):
            _t, ptrs, mc_ptr, _h = buf
            sess = get_session(self.device)
            check(lib.tfccb200_qgemm_nsplit_push(
                sess.stream_ptr, a.data_ptr(), rs_a.data_ptr(), int(off_a), b_shard.data_ptr(),
                rs_b_shard.data_ptr(), int(off_b), ptrs, self.world, self.rank, self.m, self.ns, k,
                mc_ptr, sess.status_ptr))

        return self._run(launch, wait)

    # ---- host buffers in, host buffer out ------------------------------------------------------
    def prepare_host(self, k: int):
        """Collective: peer-addressable staging for ``matmul_host`` (every rank's A [M,K], this
        rank's B shard)."""
        want_mc = os.environ.get("TFCCB200_MULTICAST", "1" if self.world >= 4 else "0") != "0"
        a_buf = self._shared((self.m, k), torch.float32, want_mc)
        b_buf = torch.empty((k, self.ns), dtype=torch.float32, device=self.device)
        self._host = (k, a_buf, b_buf)

    def matmul_host(self, ha_rows, hb_shard, hc_rows, *, precision: str = "fp32"):
        """This rank's share of ``C = A . B`` with all operands in (pinned) host memory:
        ``ha_rows`` = rows ``[rank*M/G, (rank+1)*M/G)`` of A, ``hb_shard`` = this rank's
        ``[K, N/G]`` shard of B, ``hc_rows`` receives the same rows of the full-width C.
        Synchronous.  Through ``tfccb200_sgemm_nsplit_host``."""
        if self._host is None:
            raise exceptions.InvalidArgumentError("call prepare_host(k) on every rank first")
        k, (a_t, a_ptrs, a_mc, _h), b_buf = self._host
        rows = self.m // self.world
        for t, shape in ((ha_rows, (rows, k)), (hb_shard, (k, self.ns)), (hc_rows, (rows, self.n_total))):
            if t.dtype != torch.float32 or t.is_cuda or not t.is_contiguous() or tuple(t.shape) != shape:
                raise exceptions.InvalidArgumentError(f"host operand must be contiguous float32 {shape}")
        _lane, (c_t, c_ptrs, c_mc, _h2) = 0, self.buffers[0][0]
        sess = get_session(self.device)
        errors = []

        def _barrier(_ctx, _stream):
            try:
                self.barrier(0)
                return 0
            except Exception as exc:  # an exception must not cross the C frame
                errors.append(exc)
                return -6

        cb = BARRIER_FN(_barrier)
        with torch.cuda.device(self.device):
            ws_bytes = lib.tfccb200_sgemm_workspace(self.m, self.ns, k, 1, PRECISIONS[precision])
            ws_ptr, ws_len = sess.workspace(ws_bytes) if ws_bytes else (None, 0)
            st = lib.tfccb200_sgemm_nsplit_host(
                sess.stream_ptr, ha_rows.data_ptr(), hb_shard.data_ptr(), self.ns, hc_rows.data_ptr(),
                a_ptrs, a_mc, b_buf.data_ptr(), c_ptrs, c_mc, self.world, self.rank, self.m, self.ns,
                k, PRECISIONS[precision], ws_ptr, ws_len, cb, None, sess.status_ptr)
        if errors:
            raise errors[0]
        check(st)
        return hc_rows


class DeviceGroup:
    """One process driving several GPUs: thin wrapper of ``tfccb200_group_*`` (how a TFCC
    program with one Device per GPU would use the N split; the reference's own multi-GPU model
    is independent Devices, tfcc/core/utils/tfcc_initializer.cpp:50-66)."""

    def __init__(self, devices):
        devs = (C.c_int * len(devices))(*[int(d) for d in devices])
        h = C.c_void_p()
        check(lib.tfccb200_group_create(len(devices), devs, C.byref(h)))
        self._h = h
        self.devices = [int(d) for d in devices]

    def close(self):
        if self._h is not None:
            check(lib.tfccb200_group_destroy(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self):
        return len(self.devices)

    def stream(self, member: int) -> int:
        return int(lib.tfccb200_group_stream(self._h, member) or 0)

    def sync(self):
        check(lib.tfccb200_group_sync(self._h))

    def _ptrs(self, tensors):
        return (C.c_void_p * len(tensors))(*[t.data_ptr() if t is not None else None
                                             for t in tensors])

    def sgemm_nsplit(self, a, b_shards, c, bias_shards=None, *, precision: str = "fp32"):
        """``a[i]``, ``b_shards[i]`` on member i's device; ``c[i]`` that member's full C."""
        m, k = a[0].shape
        ns = b_shards[0].shape[1]
        check(lib.tfccb200_group_sgemm_nsplit(
            self._h, self._ptrs(a), self._ptrs(b_shards), self._ptrs(c),
            self._ptrs(bias_shards) if bias_shards is not None else None, m, ns, k,
            PRECISIONS[precision]))

    def qgemm_nsplit(self, a, rs_a, off_a, b_shards, rs_b_shards, off_b, c):
        m, k = a[0].shape
        ns = b_shards[0].shape[1]
        check(lib.tfccb200_group_qgemm_nsplit(
            self._h, self._ptrs(a), self._ptrs(rs_a), int(off_a), self._ptrs(b_shards),
            self._ptrs(rs_b_shards), int(off_b), self._ptrs(c), m, ns, k))

    def sgemm_nsplit_host(self, ha, hb, hc, *, precision: str = "fp32"):
        """Host tensors (pinned for overlap) ``[M,K] . [K,N] -> [M,N]``; synchronous."""
        m, k = ha.shape
        n = hb.shape[1]
        check(lib.tfccb200_group_sgemm_nsplit_host(self._h, ha.data_ptr(), hb.data_ptr(),
                                                   hc.data_ptr(), m, n, k, PRECISIONS[precision]))
        return hc
