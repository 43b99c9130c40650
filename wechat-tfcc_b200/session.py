"""Per-device launch context: stream, scratch and the device status word.

Plays the part of the reference's thread-default Session
(tfcc/core/framework/tfcc_session.h:28-66, tfcc/cuda/framework/tfcc_cudasession.cpp:36-63):
operators enqueue on its stream and never synchronise; ``sync()`` waits and
surfaces asynchronous device-side failures, as ``Session::sync`` does.
"""
from __future__ import annotations

import threading

import torch

from . import exceptions
from ._lib import lib

_local = threading.local()


class Session:
    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise exceptions.InvalidArgumentError("a B200 session needs a CUDA device")
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._workspaces = {}  # one scratch buffer per stream: calls on two streams may overlap

    @property
    def stream_ptr(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    @property
    def status_ptr(self) -> int:
        return self._status.data_ptr()

    def workspace(self, nbytes: int):
        """Scratch of at least ``nbytes`` for calls on the current stream (grown
        geometrically, reused by later calls on that stream).  A buffer that is outgrown is
        handed back to torch's allocator, which keeps it out of other streams' hands until
        the kernels queued on this stream have used it."""
        if nbytes == 0:
            return None, 0
        stream = torch.cuda.current_stream(self.device)
        key = stream.cuda_stream
        ws = self._workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            with torch.cuda.stream(stream):
                new = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
            if ws is not None:
                ws.record_stream(stream)
            ws = self._workspaces[key] = new
        return ws.data_ptr(), ws.numel()

    def sync(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()
        st = int(self._status.item())
        if st:
            self._status.zero_()
            raise exceptions.RuntimeError(-6, f"a kernel abandoned a bounded wait (bits 0x{st:x})")


def get_session(device) -> Session:
    """Thread-default session of ``device`` (created on first use)."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    table = getattr(_local, "sessions", None)
    if table is None:
        table = _local.sessions = {}
    s = table.get(device.index)
    if s is None:
        s = table[device.index] = Session(device)
    return s
