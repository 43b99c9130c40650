"""The allocation-free M <= 8 entry point, ``tfccb200_sgemm_skinny_static``.

It serves embedders that cannot allocate device memory once they are running (all of HBM
belongs to their own arena, or cudaMalloc is banned on the serving thread) and so can neither
bring the workspace that ``tfccb200_sgemm`` wants for decode shapes nor let the library get it.
The partial sums go to a fixed array inside the library instead.  The checks: through the C
ABI, on two calls in a row with different problems (the array is reused and never cleared),
the output equals the workspace-based entry point's bit for bit (well inside the 1e-5 normwise
tolerance the other fp32 tests use), and a problem too large for the array is refused with
its own status code.  This file sorts last so that a run stopping at the first failure has
already run everything else.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(pkg, m, k, n, seed, with_bias):
    d = torch.device("cuda:0")
    g = torch.Generator(device=d)
    g.manual_seed(seed)
    x = torch.empty((m, k), dtype=torch.float32, device=d).normal_(0, 1, generator=g)
    w = torch.empty((k, n), dtype=torch.float32, device=d).normal_(0, 0.02, generator=g)
    bias = torch.empty(n, dtype=torch.float32, device=d).normal_(0, 1, generator=g) if with_bias else None
    lib = pkg.lib
    stream = torch.cuda.current_stream(d).cuda_stream
    bp = bias.data_ptr() if bias is not None else None

    ws_bytes = lib.tfccb200_sgemm_workspace(m, n, k, 1, 0)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=d)
    want = torch.full((m, n), float("nan"), dtype=torch.float32, device=d)
    st = lib.tfccb200_sgemm_ex(stream, x.data_ptr(), 0, w.data_ptr(), 0, want.data_ptr(), m * n, bp,
                               m, n, k, 1, 0, 2, ws.data_ptr(), ws.numel(), None)
    assert st == 0, lib.tfccb200_strerror(st)

    got = torch.full((m, n), float("nan"), dtype=torch.float32, device=d)
    st = lib.tfccb200_sgemm_skinny_static(stream, x.data_ptr(), w.data_ptr(), got.data_ptr(), bp,
                                          m, n, k)
    assert st == 0, lib.tfccb200_strerror(st)
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(pkg):
    assert pkg.lib.tfccb200_sgemm_skinny_static_capacity() == 20 << 20
    # first call: the benchmark's decode shape; second: a smaller, ragged one that reuses the
    # same array with stale partial sums still in it
    for (m, k, n, seed, with_bias) in ((8, 4096, 16384, 1, True), (3, 1000, 2052, 2, False)):
        got, want = _both(pkg, m, k, n, seed, with_bias)
        assert not torch.isnan(got).any()
        err = (got.double() - want.double()).norm() / want.double().norm()
        assert float(err) < 1e-5
        assert torch.equal(got, want)


def test_static_scratch_refuses_what_does_not_fit(pkg):
    lib = pkg.lib
    d = torch.device("cuda:0")
    m, k, n = 8, 16, 1 << 20
    assert lib.tfccb200_sgemm_skinny_static_need(m, n, k) > lib.tfccb200_sgemm_skinny_static_capacity()
    assert 0 < lib.tfccb200_sgemm_skinny_static_need(8, 16384, 4096) <= 20 << 20
    x = torch.zeros((m, k), dtype=torch.float32, device=d)
    w = torch.zeros((k, n), dtype=torch.float32, device=d)
    y = torch.zeros((m, n), dtype=torch.float32, device=d)
    stream = torch.cuda.current_stream(d).cuda_stream
    st = lib.tfccb200_sgemm_skinny_static(stream, x.data_ptr(), w.data_ptr(), y.data_ptr(), None, m, n, k)
    assert st == -7
    assert b"20 MiB" in lib.tfccb200_strerror(st)
    # more than 8 rows is not this kernel's shape
    assert lib.tfccb200_sgemm_skinny_static(stream, x.data_ptr(), w.data_ptr(), y.data_ptr(), None,
                                            9, 64, 64) == -5
    torch.cuda.synchronize()
