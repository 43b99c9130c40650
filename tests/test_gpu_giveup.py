"""The give-up path of a bounded device-side wait, exercised without hanging anything.

Every wait inside the tensor-core kernels has a time limit; when it runs out the kernel records
a status bit, stops waiting everywhere in that CTA and runs to its ordinary end, and the host
sees the failure at ``Session.sync()`` -- the asynchronous error model of the reference's CUDA
backend (tfcc/cuda/framework/tfcc_cudasession.cpp:45-63).  The test hook
``tfccb200_test_flag_wait`` shortens the limit of the waits on scratch counters to 1 ms and
makes them expect one arrival more than the launch delivers, so the wait is certain to run out
while every CTA still finishes its own work: nothing spins for long and nothing faults.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_abandoned_flag_wait_sets_status_and_context_survives(pkg, orc):
    d = torch.device("cuda:0")
    sess = pkg.session.get_session(d)
    sess.sync()
    g = torch.Generator(device=d)
    g.manual_seed(5)
    # few tiles, long K: with scratch the planner lets several CTAs share a tile's k-blocks,
    # and the CTA that gathers the partial tiles waits on the others' counters
    m, k, n = 1024, 3072, 768
    a = torch.empty((m, k), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    b = torch.empty((k, n), dtype=torch.float32, device=d).normal_(0, 0.02, generator=g)
    good = pkg.blas.matmul(a, b)
    sess.sync()

    pkg.lib.tfccb200_test_flag_wait(1_000_000, 1)
    try:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        pkg.blas.matmul(a, b)
        t1.record()
        with pytest.raises(pkg.exceptions.RuntimeError) as info:
            sess.sync()
        assert "0x8" in str(info.value)            # TFCCB200_DEV_TIMEOUT_EPILOGUE
        assert t0.elapsed_time(t1) < 500.0          # gave up after milliseconds, not seconds
    finally:
        pkg.lib.tfccb200_test_flag_wait(0, 0)

    # the status word was cleared by the raise, the context is intact, the next product is right
    again = pkg.blas.matmul(a, b)
    sess.sync()
    assert torch.equal(again, good)
    truth = a.cpu().numpy().astype(np.float64) @ b.cpu().numpy().astype(np.float64)
    assert orc.normwise_rel_error(again.cpu().numpy(), truth) < 1e-5
