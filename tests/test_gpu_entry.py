"""smoke() and the C-ABI argument checks on a GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_smoke_runs(pkg):
    from __graft_entry__ import smoke
    smoke()


def test_c_abi_rejects_bad_arguments(pkg):
    lib = pkg.lib
    d = torch.device("cuda:0")
    a = torch.zeros(16, 16, device=d)
    stream = torch.cuda.current_stream(d).cuda_stream
    p = a.data_ptr()
    assert lib.tfccb200_sgemm(stream, None, 0, p, 0, p, 256, None, 16, 16, 16, 1, 0, None, 0, None) == -1
    assert lib.tfccb200_sgemm(stream, p, 0, p, 0, p, 256, None, 0, 16, 16, 1, 0, None, 0, None) == -1
    assert lib.tfccb200_sgemm(stream, p, 0, p, 0, p, 256, None, 16, 16, 16, 1, 7, None, 0, None) == -1
    # the M <= 8 streaming kernel needs its scratch
    assert lib.tfccb200_sgemm_ex(stream, p, 0, p, 0, p, 64, None, 4, 16, 16, 1, 0, 2, None, 0, None) == -3
    # 2^16 x 2^16 results do not fit TFCC's 32-bit element count
    assert lib.tfccb200_sgemm(stream, p, 0, p, 0, p, 0, None, 65536, 65536, 16, 1, 0, None, 0, None) == -4
    assert lib.tfccb200_reduce_sum_u8(stream, None, 1, 4, 4, 1, p) == -1
    torch.cuda.synchronize()


def test_launch_counter_moves(pkg):
    d = torch.device("cuda:0")
    before = pkg.launch_count()
    pkg.blas.matmul(torch.ones(64, 64, device=d), torch.ones(64, 64, device=d))
    torch.cuda.synchronize()
    assert pkg.launch_count() > before
