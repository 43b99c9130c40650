"""softmax / GELU / layer norm / permutations and the fused GEMM activation on the GPU against
the float32 restatements of the reference's CPU kernels in the oracle.  Tolerance: 2e-6
normwise (fp32 formulas whose sums run in a different order and whose exp / erf come from a
different math library); permutations are exact."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-6


def dev():
    return torch.device("cuda:0")


def t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev())


@pytest.mark.parametrize("shape", [(7, 5), (12, 128, 128), (3, 100), (9, 777), (4, 1024), (2, 3000)])
def test_softmax_rows(pkg, orc, shape):
    rng = np.random.default_rng(sum(shape))
    a = rng.normal(0, 3, shape).astype(np.float32)
    for scale in (1.0, 0.125):
        got = pkg.nn.softmax(t(a), scale).cpu().numpy()
        want = orc.softmax_v2(a, scale)
        assert orc.normwise_rel_error(got, want) < TOL
        assert np.allclose(got.sum(-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("shape", [(5, 64), (8, 128, 768), (3, 1000), (16, 1024)])
def test_layer_norm_with_and_without_residual(pkg, orc, shape):
    rng = np.random.default_rng(shape[-1])
    x = rng.normal(0.5, 2, shape).astype(np.float32)
    r = rng.normal(0, 1, shape).astype(np.float32)
    g = rng.uniform(0.5, 1.5, shape[-1]).astype(np.float32)
    b = rng.normal(0, 0.1, shape[-1]).astype(np.float32)
    got = pkg.nn.layer_norm(t(x), t(g), t(b), 1e-5).cpu().numpy()
    assert orc.normwise_rel_error(got, orc.layer_normalize(x, g, b, 1e-5)) < TOL
    got = pkg.nn.layer_norm(t(x), t(g), t(b), 1e-5, residual=t(r)).cpu().numpy()
    assert orc.normwise_rel_error(got, orc.layer_normalize(x, g, b, 1e-5, residual=r)) < TOL


def test_gelu_and_fused_gelu_epilogue(pkg, orc):
    rng = np.random.default_rng(4)
    a = rng.normal(0, 2, (33, 1001)).astype(np.float32)
    assert orc.normwise_rel_error(pkg.nn.gelu(t(a)).cpu().numpy(), orc.gelu_accurate(a)) < TOL
    # MatmulWithBias + Gelu in one pass, on every kernel path
    x = rng.normal(0, 1, (300, 260)).astype(np.float32)
    w = rng.normal(0, 0.1, (260, 516)).astype(np.float32)
    bias = rng.normal(0, 0.1, 516).astype(np.float32)
    want = orc.gelu_accurate(orc.blas_matmul(x, w, bias).astype(np.float32))
    for path in ("simt", "umma", "umma2", "auto"):
        got = pkg.blas.matmul(t(x), t(w), t(bias), path=path, activation="gelu").cpu().numpy()
        assert orc.normwise_rel_error(got, want) < 1e-5, path
    x8 = rng.normal(0, 1, (4, 1024)).astype(np.float32)
    w8 = rng.normal(0, 0.1, (1024, 2048)).astype(np.float32)
    got = pkg.blas.matmul(t(x8), t(w8), activation="gelu", path="skinny").cpu().numpy()
    assert orc.normwise_rel_error(got, orc.gelu_accurate(orc.blas_matmul(x8, w8).astype(np.float32))) < 1e-5


def test_permutations_are_exact(pkg):
    rng = np.random.default_rng(6)
    a = rng.normal(0, 1, (3, 17, 5, 64)).astype(np.float32)
    assert np.array_equal(pkg.nn.permute_0213(t(a)).cpu().numpy(), a.transpose(0, 2, 1, 3))
    b = rng.normal(0, 1, (2, 3, 70, 33)).astype(np.float32)
    assert np.array_equal(pkg.nn.transpose_last2(t(b)).cpu().numpy(), b.transpose(0, 1, 3, 2))
    c = rng.normal(0, 1, (128, 64)).astype(np.float32)
    assert np.array_equal(pkg.nn.transpose_last2(t(c)).cpu().numpy(), c.T)


def test_argument_errors(pkg):
    ex = pkg.exceptions
    with pytest.raises(ex.NotImplementedError):
        pkg.nn.softmax(torch.zeros(4, 4, dtype=torch.float64, device=dev()))
    with pytest.raises(ex.InvalidArgumentError):
        pkg.nn.layer_norm(torch.zeros(4, 8, device=dev()), torch.ones(7, device=dev()), torch.zeros(8, device=dev()))
    with pytest.raises(ex.InvalidArgumentError):
        pkg.nn.permute_0213(torch.zeros(4, 8, device=dev()))
