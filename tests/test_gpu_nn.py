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


@pytest.mark.parametrize("shape", [(5, 64), (8, 128, 768), (3, 1000), (16, 1024), (7, 1028), (3, 5000)])
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


@pytest.mark.parametrize("batch,seq,heads,dim", [(8, 128, 12, 64), (2, 128, 4, 32), (3, 77, 5, 64),
                                                  (1, 1, 1, 32), (2, 100, 3, 32)])
@pytest.mark.parametrize("packed", [True, False])
def test_fused_attention_matches_operator_sequence(pkg, orc, batch, seq, heads, dim, packed):
    """One kernel for transpose / Q.K^T / scale / softmax / .V / transpose back: normwise 1e-5
    against the float32 operator sequence with exact (float64-accumulated) products, also for
    ragged sequence lengths (masked keys) and with Q, K, V as slices of one packed buffer."""
    rng = np.random.default_rng(batch * 1000 + seq * 10 + heads)
    w = heads * dim
    qkv = rng.normal(0, 1, (batch, seq, 3 * w)).astype(np.float32)
    d = dev()
    if packed:
        tq = torch.from_numpy(qkv).to(d)
        q, k, v = tq[:, :, :w], tq[:, :, w:2 * w], tq[:, :, 2 * w:]
    else:
        q, k, v = (torch.from_numpy(np.ascontiguousarray(qkv[:, :, i * w:(i + 1) * w])).to(d)
                   for i in range(3))
    got = pkg.nn.attention(q, k, v, heads).cpu().numpy()
    pkg.session.get_session(d).sync()
    want = orc.attention(qkv[:, :, :w], qkv[:, :, w:2 * w], qkv[:, :, 2 * w:], heads)
    assert got.shape == want.shape
    assert orc.normwise_rel_error(got, want) < 1e-5
    assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max())


def test_fused_attention_refuses_what_it_cannot_take(pkg):
    d = dev()
    x = torch.zeros((2, 200, 128), dtype=torch.float32, device=d)
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        pkg.nn.attention(x, x, x, 2)          # seq > 128
    y = torch.zeros((2, 64, 96), dtype=torch.float32, device=d)
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        pkg.nn.attention(y, y, y, 2)          # dim 48


def test_glue_kernels_match_reference_generator_cases(pkg, orc, golden):
    """The device softmax, erf GELU and layer normalisation on the cases of the reference's own
    generators (tests/golden/make_golden.py), compared with the reference's predicate."""
    from test_oracle_golden import _glue_cases
    d = dev()
    for kind, a, extra, expect in _glue_cases(golden):
        ta = torch.from_numpy(np.ascontiguousarray(a)).to(d)
        if kind == "softmax":
            moved = ta.movedim(extra, -1).contiguous()
            got = pkg.nn.softmax(moved).movedim(-1, extra)
        elif kind == "gelu":
            got = pkg.nn.gelu(ta)
        else:
            axis, gamma, beta = extra
            cols = int(np.prod(a.shape[axis:]))
            got = pkg.nn.layer_norm(ta.reshape(-1, cols).contiguous(),
                                    torch.from_numpy(gamma.reshape(cols).astype(np.float32)).to(d),
                                    torch.from_numpy(beta.reshape(cols).astype(np.float32)).to(d),
                                    eps=1e-12).reshape(a.shape)
        got = got.cpu().numpy()
        assert orc.is_similar(got, expect), (kind, a.shape)
        assert np.abs(got.astype(np.float64) - expect).max() < 5e-6, (kind, a.shape)
