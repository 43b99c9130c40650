"""quantize / dequantize / requantize on the device against the oracle and the reference's
vectors (QuantizationTest.quantize / dequantize / requantize, tfcc/test/quantization.cpp:40-102),
and the whole quantized dense layer (quantize -> reduce_sum -> matmul -> dequantize) without
leaving the GPU.  Integer outputs must match exactly; dequantized floats bit for bit too,
since both sides evaluate the same double-precision expression."""
import numpy as np
import pytest
import torch

from conftest import golden_cases
from test_oracle_golden import DEQUANT_EXPECT, DEQUANT_IN, REQUANT_EXPECT

pytestmark = pytest.mark.gpu
NP2T = {np.int8: torch.int8, np.uint8: torch.uint8, np.int16: torch.int16, np.uint16: torch.uint16,
        np.int32: torch.int32, np.uint32: torch.uint32}


def dev():
    return torch.device("cuda:0")


def s1(v):
    return torch.tensor([v], dtype=torch.float32, device=dev())


def test_quantize_reference_generator_cases(pkg, orc, golden):
    q = pkg.quantization
    for i, case in golden_cases(golden["quantization_quantize"], "quantization/quantize"):
        a = torch.from_numpy(case["a"]).to(dev())
        q8, mn, mx = q.quantize(a, torch.int8)
        u8, _, _ = q.quantize(a, torch.uint8)
        assert np.array_equal(q8.cpu().numpy(), case["int8_a"]), i
        assert np.array_equal(u8.cpu().numpy(), case["uint8_a"]), i
        assert float(mn.item()) == float(case["a"].min()) and float(mx.item()) == float(case["a"].max())


@pytest.mark.parametrize("np_t", [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32])
def test_quantize_dequantize_all_types_match_oracle(pkg, orc, np_t):
    rng = np.random.default_rng(int(np.dtype(np_t).itemsize) * 7 + 1)
    a = rng.normal(0, 3, (37, 1021)).astype(np.float32)
    ta = torch.from_numpy(a).to(dev())
    got, mn, mx = pkg.quantization.quantize(ta, NP2T[np_t])
    want, wmn, wmx = orc.quantize(a, np_t)
    assert np.array_equal(got.cpu().numpy().view(np_t), want)
    assert (float(mn.item()), float(mx.item())) == (wmn, wmx)
    # explicit range narrower than the data: values clamp
    got2 = pkg.quantization.quantize(ta, NP2T[np_t], s1(-1.25), s1(2.5))
    assert np.array_equal(got2.cpu().numpy().view(np_t), orc.quantize(a, np_t, -1.25, 2.5)[0])
    back = pkg.quantization.dequantize(got, mn, mx).cpu().numpy()
    assert np.array_equal(back, orc.dequantize(want, wmn, wmx))


@pytest.mark.parametrize("np_t", [np.int8, np.uint8, np.int16, np.uint16])
@pytest.mark.parametrize("mn,mx", [(-1.0, 1.0), (-128.0, 127.0), (0.0, 255.0), (-3.7, 9.25), (0.001, 0.0625),
                                   (-32768.0, 32767.0), (-1e-3, 1e6)])
def test_quantize_at_and_around_rounding_ties(pkg, orc, np_t, mn, mx):
    """round(real * scale) is half away from zero on the double-precision product.  Inputs placed
    on the half-integers of the scaled axis and one to three float steps either side of them, the
    integers themselves, zeros, denormals and values far outside the range (clamped): every
    result must be the oracle's."""
    bits = np.dtype(np_t).itemsize * 8
    scale, _ = orc.quantized_scale_info(mn, mx, bits=bits)
    lo_k, hi_k = int(np.floor(mn * scale)) - 3, int(np.ceil(mx * scale)) + 3
    rng = np.random.default_rng(bits + int(abs(mn) * 10))
    ks = np.unique(np.concatenate([np.arange(lo_k, min(hi_k, lo_k + 600)),
                                   rng.integers(lo_k, hi_k + 1, 3000),
                                   np.arange(max(lo_k, hi_k - 600), hi_k + 1)])).astype(np.float64)
    base = ((ks + 0.5) / scale).astype(np.float32)
    vals = [base]
    up, down = base.copy(), base.copy()
    for _ in range(3):
        up = np.nextafter(up, np.float32(np.inf)).astype(np.float32)
        down = np.nextafter(down, np.float32(-np.inf)).astype(np.float32)
        vals += [up.copy(), down.copy()]
    vals.append((ks / scale).astype(np.float32))  # the integers themselves
    # (products beyond the 64-bit integers are left out: the reference's conversion of those is
    # undefined behaviour)
    far = np.array([0.0, -0.0, 1e-45, -1e-45, 1e-30, 1e9, -1e9, 12345.678, 4194303.9, -4194304.5,
                    8388607.5], dtype=np.float32)
    vals.append(far[np.abs(far.astype(np.float64) * scale) < 2.0 ** 60])
    a = np.concatenate(vals).astype(np.float32)
    a = np.concatenate([a, rng.uniform(mn - 1, mx + 1, (-a.size) % 64 + 640).astype(np.float32)])
    a = a.reshape(-1, 64)
    ta = torch.from_numpy(a).to(dev())
    want = orc.quantize(a, np_t, mn, mx)[0]
    got = pkg.quantization.quantize(ta, NP2T[np_t], s1(mn), s1(mx))
    assert np.array_equal(got.cpu().numpy().view(np_t), want)
    if np_t in (np.int8, np.uint8, np.int16):
        q, sums = pkg.quantization.quantize_with_row_sums(ta, NP2T[np_t], s1(mn), s1(mx))
        assert np.array_equal(q.cpu().numpy().view(np_t), want)
        assert np.array_equal(sums.cpu().numpy(), want.astype(np.int64).sum(-1).astype(np.int32))


def test_dequantize_requantize_known_answers(pkg, orc):
    a = torch.from_numpy(DEQUANT_IN).to(dev())
    got = pkg.quantization.dequantize(a, s1(-2.5), s1(3.4)).cpu().numpy()
    assert orc.is_similar(got + np.float32(5.9), DEQUANT_EXPECT + np.float32(5.9))
    assert np.array_equal(got, orc.dequantize(DEQUANT_IN, -2.5, 3.4))
    r = pkg.quantization.requantize(a, s1(-2.5), s1(3.4), s1(-12.7), s1(24.5), torch.uint16)
    assert np.array_equal(r.cpu().numpy().view(np.uint16), REQUANT_EXPECT)


def test_requantize_type_pairs_and_degenerate_ranges(pkg, orc):
    rng = np.random.default_rng(5)
    q = pkg.quantization
    for ti, to in ((np.int32, np.int8), (np.int32, np.uint8), (np.uint8, np.int16), (np.int16, np.uint32)):
        info = np.iinfo(ti)
        a = rng.integers(max(info.min, -2**31), min(info.max, 2**31 - 1), (64, 257)).astype(ti)
        ta = torch.from_numpy(a).to(dev())
        got = q.requantize(ta, s1(-7.5), s1(11.0), s1(-3.0), s1(4.5), NP2T[to]).cpu().numpy().view(to)
        assert np.array_equal(got, orc.requantize(a, -7.5, 11.0, -3.0, 4.5, to)), (ti, to)
    a8 = torch.from_numpy(DEQUANT_IN).to(dev())
    assert np.all(q.quantize(torch.full((5, 5), 1.5, device=dev()), torch.int8)[0].cpu().numpy() == -128)
    assert np.all(q.dequantize(a8, s1(2.0), s1(2.0)).cpu().numpy() == np.float32(2.0))
    assert np.all(q.requantize(a8, s1(-1.0), s1(1.0), s1(3.0), s1(3.0), torch.int16).cpu().numpy() == -32768)
    got = q.requantize(a8, s1(1.0), s1(1.0), s1(-3.0), s1(3.0), torch.int8).cpu().numpy()
    assert np.array_equal(got, orc.requantize(DEQUANT_IN, 1.0, 1.0, -3.0, 3.0, np.int8))


def test_quantized_dense_layer_on_device_known_answers(pkg, orc):
    """mkl_quantized_matmul of the reference's tests, every step on the GPU: 5 / 11 / 17."""
    q = pkg.quantization
    v1 = np.array([1, 2, 3, 4, 5, 6, 1, 2, 3, 4, 5, 6], np.float32)
    v2 = np.array([1, 2, 1, 2], np.float32)
    for a, b in ((v1.reshape(2, 3, 2), v2.reshape(2, 2, 1)), (v1[:6].reshape(3, 2), v2.reshape(2, 2, 1)),
                 (v1.reshape(2, 3, 2), v2[:2].reshape(2, 1))):
        ta, tb = torch.from_numpy(a).to(dev()), torch.from_numpy(b).to(dev())
        qa, amin, amax = q.quantize(ta, torch.uint8)
        qb, bmin, bmax = q.quantize(tb, torch.int8)
        ra, rb = q.reduce_sum(qa, True), q.reduce_sum(qb, False)
        qc, cmin, cmax = q.matmul(qa, ra, amin, amax, qb, rb, bmin, bmax)
        r = q.dequantize(qc, cmin, cmax).cpu().numpy()
        assert [int(x) for x in r.ravel()] == [5, 11, 17, 5, 11, 17]
        assert np.array_equal(r, orc.quantized_dense(a, b))


def test_quantized_dense_layer_larger(pkg, orc):
    rng = np.random.default_rng(8)
    a = rng.normal(0, 1, (96, 768)).astype(np.float32)
    w = rng.normal(0, 0.05, (768, 512)).astype(np.float32)
    q = pkg.quantization
    ta, tw = torch.from_numpy(a).to(dev()), torch.from_numpy(w).to(dev())
    qa, amin, amax = q.quantize(ta, torch.uint8)
    qw, wmin, wmax = q.quantize(tw, torch.int8)
    qc, cmin, cmax = q.matmul(qa, q.reduce_sum(qa, True), amin, amax, qw, q.reduce_sum(qw, False), wmin, wmax)
    got = q.dequantize(qc, cmin, cmax).cpu().numpy()
    assert np.array_equal(got, orc.quantized_dense(a, w))
    # and the quantized product tracks the float product to quantization accuracy
    assert orc.normwise_rel_error(got, a.astype(np.float64) @ w.astype(np.float64)) < 2e-2


@pytest.mark.parametrize("shape", [(256, 4096), (96, 768), (3, 7, 130), (5, 33), (2, 2051)])
@pytest.mark.parametrize("dtype", [torch.uint8, torch.int8, torch.int16])
def test_quantize_with_row_sums_equals_the_two_separate_calls(pkg, orc, shape, dtype):
    """quantize + reduce_sum(row) fused into one pass over the activations
    (tfcc/test/quantization.cpp:105-121 runs them as two operators): same bits."""
    rng = np.random.default_rng(sum(shape))
    a = rng.normal(0, 1, shape).astype(np.float32)
    q = pkg.quantization
    ta = torch.from_numpy(a).to(dev())
    want_q, mn, mx = q.quantize(ta, dtype)
    want_s = q.reduce_sum(want_q, True)
    got_q, gmn, gmx, got_s = q.quantize_with_row_sums(ta, dtype)
    assert torch.equal(got_q, want_q) and torch.equal(got_s, want_s)
    assert torch.equal(gmn, mn) and torch.equal(gmx, mx)
    got_q2, got_s2 = q.quantize_with_row_sums(ta, dtype, mn, mx)
    assert torch.equal(got_q2, want_q) and torch.equal(got_s2, want_s)
    np_t = {torch.uint8: np.uint8, torch.int8: np.int8, torch.int16: np.int16}[dtype]
    oq, _, _ = orc.quantize(a, np_t)
    assert np.array_equal(got_q.cpu().numpy(), oq)
    assert np.array_equal(got_s.cpu().numpy(), orc.reduce_sum(oq, True))
