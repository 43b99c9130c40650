"""The CPU oracle against the reference's own expectations (no GPU needed).

Golden arrays come from the reference's numpy generators
(tests/golden/make_golden.py); the known answers 5 / 11 / 17 are the literal
expectations of tfcc/test/quantization.cpp:105-189.
"""
import numpy as np
import pytest

from conftest import golden_cases


def test_fp32_oracle_matches_reference_expectations(orc, golden):
    for prefix, key in (("blas/matmul", "blas_matmul"), ("blas/matmulwithblas", "blas_matmulwithblas")):
        n = 0
        for _, case in golden_cases(golden[key], prefix):
            want = case["expect"]
            for dtype in (np.float64, np.float32):
                got = orc.blas_matmul(case["a"], case["b"], case.get("c"), dtype=dtype)
                assert got.shape == want.shape
                assert orc.is_similar(got, want)
            # tighter than the reference's predicate: the float64 product is the truth
            truth = orc.blas_matmul(case["a"], case["b"], case.get("c"))
            assert orc.normwise_rel_error(want, truth) < 1e-5
            n += 1
        assert n == 20


@pytest.mark.parametrize("impl", ["numpy", "port", "ref"])
def test_int8_oracle_matches_reference_expectations_exactly(orc, golden, impl):
    if impl == "ref" and orc.ref_lib() is None:
        pytest.skip("reference kernel not built (reference tree absent)")
    npz = golden["quantization_mklquantizationmatmul"]
    n = 0
    for _, case in golden_cases(npz, "quantization/mklquantizationmatmul"):
        a, b = case["a"], case["b"]
        ra, rb = orc.reduce_sum(a, True), orc.reduce_sum(b, False)
        got, _, _ = orc.quantized_matmul(a, ra, case["aMin"][0], case["aMax"][0], b, rb,
                                         case["bMin"][0], case["bMax"][0], impl=impl)
        assert got.dtype == np.int32
        assert np.array_equal(got, case["expect"])
        n += 1
    assert n == 15


@pytest.mark.parametrize("impl", ["numpy", "port", "ref"])
def test_known_answer_quantized_dense(orc, impl):
    if impl == "ref" and orc.ref_lib() is None:
        pytest.skip("reference kernel not built (reference tree absent)")
    v1 = np.array([1, 2, 3, 4, 5, 6, 1, 2, 3, 4, 5, 6], np.float32)
    v2 = np.array([1, 2, 1, 2], np.float32)
    layouts = [(v1.reshape(2, 3, 2), v2.reshape(2, 2, 1)),      # mkl_matmul
               (v1[:6].reshape(3, 2), v2.reshape(2, 2, 1)),     # mkl_matmul2
               (v1.reshape(2, 3, 2), v2[:2].reshape(2, 1))]     # mkl_matmul3
    for a, b in layouts:
        r = orc.quantized_dense(a, b, impl=impl)
        assert [int(x) for x in r.ravel()] == [5, 11, 17, 5, 11, 17]


def test_port_and_reference_kernel_agree_on_batches(orc):
    rng = np.random.default_rng(7)
    for shape_a, shape_b in (((3, 50, 70), (3, 70, 33)), ((4, 25, 64), (64, 48)), ((30, 17), (2, 17, 9))):
        a = rng.integers(0, 256, shape_a, dtype=np.uint8)
        b = rng.integers(-128, 128, shape_b, dtype=np.int8)
        ra, rb = orc.reduce_sum(a, True), orc.reduce_sum(b, False)
        base, mn, mx = orc.quantized_matmul(a, ra, -3.0, 1.5, b, rb, -0.5, 2.5, impl="numpy")
        for impl in ("port", "ref"):
            if impl == "ref" and orc.ref_lib() is None:
                continue
            got, mn2, mx2 = orc.quantized_matmul(a, ra, -3.0, 1.5, b, rb, -0.5, 2.5, impl=impl)
            assert np.array_equal(got, base)
            assert (mn, mx) == (mn2, mx2)


def test_zero_point_config_offsets(orc):
    # "zero-point 128 / 0": ranges (-128,127) give offA = -128, offB = 0 and the full int32 range
    assert orc.matmul_params(-128, 127, -128, 127) == (-128, 0, -2147483648.0, 2147483648.0)


def test_reduce_sum_shapes_and_errors(orc):
    a = np.arange(2 * 3 * 4, dtype=np.int16).reshape(2, 3, 4)
    assert orc.reduce_sum(a, True).shape == (2, 3)
    assert orc.reduce_sum(a, False).shape == (2, 4)
    with pytest.raises(orc.OracleError):
        orc.reduce_sum(np.zeros(4, np.int8), True)


def test_matmul_shape_rules(orc):
    ok = [((2, 3), (3, 4)), ((5, 6, 2, 3), (5, 6, 3, 4)), ((5, 2, 3), (3, 4)), ((2, 3), (7, 3, 4))]
    for sa, sb in ok:
        assert orc.matmul_result_shape(sa, sb)[-2:] == (2, 4)
    bad = [((3,), (3, 4)), ((2, 3), (4, 4)), ((5, 2, 3), (6, 3, 4)), ((5, 6, 2, 3), (6, 3, 4))]
    for sa, sb in bad:
        with pytest.raises(orc.OracleError):
            orc.matmul_result_shape(sa, sb)
    with pytest.raises(orc.OracleError):
        orc.matmul_result_shape((2, 3), (3, 4), (5,))


# ---- quantize / dequantize / requantize (tfcc/test/quantization.cpp:40-102) ----
DEQUANT_IN = np.array([23, -115, -128, 127, -20, -11], np.int8)
DEQUANT_EXPECT = np.array([9.9372554e-01, -2.1992157e+00, -2.5000000e+00, 3.4000001e+00,
                           -1.1765957e-03, 2.0705891e-01], np.float32)
REQUANT_EXPECT = np.array([24125, 18500, 17970, 28364, 22372, 22739], np.uint16)


def test_quantize_oracle_matches_reference_generator(orc, golden):
    n = 0
    for _, case in golden_cases(golden["quantization_quantize"], "quantization/quantize"):
        q8, _, _ = orc.quantize(case["a"], np.int8)
        u8, _, _ = orc.quantize(case["a"], np.uint8)
        assert np.array_equal(q8, case["int8_a"]) and np.array_equal(u8, case["uint8_a"])
        n += 1
    assert n == 20


def test_dequantize_and_requantize_known_answers(orc):
    got = orc.dequantize(DEQUANT_IN, -2.5, 3.4)
    # the reference compares after adding (max - min) to both sides, with is_similar
    assert orc.is_similar(got + np.float32(5.9), DEQUANT_EXPECT + np.float32(5.9))
    assert np.array_equal(orc.requantize(DEQUANT_IN, -2.5, 3.4, -12.7, 24.5, np.uint16), REQUANT_EXPECT)
    # degenerate ranges
    assert np.all(orc.quantize(np.full((3, 3), 1.5, np.float32), np.int8)[0] == -128)
    assert np.all(orc.dequantize(DEQUANT_IN, 2.0, 2.0) == np.float32(2.0))
    assert np.all(orc.requantize(DEQUANT_IN, -1.0, 1.0, 3.0, 3.0, np.int16) == -32768)


def _glue_cases(golden):
    """(kind, a float32, extra, expect) for the reference generators of softmax, gelu_accurate
    and layer_normalization (tfcc/test/python/testcase/math/softmax.py, math/gelu_accurate.py,
    layer/layer_normalization.py; consumed by tfcc/test/math.cpp:577-655, layer.cpp:36-50)."""
    for _, c in golden_cases(golden["math_softmax"], "math/softmax"):
        yield "softmax", c["a"], int(c["axis"][0]), c["expect"]
    for _, c in golden_cases(golden["math_gelu_accurate"], "math/gelu_accurate"):
        yield "gelu", c["a"], None, c["expect"]
    for _, c in golden_cases(golden["layer_layer_normalization"], "layer/layer_normalization"):
        yield "layer_norm", c["a"], (int(c["axis"][0]), c["LayerNorm/gamma"], c["LayerNorm/beta"]), c["expect"]


def glue_oracle(orc, kind, a, extra):
    """The oracle's restatement applied the way the reference operator is: softmax along any
    axis is the last-axis softmax of the moved axis; layer normalisation over the trailing
    axes is the row-wise one over their flattened extent (epsilon 1e-12 as the generator)."""
    if kind == "softmax":
        moved = np.moveaxis(a, extra, -1)
        return np.moveaxis(orc.softmax_v2(np.ascontiguousarray(moved)), -1, extra)
    if kind == "gelu":
        return orc.gelu_accurate(a)
    axis, gamma, beta = extra
    cols = int(np.prod(a.shape[axis:]))
    out = orc.layer_normalize(a.reshape(-1, cols), gamma.reshape(cols), beta.reshape(cols), eps=1e-12)
    return out.reshape(a.shape)


def test_glue_oracles_match_reference_expectations(orc, golden):
    """softmaxV2, geluAccurate and the layer normalisation restated in the oracle, pinned to
    the expectations of the reference's own generators with the reference's predicate."""
    seen = {"softmax": 0, "gelu": 0, "layer_norm": 0}
    for kind, a, extra, expect in _glue_cases(golden):
        got = glue_oracle(orc, kind, a, extra)
        assert got.shape == expect.shape
        assert orc.is_similar(got, expect), (kind, a.shape)
        assert np.abs(got.astype(np.float64) - expect).max() < 5e-6, (kind, a.shape)
        seen[kind] += 1
    assert all(v == 5 for v in seen.values()), seen
