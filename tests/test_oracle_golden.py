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
