"""Quantized matmul and reduce_sum on the GPU: bit-exact against the oracle and against the
reference generator's expectations (QuantizationTest.mkl_matmul..4,
tfcc/test/quantization.cpp:105-218)."""
import numpy as np
import pytest
import torch

from conftest import golden_cases

pytestmark = pytest.mark.gpu


def dev_of():
    return torch.device("cuda:0")


def f1(v):
    return torch.tensor([v], dtype=torch.float32)


def qrun(pkg, a, b, amin, amax, bmin, bmax, path="auto", rs_shared=False):
    d = dev_of()
    ta, tb = torch.from_numpy(a).to(d), torch.from_numpy(b).to(d)
    ra = pkg.quantization.reduce_sum(ta, True)
    rb = pkg.quantization.reduce_sum(tb, False)
    c, mn, mx = pkg.quantization.matmul(ta, ra, f1(amin), f1(amax), tb, rb, f1(bmin), f1(bmax),
                                        path=path)
    pkg.session.get_session(d).sync()
    return c.cpu().numpy(), float(mn.item()), float(mx.item()), ra.cpu().numpy(), rb.cpu().numpy()


def test_reference_generator_cases_bit_exact(pkg, golden):
    npz = golden["quantization_mklquantizationmatmul"]
    for i, case in golden_cases(npz, "quantization/mklquantizationmatmul"):
        got, _, _, _, _ = qrun(pkg, case["a"], case["b"], case["aMin"][0], case["aMax"][0],
                               case["bMin"][0], case["bMax"][0])
        assert got.dtype == np.int32
        assert np.array_equal(got, case["expect"]), i


def test_known_answers_5_11_17(pkg, orc):
    """quantize -> reduce_sum -> matmul -> dequantize; quantize/dequantize on the host by the
    oracle (they are outside this library), the middle on the GPU."""
    v1 = np.array([1, 2, 3, 4, 5, 6, 1, 2, 3, 4, 5, 6], np.float32)
    v2 = np.array([1, 2, 1, 2], np.float32)
    layouts = [(v1.reshape(2, 3, 2), v2.reshape(2, 2, 1)), (v1[:6].reshape(3, 2), v2.reshape(2, 2, 1)),
               (v1.reshape(2, 3, 2), v2[:2].reshape(2, 1))]
    for a, b in layouts:
        qa, amin, amax = orc.quantize(a, np.uint8)
        qb, bmin, bmax = orc.quantize(b, np.int8)
        qc, mn, mx, _, _ = qrun(pkg, qa, qb, amin, amax, bmin, bmax)
        r = orc.dequantize(qc, mn, mx)
        assert [int(x) for x in r.ravel()] == [5, 11, 17, 5, 11, 17]


@pytest.mark.parametrize("path", ["simt", "umma", "umma2"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (200, 384, 512), (130, 272, 144), (600, 1040, 2064)])
def test_paths_bit_exact(pkg, orc, path, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    got, mn, mx, ra, rb = qrun(pkg, a, b, -1.5, 2.0, -0.7, 0.9, path=path)
    want, wmn, wmx = orc.quantized_matmul(a, orc.reduce_sum(a, True), -1.5, 2.0, b,
                                          orc.reduce_sum(b, False), -0.7, 0.9, impl="port")
    assert np.array_equal(ra, orc.reduce_sum(a, True)) and np.array_equal(rb, orc.reduce_sum(b, False))
    assert np.array_equal(got, want)
    assert np.float32(mn) == np.float32(wmn) and np.float32(mx) == np.float32(wmx)


def test_batched_layouts_bit_exact(pkg, orc):
    rng = np.random.default_rng(21)
    for sa, sb in (((3, 50, 64), (3, 64, 48)), ((4, 40, 128), (128, 144)), ((30, 32), (2, 32, 16)),
                   ((2, 130, 256), (2, 256, 272))):
        a = rng.integers(0, 256, sa, dtype=np.uint8)
        b = rng.integers(-128, 128, sb, dtype=np.int8)
        for path in ("simt", "auto") + (("umma",) if sa[-1] % 16 == 0 and sb[-1] % 16 == 0 else ()):
            got, _, _, _, _ = qrun(pkg, a, b, -2.0, 3.0, -1.0, 1.0, path=path)
            want, _, _ = orc.quantized_matmul(a, orc.reduce_sum(a, True), -2.0, 3.0, b,
                                              orc.reduce_sum(b, False), -1.0, 1.0, impl="numpy")
            assert np.array_equal(got, want), (sa, sb, path)


@pytest.mark.parametrize("m,n,k", [(100, 128, 8192), (256, 512, 4096), (130, 144, 1040)])
def test_few_tiles_long_k_exact(pkg, orc, m, n, k):
    """Few output tiles and a long K (up to 64 k-blocks through one accumulator)."""
    rng = np.random.default_rng(m + k)
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, (k, n), dtype=np.int8)
    want, _, _ = orc.quantized_matmul(a, orc.reduce_sum(a, True), -1.5, 2.0, b,
                                      orc.reduce_sum(b, False), -0.7, 0.9, impl="port")
    for path in ("umma", "umma2", "auto"):
        got, _, _, _, _ = qrun(pkg, a, b, -1.5, 2.0, -0.7, 0.9, path=path)
        assert np.array_equal(got, want), path


@pytest.mark.parametrize("path", ["simt", "umma"])
def test_device_resident_ranges_match_host_derivation(pkg, orc, path):
    """With (min, max) in device memory the offsets and the result range are derived by a
    prologue kernel and read by the GEMM from device memory: same C, same (minC, maxC) bits as
    the host derivation of tfcc_mklquantization.cpp:181-193, for many ranges."""
    rng = np.random.default_rng(99)
    d = dev_of()
    m, n, k = 136, 272, 384
    qa = rng.integers(0, 256, (m, k), dtype=np.uint8)
    qb = rng.integers(-128, 128, (k, n), dtype=np.int8)
    ta, tb = torch.from_numpy(qa).to(d), torch.from_numpy(qb).to(d)
    ra, rb = pkg.quantization.reduce_sum(ta, True), pkg.quantization.reduce_sum(tb, False)
    dv = lambda v: torch.tensor([v], dtype=torch.float32, device=d)
    cases = [(-128.0, 127.0, -128.0, 127.0), (0.0, 1.0, -1.0, 1.0), (-3.0, -3.0, 1.0, 2.0)]
    for _ in range(20):
        lo_a, lo_b = rng.uniform(-5, 5), rng.uniform(-5, 5)
        cases.append((lo_a, lo_a + rng.uniform(0.05, 5), lo_b, lo_b + rng.uniform(0.05, 5)))
    for c in cases:
        c = tuple(float(np.float32(x)) for x in c)
        if c[0] >= c[1]:
            continue  # the reference divides by zero here; not a defined case
        got, gmin, gmax = pkg.quantization.matmul(ta, ra, dv(c[0]), dv(c[1]), tb, rb, dv(c[2]), dv(c[3]),
                                                  path=path)
        want, wmin, wmax = orc.quantized_matmul(qa, orc.reduce_sum(qa, True), c[0], c[1], qb,
                                                orc.reduce_sum(qb, False), c[2], c[3], impl="port")
        assert np.array_equal(got.cpu().numpy(), want), c
        assert np.float32(gmin.item()) == np.float32(wmin) and np.float32(gmax.item()) == np.float32(wmax), c


def test_n_equals_one_fast_path_shape(pkg, orc):
    rng = np.random.default_rng(22)
    a = rng.integers(0, 256, (333, 401), dtype=np.uint8)
    b = rng.integers(-128, 128, (401, 1), dtype=np.int8)
    got, _, _, _, _ = qrun(pkg, a, b, -4.0, -1.0, 0.5, 3.0)
    want, _, _ = orc.quantized_matmul(a, orc.reduce_sum(a, True), -4.0, -1.0, b,
                                      orc.reduce_sum(b, False), 0.5, 3.0, impl="port")
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,path", [(256, "auto"), (256, "umma"), (4096, "umma2")])
def test_config3_zero_points_bit_exact(pkg, orc, m, path):
    """u8 [m,4096] x s8 [4096,4096], zero points 128 / 0 (ranges (-128,127)).  The expectation
    is computed in float64 BLAS, which is exact here: every partial sum is an integer below 2^53."""
    rng = np.random.default_rng(2)
    a = rng.integers(0, 256, (m, 4096), dtype=np.uint8)
    b = rng.integers(-127, 128, (4096, 4096), dtype=np.int8)
    got, mn, mx, _, rb = qrun(pkg, a, b, -128.0, 127.0, -128.0, 127.0, path=path)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64) - 128 * rb.astype(np.int64)[None, :]
    assert np.array_equal(got.astype(np.int64), want)
    assert (mn, mx) == (-2147483648.0, 2147483648.0)
    if m == 256:  # and the C restatement of the reference algorithm agrees
        port, _, _ = orc.quantized_matmul(a, orc.reduce_sum(a, True), -128.0, 127.0, b,
                                          orc.reduce_sum(b, False), -128.0, 127.0, impl="port")
        assert np.array_equal(got, port)


def test_int32_wraparound_matches_reference_arithmetic(pkg, orc):
    """Offsets large enough to overflow int32 in the correction terms: the result must wrap
    exactly as the reference's int32 arithmetic does."""
    rng = np.random.default_rng(23)
    a = rng.integers(200, 256, (64, 4096), dtype=np.uint8)
    b = rng.integers(100, 128, (4096, 128), dtype=np.int8)
    got, _, _, _, _ = qrun(pkg, a, b, 3.0, 3.05, 4.0, 4.05)   # offsets in the tens of thousands
    want, _, _ = orc.quantized_matmul(a, orc.reduce_sum(a, True), 3.0, 3.05, b,
                                      orc.reduce_sum(b, False), 4.0, 4.05, impl="port")
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.int16])
def test_reduce_sum_all_types(pkg, orc, dtype):
    rng = np.random.default_rng(24)
    info = np.iinfo(dtype)
    d = dev_of()
    for shape in ((257, 515), (3, 64, 4096), (2, 2, 33, 17), (1, 1), (4096, 4096), (256, 4096),
                  (5, 1000, 48), (70, 16400), (3, 9, 2064), (1037, 640), (600, 10240),
                  (2, 300, 5120)):
        a = rng.integers(info.min, info.max + 1, shape).astype(dtype)
        t = torch.from_numpy(a).to(d)
        for row in (True, False):
            got = pkg.quantization.reduce_sum(t, row).cpu().numpy()
            assert got.dtype == np.int32
            assert np.array_equal(got, orc.reduce_sum(a, row)), (shape, row)


def test_host_buffer_entry_point(pkg, orc):
    rng = np.random.default_rng(25)
    a = rng.integers(0, 256, (2, 96, 256), dtype=np.uint8)
    b = rng.integers(-128, 128, (256, 160), dtype=np.int8)
    got, mn, mx = pkg.quantization.matmul_host(a, b, -1.0, 1.0, -2.0, 2.0)
    want, wmn, wmx = orc.quantized_matmul(a, orc.reduce_sum(a, True), -1.0, 1.0, b,
                                          orc.reduce_sum(b, False), -2.0, 2.0, impl="numpy")
    assert np.array_equal(got, want)
    assert np.float32(mn) == np.float32(wmn) and np.float32(mx) == np.float32(wmx)
