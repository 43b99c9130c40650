"""Host-side checks that need no GPU: the library loads and exports its whole C ABI,
scalar host math agrees with the oracle, shape rules raise what the reference raises."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(pkg):
    header = (ROOT / "include" / "tfcc_b200.h").read_text()
    declared = set(re.findall(r"\b(tfccb200_\w+)\s*\(", header))
    assert len(declared) >= 16
    dll = ctypes.CDLL(str(pkg.library_path()))
    for name in sorted(declared):
        assert hasattr(dll, name), f"{name} is declared in include/tfcc_b200.h but not exported"
    from wechat_tfcc_b200._lib import EXPORTED_SYMBOLS
    assert declared == set(EXPORTED_SYMBOLS)


def test_version_and_strerror(pkg):
    assert pkg.lib.tfccb200_version() >= 100
    assert pkg.lib.tfccb200_strerror(0) == b"ok"
    assert b"invalid" in pkg.lib.tfccb200_strerror(-1)


def test_quantized_params_match_oracle(pkg, orc):
    rng = np.random.default_rng(11)
    cases = [(-128.0, 127.0, -128.0, 127.0), (0.0, 1.0, -1.0, 1.0)]
    for _ in range(200):
        amin = rng.uniform(-5, 5)
        bmin = rng.uniform(-5, 5)
        cases.append((amin, amin + rng.uniform(0.05, 5), bmin, bmin + rng.uniform(0.05, 5)))
    for c in cases:
        c = tuple(float(np.float32(x)) for x in c)
        got = pkg.quantization.matmul_params(*c)
        want = orc.matmul_params(*c)
        assert got[:2] == want[:2]
        assert np.float32(got[2]) == np.float32(want[2]) and np.float32(got[3]) == np.float32(want[3])


def test_golden_generator_offsets_match(pkg, golden):
    """Offsets the reference's generator used (a + aOffset) . (b + bOffset) are the ones the
    library derives: check through the expectation's first element."""
    from conftest import golden_cases
    npz = golden["quantization_mklquantizationmatmul"]
    for _, case in golden_cases(npz, "quantization/mklquantizationmatmul"):
        oa, ob, _, _ = pkg.quantization.matmul_params(case["aMin"][0], case["aMax"][0],
                                                      case["bMin"][0], case["bMax"][0])
        a, b = case["a"].astype(np.int64), case["b"].astype(np.int64)
        assert int(((a[0] + oa) * (b[:, 0] + ob)).sum()) == int(case["expect"][0, 0])


def test_path_choice_is_host_only(pkg):
    lib = pkg.lib
    assert lib.tfccb200_sgemm_path(1, 16384, 4096, 1, 0, 0, 0) == 2      # skinny
    assert lib.tfccb200_sgemm_path(8192, 8192, 8192, 1, 0, 0, 0) == 4   # CTA pairs
    assert lib.tfccb200_sgemm_path(32, 2048, 512, 1, 0, 0, 0) == 5       # config 1: few rows, small B
    assert lib.tfccb200_sgemm_path(16, 16384, 4096, 1, 0, 0, 0) == 2     # few rows, large B: streaming
    assert lib.tfccb200_sgemm_path(37, 41, 53, 1, 0, 0, 0) == 1         # ragged -> CUDA cores
    assert lib.tfccb200_sgemm_path(0, 4, 4, 1, 0, 0, 0) == -1
    # rank-3 x rank-2 folds the batch into rows: [8,128,768] x [768,3072]
    assert lib.tfccb200_sgemm_path(128, 3072, 768, 8, 128 * 768, 0, 0) in (3, 4)


def test_matmul_shape_errors_mirror_reference(pkg):
    ex = pkg.exceptions
    t = lambda *s: torch.zeros(*s)
    with pytest.raises(ex.InvalidArgumentError, match="two or more dimensions"):
        pkg.blas.matmul(t(3), t(3, 4))
    with pytest.raises(ex.InvalidArgumentError, match="shape invalid"):
        pkg.blas.matmul(t(2, 3), t(4, 4))
    with pytest.raises(ex.InvalidArgumentError, match="shape invalid"):
        pkg.blas.matmul(t(5, 2, 3), t(6, 3, 4))
    with pytest.raises(ex.InvalidArgumentError, match="shape invalid"):
        pkg.blas.matmul(t(2, 3), t(3, 4), t(5))
    with pytest.raises(ex.NotImplementedError):
        pkg.blas.matmul(torch.zeros(2, 3, dtype=torch.float64), torch.zeros(3, 4, dtype=torch.float64))
    # a CPU tensor is not "available" to the device session: loud error, no CPU fallback
    with pytest.raises(ex.InvalidArgumentError, match="CUDA"):
        pkg.blas.matmul(t(2, 3), t(3, 4))


def test_quantized_matmul_argument_errors_mirror_reference(pkg):
    ex = pkg.exceptions
    q = pkg.quantization
    a = torch.zeros(4, 8, dtype=torch.uint8)
    b = torch.zeros(8, 5, dtype=torch.int8)
    ra, rb = torch.zeros(4, dtype=torch.int32), torch.zeros(5, dtype=torch.int32)
    f = lambda v: torch.tensor([v], dtype=torch.float32)
    with pytest.raises(ex.InvalidArgumentError, match="invalid input tensor a"):
        q.matmul(torch.zeros(8, dtype=torch.uint8), ra, f(0), f(1), b, rb, f(0), f(1))
    with pytest.raises(ex.InvalidArgumentError, match="invalid tensor minA"):
        q.matmul(a, ra, torch.zeros(2), f(1), b, rb, f(0), f(1))
    with pytest.raises(ex.InvalidArgumentError, match="a and b don't match"):
        q.matmul(a, ra, f(0), f(1), torch.zeros(7, 5, dtype=torch.int8), rb, f(0), f(1))
    with pytest.raises(ex.InvalidArgumentError, match="reduceSumA don't match"):
        q.matmul(a, torch.zeros(3, dtype=torch.int32), f(0), f(1), b, rb, f(0), f(1))
    with pytest.raises(ex.InvalidArgumentError, match="reduceSumB don't match"):
        q.matmul(a, ra, f(0), f(1), b, torch.zeros(6, dtype=torch.int32), f(0), f(1))
    with pytest.raises(ex.InvalidArgumentError, match="invalid input tensor a"):
        q.reduce_sum(torch.zeros(4, dtype=torch.int8), True)


def test_shard_range(pkg):
    sr = pkg.parallel.shard_range
    for total in (0, 1, 7, 96, 8192):
        for world in (1, 2, 3, 8):
            spans = [sr(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        sr(10, 2, 2)
