"""fp32 matmul parity on the GPU, through the package's operator (which calls the C ABI).

Tolerances.  FP32 mode: normwise relative error against the float64 product <= 1e-5 (the
stated target), and the reference's own predicate ``is_similar`` (|a-b| < 1e-3|a+b| or
< 1e-5, tfcc/core/utils/tfcc_debugutils.cpp:102-127) against the reference generator's
expectation.  TF32 mode (opt-in): normwise <= 2e-3.
"""
import numpy as np
import pytest
import torch

from conftest import golden_cases

pytestmark = pytest.mark.gpu
TOL_FP32 = 1e-5
TOL_TF32 = 2e-3


def dev_of():
    return torch.device("cuda:0")


def run(pkg, a, b, c=None, **kw):
    d = dev_of()
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(d)
    out = pkg.blas.matmul(t(a), t(b), t(c) if c is not None else None, **kw)
    pkg.session.get_session(d).sync()
    return out.cpu().numpy()


@pytest.mark.parametrize("key,prefix", [("blas_matmul", "blas/matmul"),
                                        ("blas_matmulwithblas", "blas/matmulwithblas")])
def test_reference_generator_cases(pkg, orc, golden, key, prefix):
    """BlasTest.matmul / matmul_with_blas (tfcc/test/blas.cpp:34-61): all four batch layouts,
    m,n,k in [1,100), values U(-1,1)."""
    for i, case in golden_cases(golden[key], prefix):
        got = run(pkg, case["a"], case["b"], case.get("c"))
        assert got.shape == case["expect"].shape, i
        assert orc.is_similar(got, case["expect"]), i
        truth = orc.blas_matmul(case["a"], case["b"], case.get("c"))
        assert orc.normwise_rel_error(got, truth) < TOL_FP32, i


@pytest.mark.parametrize("path", ["simt", "umma", "umma2", "auto"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 32), (300, 516, 132), (129, 260, 36), (1, 64, 64),
                                   (257, 1028, 1000), (1024, 768, 768)])
def test_paths_agree_with_float64_product(pkg, orc, path, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.5, (k, n)).astype(np.float32)
    c = rng.normal(0, 1, n).astype(np.float32)
    truth = orc.blas_matmul(a, b, c)
    got = run(pkg, a, b, c, path=path)
    assert orc.normwise_rel_error(got, truth) < TOL_FP32


@pytest.mark.parametrize("path", ["umma", "umma2", "simt"])
def test_batched_layouts(pkg, orc, path):
    rng = np.random.default_rng(5)
    shapes = [((6, 128, 64), (6, 64, 128)),       # equal ranks
              ((3, 2, 40, 64), (3, 2, 64, 72)),   # rank 4
              ((5, 70, 96), (96, 132)),           # rank-2 B shared (folds into rows)
              ((50, 96), (4, 96, 68))]            # rank-2 A shared
    for sa, sb in shapes:
        a = rng.uniform(-1, 1, sa).astype(np.float32)
        b = rng.uniform(-1, 1, sb).astype(np.float32)
        got = run(pkg, a, b, path=path)
        truth = orc.blas_matmul(a, b)
        assert got.shape == truth.shape
        assert orc.normwise_rel_error(got, truth) < TOL_FP32, (sa, sb)


def test_tensor_core_path_rejects_unaligned_pitch(pkg):
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (64, 33)).astype(np.float32)
    b = rng.uniform(-1, 1, (33, 64)).astype(np.float32)
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        run(pkg, a, b, path="umma")


def test_config1_single_matmul(pkg, orc):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (32, 512)).astype(np.float32)
    b = rng.normal(0, 0.02, (512, 2048)).astype(np.float32)
    got = run(pkg, a, b)
    assert orc.normwise_rel_error(got, orc.blas_matmul(a, b)) < TOL_FP32
    assert orc.is_similar(got, orc.blas_matmul(a, b, dtype=np.float32))


def test_config2_attention_batches(pkg, orc):
    rng = np.random.default_rng(1)
    q, k, v = (rng.normal(0, 1, (96, 128, 64)).astype(np.float32) for _ in range(3))
    kt = np.ascontiguousarray(k.transpose(0, 2, 1))
    s_truth = orc.blas_matmul(q, kt)
    s = run(pkg, q, kt)
    assert orc.normwise_rel_error(s, s_truth) < TOL_FP32
    # row softmax of S/8 in fp32 from the oracle's S, so both sides multiply the same P
    z = (s_truth.astype(np.float32) / np.float32(8.0))
    z = np.exp(z - z.max(axis=-1, keepdims=True))
    p = (z / z.sum(axis=-1, keepdims=True)).astype(np.float32)
    o = run(pkg, p, v)
    assert orc.normwise_rel_error(o, orc.blas_matmul(p, v)) < TOL_FP32


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 12, 16, 27, 32])
def test_skinny_decode_shapes(pkg, orc, m):
    rng = np.random.default_rng(50 + m)
    w = rng.normal(0, 0.02, (4096, 16384)).astype(np.float32)
    x = rng.normal(0, 1, (m, 4096)).astype(np.float32)
    bias = rng.normal(0, 1, 16384).astype(np.float32)
    truth = orc.blas_matmul(x, w, bias)
    for path in ("skinny", "auto"):
        got = run(pkg, x, w, bias, path=path)
        assert orc.normwise_rel_error(got, truth) < TOL_FP32


def test_streaming_kernel_takes_config1(pkg, orc):
    """Config 1 (32 x 512 x 2048) through the streaming kernel, which can serve up to 32 rows
    (left to itself the planner uses it up to 16 rows against a large B, and the one-launch
    cluster kernel for this shape): fp32 FMA in k order, within the fp32 tolerance like every
    other path."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (32, 512)).astype(np.float32)
    b = rng.normal(0, 0.02, (512, 2048)).astype(np.float32)
    bias = rng.normal(0, 1, 2048).astype(np.float32)
    for path in ("skinny", "auto"):
        got = run(pkg, a, b, bias, path=path)
        assert orc.normwise_rel_error(got, orc.blas_matmul(a, b, bias)) < TOL_FP32


@pytest.mark.parametrize("m,k,n", [(32, 512, 2048), (1, 64, 4), (7, 100, 260), (32, 2048, 512),
                                   (17, 2044, 300), (8, 8, 8), (25, 33, 1028), (9, 777, 1024)])
def test_cluster_kernel_for_few_rows_and_small_b(pkg, orc, m, k, n):
    """One launch on CUDA cores, K cut into ways and cluster slices that are added through
    distributed shared memory (config 1 is the first shape): fp32 FMA, fp32 tolerance, with and
    without bias, with the GELU epilogue, and the same bits on every run (fixed order of the
    slices)."""
    rng = np.random.default_rng(m * 31 + k + n)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.05, (k, n)).astype(np.float32)
    bias = rng.normal(0, 1, n).astype(np.float32)
    got = run(pkg, a, b, path="cluster_simt")
    assert orc.normwise_rel_error(got, orc.blas_matmul(a, b)) < TOL_FP32
    got_b = run(pkg, a, b, bias, path="cluster_simt")
    assert orc.normwise_rel_error(got_b, orc.blas_matmul(a, b, bias)) < TOL_FP32
    assert np.array_equal(got_b, run(pkg, a, b, bias, path="cluster_simt"))
    got_g = run(pkg, a, b, bias, path="cluster_simt", activation="gelu")
    want_g = orc.gelu_accurate(orc.blas_matmul(a, b, bias).astype(np.float32))
    assert orc.normwise_rel_error(got_g, want_g) < TOL_FP32


def test_cluster_kernel_batched_and_planner(pkg, orc):
    rng = np.random.default_rng(77)
    x = rng.normal(0, 1, (3, 5, 333)).astype(np.float32)
    w = rng.normal(0, 1, (3, 333, 1100)).astype(np.float32)
    got = run(pkg, x, w, path="cluster_simt")
    assert orc.normwise_rel_error(got, orc.blas_matmul(x, w)) < TOL_FP32
    # rank-3 A against one B: the batch becomes rows (here 4 x 6 = 24 rows)
    x2 = rng.normal(0, 1, (4, 6, 256)).astype(np.float32)
    w2 = rng.normal(0, 1, (256, 512)).astype(np.float32)
    assert orc.normwise_rel_error(run(pkg, x2, w2, path="cluster_simt"), orc.blas_matmul(x2, w2)) < TOL_FP32
    # config 1 goes there by itself; a long K or a large B does not
    assert pkg.lib.tfccb200_sgemm_path(32, 2048, 512, 1, 0, 0, 0) == 5
    assert pkg.lib.tfccb200_sgemm_path(32, 2048, 4096, 1, 0, 0, 0) != 5
    assert pkg.lib.tfccb200_sgemm_path(8, 16384, 1024, 1, 0, 0, 0) != 5
    with pytest.raises(pkg.exceptions.TFCCError):
        run(pkg, rng.normal(0, 1, (4, 4096)).astype(np.float32),
            rng.normal(0, 1, (4096, 64)).astype(np.float32), path="cluster_simt")


def test_skinny_ragged_and_batched(pkg, orc):
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, (3, 5, 333)).astype(np.float32)
    w = rng.normal(0, 1, (3, 333, 1100)).astype(np.float32)
    got = run(pkg, x, w, path="skinny")
    assert orc.normwise_rel_error(got, orc.blas_matmul(x, w)) < TOL_FP32


def test_tf32_mode_has_its_own_tolerance(pkg, orc):
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (512, 1024)).astype(np.float32)
    b = rng.uniform(-1, 1, (1024, 512)).astype(np.float32)
    truth = orc.blas_matmul(a, b)
    for path in ("umma", "umma2"):
        err = orc.normwise_rel_error(run(pkg, a, b, path=path, precision="tf32"), truth)
        assert 1e-5 < err < TOL_TF32   # really a single TF32 pass, and within its bound


def test_bf16_mode_has_its_own_tolerance(pkg, orc):
    """Opt-in bfloat16 products (operands rounded to bf16, fp32 accumulation): normwise error
    against float64 below 1e-2, and equal to the float64 product of the bf16-rounded operands
    to fp32 accuracy, which shows that rounding the inputs is the only loss."""
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (384, 1024)).astype(np.float32)
    b = rng.uniform(-1, 1, (1024, 640)).astype(np.float32)
    bias = rng.uniform(-1, 1, 640).astype(np.float32)
    truth = orc.blas_matmul(a, b, bias)
    r16 = lambda x: torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    truth16 = orc.blas_matmul(r16(a), r16(b), bias)
    for path in ("umma", "umma2", "auto"):
        got = run(pkg, a, b, bias, path=path, precision="bf16")
        err = orc.normwise_rel_error(got, truth)
        assert 1e-4 < err < 1e-2, (path, err)
        assert orc.normwise_rel_error(got, truth16) < 1e-5, path
    # batched, and a pitch the bf16 tensor maps cannot take (falls back to fp32 accuracy)
    a3 = rng.uniform(-1, 1, (3, 130, 72)).astype(np.float32)
    b3 = rng.uniform(-1, 1, (3, 72, 136)).astype(np.float32)
    assert orc.normwise_rel_error(run(pkg, a3, b3, precision="bf16"), orc.blas_matmul(a3, b3)) < 1e-2
    a4 = rng.uniform(-1, 1, (64, 36)).astype(np.float32)
    b4 = rng.uniform(-1, 1, (36, 68)).astype(np.float32)
    assert orc.normwise_rel_error(run(pkg, a4, b4, precision="bf16"), orc.blas_matmul(a4, b4)) < 1e-5


def test_large_gemm_sampled_rows_and_linearity(pkg, orc):
    """4096 x 8192 x 8192 on the CTA-pair path: sampled rows against float64, bit-for-bit
    repeatability, and exact scaling by a power of two (a property that holds at any size)."""
    d = dev_of()
    g = torch.Generator(device=d)
    g.manual_seed(4)
    a = torch.empty((4096, 8192), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    b = torch.empty((8192, 8192), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    c1 = pkg.blas.matmul(a, b)
    c2 = pkg.blas.matmul(a, b)
    c4 = pkg.blas.matmul(a * 4.0, b)
    pkg.session.get_session(d).sync()
    assert torch.equal(c1, c2)
    assert torch.equal(c4, c1 * 4.0)
    rows = np.sort(np.random.default_rng(0).choice(4096, 64, replace=False))
    truth = a[rows].double().cpu().numpy() @ b.double().cpu().numpy()
    assert orc.normwise_rel_error(c1[rows].cpu().numpy(), truth) < TOL_FP32


def test_empty_operand_returns_result_shape(pkg):
    d = dev_of()
    out = pkg.blas.matmul(torch.zeros((0, 5), device=d), torch.zeros((5, 7), device=d))
    assert tuple(out.shape) == (0, 7)


def test_host_buffer_entry_point(pkg, orc):
    rng = np.random.default_rng(12)
    a = rng.uniform(-1, 1, (3, 200, 260)).astype(np.float32)
    b = rng.uniform(-1, 1, (260, 516)).astype(np.float32)
    c = rng.uniform(-1, 1, 516).astype(np.float32)
    got = pkg.blas.matmul_host(a, b, c)
    assert orc.normwise_rel_error(got, orc.blas_matmul(a, b, c)) < TOL_FP32
    x = rng.normal(0, 1, (2, 1024)).astype(np.float32)
    w = rng.normal(0, 1, (1024, 2048)).astype(np.float32)
    assert orc.normwise_rel_error(pkg.blas.matmul_host(x, w), orc.blas_matmul(x, w)) < TOL_FP32


@pytest.mark.parametrize("m", [2049, 2056, 2057, 3000])
def test_host_buffer_pipelined_path_ragged_rows(pkg, orc, m):
    """Large single products go up in row blocks (512 rows) while earlier blocks are multiplied and
    downloaded.  A row count that leaves eight rows or fewer for the last block must not send
    that block to the M <= 8 kernel (which would need scratch of another size): it is merged
    into the block before it.  Sampled rows, including the very last ones, against float64."""
    rng = np.random.default_rng(m)
    n, k = 3072, 3076  # 4 (m k + k n + m n) is past the 64 MB that turns the pipeline on
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    got = pkg.blas.matmul_host(a, b, bias)
    rows = np.unique(np.concatenate([rng.choice(m, 24, replace=False), np.arange(m - 10, m),
                                     np.arange(1020, 1028)]))
    want = orc.blas_matmul(a[rows], b, bias)
    assert orc.normwise_rel_error(got[rows], want) < TOL_FP32
    assert np.isfinite(got).all()


def test_head_truncation_setting_does_not_change_bits(pkg):
    """The library feeds raw fp32 tiles as the TF32 head operand.  That is only right if the
    tensor core ignores the 13 low mantissa bits; masking them explicitly on the host must
    then give the same single-pass product bit for bit."""
    d = dev_of()
    g = torch.Generator(device=d)
    g.manual_seed(9)
    a = torch.empty((256, 512), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    b = torch.empty((512, 256), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    mask = lambda t: (t.view(torch.int32) & -8192).view(torch.float32)
    c_raw = pkg.blas.matmul(a, b, precision="tf32", path="umma")
    c_msk = pkg.blas.matmul(mask(a), mask(b), precision="tf32", path="umma")
    pkg.session.get_session(d).sync()
    assert torch.equal(c_raw, c_msk)


def test_nsplit_push_entry_point_on_one_gpu(pkg, orc):
    """tfccb200_sgemm_nsplit_push with two 'ranks' played one after the other on one GPU: each
    pushes its column shard of C into both full-size result matrices.  Checks the column
    offsets, the row pitch and the multi-destination stores; the NVLink part needs two GPUs
    and is exercised by `bench.py --gpus N --check`."""
    import ctypes as C
    d = dev_of()
    rng = np.random.default_rng(77)
    m, k, ns, g = 300, 260, 132, 2
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, g * ns)).astype(np.float32)
    bias = rng.uniform(-1, 1, g * ns).astype(np.float32)
    ta = torch.from_numpy(a).to(d)
    outs = [torch.full((m, g * ns), float("nan"), dtype=torch.float32, device=d) for _ in range(g)]
    ptrs = (C.c_void_p * g)(*[o.data_ptr() for o in outs])
    stream = torch.cuda.current_stream(d).cuda_stream
    for r in range(g):
        tb = torch.from_numpy(np.ascontiguousarray(b[:, r * ns:(r + 1) * ns])).to(d)
        tbias = torch.from_numpy(np.ascontiguousarray(bias[r * ns:(r + 1) * ns])).to(d)
        st = pkg.lib.tfccb200_sgemm_nsplit_push(stream, ta.data_ptr(), tb.data_ptr(), ptrs, g, r,
                                                tbias.data_ptr(), m, ns, k, 0, None, None, 0, None)
        assert st == 0, pkg.lib.tfccb200_strerror(st)
        torch.cuda.synchronize()
    truth = orc.blas_matmul(a, b, bias)
    for o in outs:
        assert orc.normwise_rel_error(o.cpu().numpy(), truth) < TOL_FP32
    assert torch.equal(outs[0], outs[1])
    # misaligned shard width is refused
    assert pkg.lib.tfccb200_sgemm_nsplit_push(stream, ta.data_ptr(), ta.data_ptr(), ptrs, g, 0, None,
                                              m, 130, k, 0, None, None, 0, None) == -2


def _sgemm_raw(pkg, a, b, bias, path, workspace):
    """tfccb200_sgemm_ex on device tensors, with or without scratch."""
    d = a.device
    batch = a.shape[0] if a.dim() == 3 else 1
    m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
    out = torch.empty((batch, m, n) if a.dim() == 3 else (m, n), dtype=torch.float32, device=d)
    ws = None
    if workspace:
        nbytes = pkg.lib.tfccb200_sgemm_workspace(m, n, k, batch, 0)
        assert nbytes > 0
        ws = torch.empty(nbytes, dtype=torch.uint8, device=d)
    st = pkg.lib.tfccb200_sgemm_ex(
        torch.cuda.current_stream(d).cuda_stream, a.data_ptr(), m * k if a.dim() == 3 else 0,
        b.data_ptr(), k * n if b.dim() == 3 else 0, out.data_ptr(), m * n,
        bias.data_ptr() if bias is not None else None, m, n, k, batch, 0, pkg._lib.PATHS[path],
        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, None)
    assert st == 0, pkg.lib.tfccb200_strerror(st)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("path,m,n,k,batch", [
    ("umma2", 4096, 4096, 1024, 1),   # 256 pair tiles on 74 pairs: 3.46 waves
    ("umma", 1024, 3072, 768, 1),     # 192 tiles on 148 CTAs: 1.3 waves
    ("umma", 2176, 2304, 512, 1),     # ragged edge tiles
    ("umma", 256, 256, 384, 40),      # batched
    ("umma2", 4096, 2048, 1000, 1),   # K not a whole number of chunks: falls back to tile order
])
def test_k_shared_last_wave_is_bit_identical(pkg, orc, path, m, n, k, batch):
    """With scratch the fp32 tensor-core kernel shares the tiles of a ragged last wave by
    k-block between CTAs; the cuts fall on accumulation-chunk boundaries and the finishing CTA
    continues the running sums, so the result equals the tile-by-tile run bit for bit."""
    d = dev_of()
    g = torch.Generator(device=d)
    g.manual_seed(m + n + k)
    shape_a = (batch, m, k) if batch > 1 else (m, k)
    shape_b = (batch, k, n) if batch > 1 else (k, n)
    a = torch.empty(shape_a, dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    b = torch.empty(shape_b, dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    bias = torch.empty((n,), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    plain = _sgemm_raw(pkg, a, b, bias, path, workspace=False)
    shared = _sgemm_raw(pkg, a, b, bias, path, workspace=True)
    again = _sgemm_raw(pkg, a, b, bias, path, workspace=True)
    assert torch.equal(plain, shared)
    assert torch.equal(shared, again)
    rows = np.random.default_rng(0).choice(m, size=8, replace=False)
    a0 = (a[0] if batch > 1 else a).cpu().numpy()
    b0 = (b[0] if batch > 1 else b).cpu().numpy()
    truth = a0[rows].astype(np.float64) @ b0.astype(np.float64) + bias.cpu().numpy().astype(np.float64)
    got = (shared[0] if batch > 1 else shared)[torch.from_numpy(rows).to(d)].cpu().numpy()
    assert orc.normwise_rel_error(got, truth) < TOL_FP32


def test_k_shared_by_consecutive_ctas_through_scratch(pkg, orc):
    """Few tiles and a long K (the encoder's second FFN layer): with scratch the plan lets
    three consecutive CTAs share a tile's k-blocks and the first of them adds the others'
    partial tiles in rank order.  Deterministic, within the fp32 tolerance; the grouping of the
    sum differs from the unsplit run, so the two are compared by error, not bit for bit."""
    d = dev_of()
    g = torch.Generator(device=d)
    g.manual_seed(77)
    m, k, n = 1024, 3072, 768
    a = torch.empty((m, k), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    b = torch.empty((k, n), dtype=torch.float32, device=d).normal_(0, 0.02, generator=g)
    bias = torch.empty((n,), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
    plain = _sgemm_raw(pkg, a, b, bias, "auto", workspace=False)
    shared = _sgemm_raw(pkg, a, b, bias, "auto", workspace=True)
    again = _sgemm_raw(pkg, a, b, bias, "auto", workspace=True)
    assert torch.equal(shared, again)
    truth = a.cpu().numpy().astype(np.float64) @ b.cpu().numpy().astype(np.float64) + \
        bias.cpu().numpy().astype(np.float64)
    assert orc.normwise_rel_error(shared.cpu().numpy(), truth) < TOL_FP32
    assert orc.normwise_rel_error(plain.cpu().numpy(), truth) < TOL_FP32


def test_random_shapes_through_the_planner(pkg, orc):
    """Forty seeded shapes in the tensor-core range, with scratch (so that the planner may pick
    any of: whole tiles, K split over a cluster, K split through scratch, k-shared last wave,
    CTA pairs): every result within the fp32 tolerance of the float64 product on sampled rows,
    and identical on a second run."""
    d = dev_of()
    rng = np.random.default_rng(2024)
    g = torch.Generator(device=d)
    g.manual_seed(2024)
    for case in range(40):
        batch = int(rng.choice([1, 1, 1, 2, 5, 24]))
        m = int(rng.choice([32, 96, 128, 200, 256, 520, 1024, 1536, 2048, 3000]))
        n = 4 * int(rng.integers(16, 800))
        k = 4 * int(rng.integers(8, 1100))
        if batch * m * n * k > 3 * 10 ** 10:
            continue
        shape_a = (batch, m, k) if batch > 1 else (m, k)
        shape_b = (batch, k, n) if batch > 1 else (k, n)
        a = torch.empty(shape_a, dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
        b = torch.empty(shape_b, dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
        bias = torch.empty((n,), dtype=torch.float32, device=d).uniform_(-1, 1, generator=g)
        got = _sgemm_raw(pkg, a, b, bias, "auto", workspace=True)
        again = _sgemm_raw(pkg, a, b, bias, "auto", workspace=True)
        assert torch.equal(got, again), (case, batch, m, n, k)
        rows = rng.choice(m, size=min(m, 6), replace=False)
        bi = int(rng.integers(0, batch))
        a0 = (a[bi] if batch > 1 else a).cpu().numpy()
        b0 = (b[bi] if batch > 1 else b).cpu().numpy()
        truth = a0[rows].astype(np.float64) @ b0.astype(np.float64) + \
            bias.cpu().numpy().astype(np.float64)
        sel = (got[bi] if batch > 1 else got)[torch.from_numpy(rows).to(d)].cpu().numpy()
        assert orc.normwise_rel_error(sel, truth) < TOL_FP32, (case, batch, m, n, k)


def _encoder_stack_f64(x, weights):
    """Config 4 in float64 numpy: 4-layer BERT-base-shaped post-LN encoder with the reference's
    formulas (softmax with max subtraction, erf GELU, two-pass layer norm, gamma 1, beta 0,
    eps 1e-5)."""
    from scipy.special import erf
    b, s, h = x.shape
    heads, dh = 12, 64

    def ln(t):
        mu = t.mean(-1, keepdims=True)
        var = ((t - mu) ** 2).mean(-1, keepdims=True)
        return (t - mu) / np.sqrt(var + 1e-5)

    split = lambda t: t.reshape(b, s, heads, dh).transpose(0, 2, 1, 3)
    for (wq, bq, wk, bk, wv, bv, wo, bo, w1, b1, w2, b2) in weights:
        q, k, v = split(x @ wq + bq), split(x @ wk + bk), split(x @ wv + bv)
        sc = (q @ k.transpose(0, 1, 3, 2)) / 8.0
        e = np.exp(sc - sc.max(-1, keepdims=True))
        p = e / e.sum(-1, keepdims=True)
        o = (p @ v).transpose(0, 2, 1, 3).reshape(b, s, h)
        x = ln(x + (o @ wo + bo))
        f = x @ w1 + b1
        f = 0.5 * f * (1.0 + erf(f / np.sqrt(2.0)))
        x = ln(x + (f @ w2 + b2))
    return x


def encoder_stack_device(pkg, x, weights, gamma, beta):
    """The same stack with every operator from this library: 6 dense matmuls with fused bias
    (the FFN's first one with fused GELU), two batched attention matmuls, fused scale+softmax,
    fused residual+layer norm, head split / merge permutations and K transposed."""
    mm, nn = pkg.blas.matmul, pkg.nn
    b, s, h = x.shape
    heads, dh = 12, 64
    split = lambda t: nn.permute_0213(t.view(b, s, heads, dh))
    for (wq, bq, wk, bk, wv, bv, wo, bo, w1, b1, w2, b2) in weights:
        q, k, v = split(mm(x, wq, bq)), split(mm(x, wk, bk)), split(mm(x, wv, bv))
        p = nn.softmax(mm(q, nn.transpose_last2(k)), scale=0.125)
        o = nn.permute_0213(mm(p, v)).view(b, s, h)
        x = nn.layer_norm(mm(o, wo, bo), gamma, beta, 1e-5, residual=x)
        f = mm(x, w1, b1, activation="gelu")
        x = nn.layer_norm(mm(f, w2, b2), gamma, beta, 1e-5, residual=x)
    return x


def encoder_stack_device_fused(pkg, x, weights, gamma, beta):
    """The same stack with the Q/K/V projections as one launch on a packed weight and the whole
    attention (head split, Q.K^T, scale, softmax, .V, head merge) as one kernel: 8 or 9 launches
    per layer instead of 17."""
    mm, nn = pkg.blas.matmul, pkg.nn
    heads, w = 12, 768
    packed = [nn.pack_qkv(*l[:6]) + tuple(l[6:]) for l in weights]  # once, at constant load
    for (wqkv, bqkv, wo, bo, w1, b1, w2, b2) in packed:
        qkv = mm(x, wqkv, bqkv)
        o = nn.attention(qkv[:, :, :w], qkv[:, :, w:2 * w], qkv[:, :, 2 * w:], heads, scale=0.125)
        x = nn.layer_norm(mm(o, wo, bo), gamma, beta, 1e-5, residual=x)
        f = mm(x, w1, b1, activation="gelu")
        x = nn.layer_norm(mm(f, w2, b2), gamma, beta, 1e-5, residual=x)
    return x


def make_encoder_weights(rng):
    shapes = [(768, 768)] * 4 + [(768, 3072), (3072, 768)]
    weights = []
    for _ in range(4):
        layer = []
        for (k, n) in shapes:
            layer += [rng.normal(0, 0.02, (k, n)).astype(np.float32), np.zeros(n, np.float32)]
        weights.append(layer)
    return weights


@pytest.mark.parametrize("fused", [False, True])
def test_config4_encoder_stack_on_device(pkg, orc, fused):
    """Config 4: 4-layer BERT-base-shaped encoder, batch 8, sequence 128, every operator from
    this library, against the same stack in float64; operator by operator, and with the packed
    Q/K/V projection and the one-kernel attention."""
    d = dev_of()
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (8, 128, 768)).astype(np.float32)
    weights = make_encoder_weights(rng)
    truth = _encoder_stack_f64(x.astype(np.float64), [[w.astype(np.float64) for w in l] for l in weights])
    tw = [[torch.from_numpy(w).to(d) for w in l] for l in weights]
    gamma, beta = torch.ones(768, device=d), torch.zeros(768, device=d)
    run_stack = encoder_stack_device_fused if fused else encoder_stack_device
    got = run_stack(pkg, torch.from_numpy(x).to(d), tw, gamma, beta)
    pkg.session.get_session(d).sync()
    got = got.cpu().numpy()
    assert orc.normwise_rel_error(got, truth) < 1e-5
    assert orc.is_similar(got, truth.astype(np.float32))
