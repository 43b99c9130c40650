"""The in-process device group (tfccb200_group_*): N-split products whose tiles are stored into
every member's C from the GEMM epilogue.  With one GPU the group's two members share it, which
exercises everything except the NVLink hop (column offsets, row pitch, multi-destination
stores, row exchange, per-member row slices of the host path); with two or more GPUs the same
cases run across devices.  Sharded results must equal the unsharded ones bit for bit: the N
split does not touch the order of the K sum.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _members():
    cases = [[0, 0], [0, 0, 0, 0]]
    if torch.cuda.device_count() >= 2:
        cases.append([0, 1])
    if torch.cuda.device_count() >= 4:
        cases.append([0, 1, 2, 3])
    return cases


@pytest.mark.parametrize("k", [132, 516])
@pytest.mark.parametrize("devices", _members())
def test_group_fp32_nsplit_matches_unsharded_product(pkg, orc, devices, k):
    """k = 132 is too short for the planner to share a tile's K range among CTAs, so the sharded
    and the unsharded product sum in the same order and must agree bit for bit (as the large
    products of the benchmark do); with k = 516 the planner may split K differently for the two
    widths, and they are compared with the fp32 tolerance."""
    g = len(devices)
    rng = np.random.default_rng(31)
    m, ns = 384, 264
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, g * ns)).astype(np.float32)
    bias = rng.uniform(-1, 1, g * ns).astype(np.float32)
    grp = pkg.parallel.DeviceGroup(devices)
    dev = [torch.device("cuda", d) for d in devices]
    ta = [torch.from_numpy(a).to(d) for d in dev]
    tb = [torch.from_numpy(np.ascontiguousarray(b[:, i * ns:(i + 1) * ns])).to(dev[i]) for i in range(g)]
    tbias = [torch.from_numpy(np.ascontiguousarray(bias[i * ns:(i + 1) * ns])).to(dev[i]) for i in range(g)]
    tc = [torch.full((m, g * ns), float("nan"), dtype=torch.float32, device=d) for d in dev]
    for d in dev:
        torch.cuda.synchronize(d)
    for _ in range(2):  # a second call reuses streams, events and scratch
        grp.sgemm_nsplit(ta, tb, tc, tbias)
    grp.sync()
    truth = orc.blas_matmul(a, b, bias)
    # the unsharded product through the same entry point (a group of one)
    one = pkg.parallel.DeviceGroup(devices[:1])
    whole = torch.empty((m, g * ns), dtype=torch.float32, device=dev[0])
    one.sgemm_nsplit(ta[:1], [torch.from_numpy(b).to(dev[0])], [whole],
                     [torch.from_numpy(bias).to(dev[0])])
    one.sync()
    one.close()
    for i in range(g):
        got = tc[i].cpu().numpy()
        assert orc.normwise_rel_error(got, truth) < 1e-5
        assert np.array_equal(got, tc[0].cpu().numpy())
    if k == 132:  # the same K order as the unsharded tensor-core product: identical bits
        assert np.array_equal(tc[0].cpu().numpy(), whole.cpu().numpy())
    else:
        assert orc.normwise_rel_error(whole.cpu().numpy(), truth) < 1e-5
    grp.close()


@pytest.mark.parametrize("devices", _members())
def test_group_int8_nsplit_bit_exact(pkg, orc, devices):
    g = len(devices)
    rng = np.random.default_rng(32)
    m, k, ns = 300, 512, 256
    qa = rng.integers(0, 256, (m, k), dtype=np.uint8)
    qb = rng.integers(-127, 128, (k, g * ns), dtype=np.int8)
    rs_a, rs_b = orc.reduce_sum(qa, True), orc.reduce_sum(qb, False)
    off_a, off_b, _, _ = orc.matmul_params(-1.5, 2.0, -0.7, 0.9)
    want, _, _ = orc.quantized_matmul(qa, rs_a, -1.5, 2.0, qb, rs_b, -0.7, 0.9, impl="port")
    grp = pkg.parallel.DeviceGroup(devices)
    dev = [torch.device("cuda", d) for d in devices]
    ta = [torch.from_numpy(qa).to(d) for d in dev]
    tra = [torch.from_numpy(rs_a).to(d) for d in dev]
    tb = [torch.from_numpy(np.ascontiguousarray(qb[:, i * ns:(i + 1) * ns])).to(dev[i]) for i in range(g)]
    trb = [torch.from_numpy(np.ascontiguousarray(rs_b[i * ns:(i + 1) * ns])).to(dev[i]) for i in range(g)]
    tc = [torch.full((m, g * ns), -1, dtype=torch.int32, device=d) for d in dev]
    for d in dev:
        torch.cuda.synchronize(d)
    grp.qgemm_nsplit(ta, tra, off_a, tb, trb, off_b, tc)
    grp.sync()
    for i in range(g):
        assert np.array_equal(tc[i].cpu().numpy(), want)
    grp.close()


@pytest.mark.parametrize("rows", [128, 550, 1536])
@pytest.mark.parametrize("devices", _members())
def test_group_host_buffers_round_trip(pkg, orc, devices, rows):
    """Host buffers in, host buffer out.  ``rows`` per member: one row block (128), two blocks of
    275 (550) and six of 256 (1536) -- with several blocks the uploads, the exchange of A rows,
    the products and the downloads of different blocks overlap on four streams per member."""
    g = len(devices)
    rng = np.random.default_rng(33 + rows)
    m, k, n = rows * g, 260, 136 * g
    ha = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).pin_memory()
    hb = torch.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32)).pin_memory()
    hc = torch.full((m, n), float("nan"), dtype=torch.float32).pin_memory()
    grp = pkg.parallel.DeviceGroup(devices)
    grp.sgemm_nsplit_host(ha, hb, hc)
    truth = orc.blas_matmul(ha.numpy(), hb.numpy())
    assert orc.normwise_rel_error(hc.numpy(), truth) < 1e-5
    # second call on other data reuses the group's staging
    ha.mul_(0.5)
    grp.sgemm_nsplit_host(ha, hb, hc)
    assert orc.normwise_rel_error(hc.numpy(), 0.5 * truth) < 1e-5
    # a shape the split cannot take is refused, nothing is launched
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        grp.sgemm_nsplit_host(ha[: m - 1], hb, hc[: m - 1])
    grp.close()


def test_group_rejects_bad_devices(pkg):
    with pytest.raises(pkg.exceptions.InvalidArgumentError):
        pkg.parallel.DeviceGroup([torch.cuda.device_count() + 3])
