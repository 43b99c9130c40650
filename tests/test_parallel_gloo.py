"""The multi-GPU shim's host logic on two CPU ranks over gloo.

The local product and the panel interleave are injected stand-ins (numpy float64 product,
torch permute) because the package's own operators only run on a GPU; what is under test is
the partitioning, the gather order and the layout of the assembled result.
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load_package
    pkg = load_package()

    def cpu_matmul(a, b, c=None):
        r = torch.from_numpy(a.numpy().astype(np.float64) @ b.numpy().astype(np.float64)).float()
        return r + c if c is not None else r

    def cpu_interleave(staging, out):
        g, m, ns = staging.shape
        out.view(m, g, ns).copy_(staging.permute(1, 0, 2))

    rng = np.random.default_rng(3)
    a = torch.from_numpy(rng.uniform(-1, 1, (24, 40)).astype(np.float32))
    b = torch.from_numpy(rng.uniform(-1, 1, (40, 16 * world)).astype(np.float32))
    bias = torch.from_numpy(rng.uniform(-1, 1, 16 * world).astype(np.float32))
    ns = b.shape[1] // world
    full = pkg.parallel.nsplit_matmul(a, b[:, rank * ns:(rank + 1) * ns].contiguous(),
                                      bias[rank * ns:(rank + 1) * ns].contiguous(),
                                      matmul_fn=cpu_matmul, interleave_fn=cpu_interleave)
    ok_nsplit = torch.allclose(full, cpu_matmul(a, b, bias), atol=1e-5)

    qa = torch.from_numpy(rng.normal(0, 1, (7, 5, 6)).astype(np.float32))
    kb = torch.from_numpy(rng.normal(0, 1, (7, 6, 4)).astype(np.float32))
    part, (s0, s1) = pkg.parallel.batch_split_matmul(qa, kb, matmul_fn=lambda x, y: torch.matmul(x, y))
    ok_batch = torch.allclose(part, torch.matmul(qa, kb)[s0:s1], atol=1e-5)
    shared, (t0, t1) = pkg.parallel.batch_split_matmul(qa, kb[0], matmul_fn=lambda x, y: torch.matmul(x, y))
    ok_shared = torch.allclose(shared, torch.matmul(qa, kb[0])[t0:t1], atol=1e-5)
    results[rank] = (bool(ok_nsplit), bool(ok_batch), bool(ok_shared), (s0, s1))
    dist.destroy_process_group()


def test_nsplit_and_batch_split_on_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        res = dict(results)
    assert set(res) == {0, 1}
    for r in range(world):
        assert res[r][:3] == (True, True, True), res
    assert res[0][3] == (0, 4) and res[1][3] == (4, 7)
