"""Benchmark of the TFCC matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]

Headline workload (one "step"): the fp32 GEMM A[8192,8192] . B[8192,8192] through
``blas.matmul`` (3xTF32 on tcgen05 tensor cores).  With N > 1 ranks B is column-sharded,
every rank multiplies its shard and one NCCL all-gather plus a local interleave leaves the
full row-major C on every rank (strong scaling: the job is the same GEMM at every N).

One JSON line is printed by rank 0.  ``value`` is TFLOP/s (2*M*N*K per step) with operands
resident in HBM; ``e2e`` is the same metric through the host-buffer C-ABI call, uploads
and download inside the timed region; ``roofline`` describes the tcgen05 kernel;
``cpu_baseline`` is the CPU oracle (numpy sgemm, all host threads) timed on a bounded
row panel of the same GEMM; ``extra`` holds the other configurations of the path
(attention-shaped batches, int8, M<=8 streaming) measured with an L2 flush between
launches.  ``--impl reference`` times only the CPU implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
from __graft_entry__ import load_oracle, load_package  # noqa: E402

M = N = K = 8192   # --size overrides this for profiler captures; the headline is 8192
FLOP_PER_STEP = 2.0 * M * N * K

# dram__bytes_read.sum + dram__bytes_write.sum of one umma_gemm_kernel launch on the 8192^3
# problem, from the ncu capture summarised in profiles/umma_gemm_tf32x3_pair_8192_traffic.md
# (2,288,931,584 B read + 256,376,832 B written).  Only valid for the single-GPU headline size.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2536176640


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs: one
    `nvidia-smi -lms 100` child process whose lines are collected by a reader thread."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._proc = None
        self._thread = None

    def _read(self):
        for line in self._proc.stdout:
            parts = [x.strip() for x in line.strip().split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
            time.sleep(0.35)  # let the first samples arrive before the region starts
            self.samples.clear()
        except Exception:
            self._proc = None
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            time.sleep(0.12)
            self._proc.terminate()  # this exact child, by handle
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
            self._thread.join(timeout=5)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = max((int(s[1]) for s in self.samples if s[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------- CPU arm
def blas_threads() -> int:
    """Threads numpy's BLAS really uses (falls back to the visible core count)."""
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 0) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_sgemm_panel(seconds_target: float = 12.0):
    """The oracle's fp32 GEMM (numpy sgemm, every host thread) on a bounded sample of the
    8192^3 problem: a row panel sized for about `seconds_target` of CPU work, or the whole
    GEMM repeated when one pass is shorter than that.  Returns (TFLOP/s, threads, text)."""
    orc = load_oracle()
    rng = np.random.default_rng(4)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    rows = 64
    a = rng.uniform(-1, 1, (rows, K)).astype(np.float32)
    orc.blas_matmul(a, b, dtype=np.float32)  # warm the BLAS threads
    t0 = time.perf_counter()
    orc.blas_matmul(a, b, dtype=np.float32)
    dt = time.perf_counter() - t0
    rate = 2.0 * rows * N * K / dt
    rows = int(min(M, max(64, (seconds_target * rate) / (2.0 * N * K) // 64 * 64)))
    a = rng.uniform(-1, 1, (rows, K)).astype(np.float32)
    orc.blas_matmul(a, b, dtype=np.float32)
    reps, t0 = 0, time.perf_counter()
    while True:
        orc.blas_matmul(a, b, dtype=np.float32)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_target * 0.8 or reps >= 50:
            break
    return (2.0 * rows * N * K * reps / dt / 1e12, blas_threads(),
            f"rows 0..{rows} of the {M}^3 GEMM x {reps} passes ({dt:.2f} s)")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    sample = ""
    cores = 1
    for i in range(args.warmup + args.steps):
        v, cores, sample = cpu_sgemm_panel(seconds_target=max(0.5, 60.0 / (args.warmup + args.steps)))
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": f"fp32 matmul TFLOP/s ({M}^3)", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": FLOP_PER_STEP / (value * 1e12) * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg5-large: fp32 A[{M},{K}] x B[{K},{N}], U(-1,1), seed 4",
                   "note": "CPU arm: oneDNN v1.8.1 (the reference's fp32 backend) is not in the "
                           "reference tree and cannot be built; the oracle's numpy sgemm stands in"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def flush_l2(torch, scratch):
    scratch.add_(1)  # read+write a buffer larger than L2


def time_launches(torch, fn, iters, flush=None):
    """Average device time of `fn` over `iters` launches, each bracketed by events, with an
    optional L2 flush before every launch (not timed)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(iters)]
    for a, b in evs:
        if flush is not None:
            flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return float(np.mean(ts)), float(ts[len(ts) // 2])


def time_graph_train(torch, calls, replays=5):
    """Device time per launch of a train of calls captured in one CUDA graph.

    `calls` is a list of zero-argument functions, each launching one operator on its own
    operands; together the operand sets exceed twice the L2 size, so no launch finds its
    inputs cached by the previous one.  Replaying the graph removes host launch cost, which
    is how a latency-bound operator sequence is deployed.  Returns (mean us per call, best)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for c in calls:   # warm-up outside capture (lazy module load, allocator growth)
            c()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for c in calls:
                c()
        graph.replay()
        stream.synchronize()
        ts = []
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / len(calls))
    torch.cuda.current_stream().wait_stream(stream)
    return float(np.mean(ts)), float(min(ts))


def profile_case(torch, pkg, dev, name):
    """Launch one configuration's kernel a few times and return: the small, self-ending
    workload that `ncu -k <kernel> -c 1` captures (`--profile-case NAME`)."""
    rng = np.random.default_rng(5)
    to = lambda x: torch.from_numpy(x).to(dev)
    sess = pkg.session.get_session(dev)
    if name.startswith("gemv_M"):
        m = int(name[len("gemv_M"):])
        w = to(rng.normal(0, 0.02, (4096, 16384)).astype(np.float32))
        x = to(rng.normal(0, 1, (m, 4096)).astype(np.float32))
        fn = lambda: pkg.blas.matmul(x, w)
    elif name.startswith("int8_M"):
        m = int(name[len("int8_M"):])
        qa = to(rng.integers(0, 256, (m, 4096), dtype=np.uint8))
        qb = to(rng.integers(-127, 128, (4096, 4096), dtype=np.int8))
        ra, rb = pkg.quantization.reduce_sum(qa, True), pkg.quantization.reduce_sum(qb, False)
        f = lambda v: torch.tensor([v], dtype=torch.float32)
        fn = lambda: pkg.quantization.matmul(qa, ra, f(-128.0), f(127.0), qb, rb, f(-128.0), f(127.0))
    elif name == "attention_qk":
        q = to(rng.normal(0, 1, (96, 128, 64)).astype(np.float32))
        kt = to(rng.normal(0, 1, (96, 64, 128)).astype(np.float32))
        fn = lambda: pkg.blas.matmul(q, kt)
    elif name == "ffn1":
        x = to(rng.normal(0, 1, (8, 128, 768)).astype(np.float32))
        w = to(rng.normal(0, 0.02, (768, 3072)).astype(np.float32))
        b = to(np.zeros(3072, np.float32))
        fn = lambda: pkg.blas.matmul(x, w, b)
    elif name == "encoder_stack":
        shapes4 = [(768, 768)] * 4 + [(768, 3072), (3072, 768)]
        w4 = [[t for (k, n) in shapes4 for t in (to(rng.normal(0, 0.02, (k, n)).astype(np.float32)),
                                                 torch.zeros(n, device=dev))] for _ in range(4)]
        x4 = to(rng.normal(0, 1, (8, 128, 768)).astype(np.float32))
        g4, b4 = torch.ones(768, device=dev), torch.zeros(768, device=dev)
        mm, nnops = pkg.blas.matmul, pkg.nn

        def fn():
            x = x4
            split = lambda t: nnops.permute_0213(t.view(8, 128, 12, 64))
            for (wq, bq, wk, bk, wv, bv, wo, bo, w1, b1, w2, b2) in w4:
                q, k, v = split(mm(x, wq, bq)), split(mm(x, wk, bk)), split(mm(x, wv, bv))
                p = nnops.softmax(mm(q, nnops.transpose_last2(k)), scale=0.125)
                o = nnops.permute_0213(mm(p, v)).view(8, 128, 768)
                x = nnops.layer_norm(mm(o, wo, bo), g4, b4, 1e-5, residual=x)
                x = nnops.layer_norm(mm(mm(x, w1, b1, activation="gelu"), w2, b2), g4, b4, 1e-5,
                                     residual=x)
            return x
    else:
        raise SystemExit(f"unknown --profile-case {name}")
    for _ in range(5):
        fn()
    sess.sync()
    print(json.dumps({"profile_case": name, "launches": pkg.launch_count()}))


def extra_measurements(torch, pkg, dev, peaks):
    """Other configurations of the path, single GPU, L2 flushed between launches."""
    lib = pkg.lib
    sess = pkg.session.get_session(dev)
    rng = np.random.default_rng(5)
    scratch = torch.zeros(96 * 1024 * 1024, dtype=torch.float32, device=dev)  # 384 MB > L2
    fl = lambda: flush_l2(torch, scratch)
    out = {}
    to = lambda x: torch.from_numpy(x).to(dev)

    l2_bytes = 126 * 1024 * 1024

    def sgemm_case(name, a, b, bias=None, iters=30, precision="fp32"):
        """Two timings of one configuration: `us` = one launch after an L2 flush, CUDA events
        around that launch (includes the launch gap an isolated call pays); `train_us` = mean
        per launch of a CUDA-graph train over rotating operand sets larger than 2x L2."""
        ta, tb = to(a), to(b)
        tbias = to(bias) if bias is not None else None
        fn = lambda: pkg.blas.matmul(ta, tb, tbias, precision=precision)
        for _ in range(3):
            fn()
        mean_ms, med_ms = time_launches(torch, fn, iters, fl)
        m, k, n = a.shape[-2], a.shape[-1], b.shape[-1]
        batch = max(int(np.prod(a.shape[:-2])), int(np.prod(b.shape[:-2])), 1)
        flop = 2.0 * m * n * k * batch
        nbytes = 4.0 * (a.size + b.size + batch * m * n)
        sets = max(2, int(2 * l2_bytes // nbytes) + 1)
        ops = [(ta.clone(), tb.clone()) for _ in range(sets)]
        calls = [(lambda x=x, y=y: pkg.blas.matmul(x, y, tbias, precision=precision))
                 for x, y in ops]
        calls = calls * max(1, 16 // len(calls))
        train_us, _ = time_graph_train(torch, calls)
        out[name] = {"us": med_ms * 1e3, "train_us": train_us, "operand_sets": sets,
                     "tflops": flop / (train_us * 1e-6) / 1e12,
                     "gbs": nbytes / (train_us * 1e-6) / 1e9,
                     "hbm_frac": nbytes / (train_us * 1e-6) / 1e9 / peaks["hbm_gbs"]}
        del ops, calls

    # cfg1
    sgemm_case("cfg1_32x512x2048", rng.uniform(-1, 1, (32, 512)).astype(np.float32),
               rng.normal(0, 0.02, (512, 2048)).astype(np.float32))
    # cfg2: attention-shaped batches
    q = rng.normal(0, 1, (96, 128, 64)).astype(np.float32)
    kt = rng.normal(0, 1, (96, 64, 128)).astype(np.float32)
    pm = rng.uniform(0, 1, (96, 128, 128)).astype(np.float32)
    v = rng.normal(0, 1, (96, 128, 64)).astype(np.float32)
    sgemm_case("cfg2_qk_96x128x64x128", q, kt)
    sgemm_case("cfg2_pv_96x128x128x64", pm, v)
    # cfg4-shaped dense layers (batch folded into rows)
    x = rng.normal(0, 1, (8, 128, 768)).astype(np.float32)
    sgemm_case("cfg4_ffn1_1024x768x3072", x, rng.normal(0, 0.02, (768, 3072)).astype(np.float32),
               bias=np.zeros(3072, np.float32))
    # cfg4: the whole 4-layer encoder stack on this library's operators, and its matmuls alone
    d_model, heads, dh, b4, s4 = 768, 12, 64, 8, 128
    shapes4 = [(768, 768)] * 4 + [(768, 3072), (3072, 768)]
    w4 = [[t for (k, n) in shapes4 for t in (to(rng.normal(0, 0.02, (k, n)).astype(np.float32)),
                                             torch.zeros(n, device=dev))] for _ in range(4)]
    x4 = to(rng.normal(0, 1, (b4, s4, d_model)).astype(np.float32))
    gamma4, beta4 = torch.ones(d_model, device=dev), torch.zeros(d_model, device=dev)
    mm, nnops = pkg.blas.matmul, pkg.nn

    def stack(x):
        split = lambda t: nnops.permute_0213(t.view(b4, s4, heads, dh))
        for (wq, bq, wk, bk, wv, bv, wo, bo, w1, b1, w2, b2) in w4:
            q, k, v = split(mm(x, wq, bq)), split(mm(x, wk, bk)), split(mm(x, wv, bv))
            p = nnops.softmax(mm(q, nnops.transpose_last2(k)), scale=0.125)
            o = nnops.permute_0213(mm(p, v)).view(b4, s4, d_model)
            x = nnops.layer_norm(mm(o, wo, bo), gamma4, beta4, 1e-5, residual=x)
            x = nnops.layer_norm(mm(mm(x, w1, b1, activation="gelu"), w2, b2), gamma4, beta4, 1e-5,
                                 residual=x)
        return x

    q4 = to(rng.normal(0, 1, (b4, heads, s4, dh)).astype(np.float32))
    k4 = to(rng.normal(0, 1, (b4, heads, dh, s4)).astype(np.float32))
    p4 = to(rng.uniform(0, 1, (b4, heads, s4, s4)).astype(np.float32))
    f4 = to(rng.normal(0, 1, (b4, s4, 3072)).astype(np.float32))

    def matmuls_only():
        for (wq, bq, wk, bk, wv, bv, wo, bo, w1, b1, w2, b2) in w4:
            mm(x4, wq, bq); mm(x4, wk, bk); mm(x4, wv, bv)
            mm(q4, k4); mm(p4, q4)
            mm(x4, wo, bo); mm(x4, w1, b1); mm(f4, w2, b2)

    launches_before = pkg.launch_count()
    stack(x4)
    stack_launches = pkg.launch_count() - launches_before
    stack_us, _ = time_graph_train(torch, [lambda: stack(x4)])
    mm_us, _ = time_graph_train(torch, [matmuls_only])
    flop4 = 4 * 14898167808.0
    out["cfg4_encoder_stack"] = {"ms": stack_us / 1e3, "matmul_only_ms": mm_us / 1e3,
                                 "kernels_per_forward": stack_launches,
                                 "matmul_tflops": flop4 / (mm_us * 1e-6) / 1e12}
    del w4
    # cfg5 skinny sweep
    w = rng.normal(0, 0.02, (4096, 16384)).astype(np.float32)
    for m in (1, 4, 8):
        sgemm_case(f"cfg5_gemv_M{m}", rng.normal(0, 1, (m, 4096)).astype(np.float32), w, iters=40)
    del w
    # TF32 single pass on the headline shape (what one MMA per product reaches)
    a8 = torch.empty((M, K), dtype=torch.float32, device=dev).uniform_(-1, 1)
    b8 = torch.empty((K, N), dtype=torch.float32, device=dev).uniform_(-1, 1)
    fn = lambda: pkg.blas.matmul(a8, b8, precision="tf32")
    for _ in range(2):
        fn()
    _, med = time_launches(torch, fn, 5)
    out["tf32_single_pass_8192"] = {"us": med * 1e3, "tflops": FLOP_PER_STEP / (med * 1e-3) / 1e12}
    # opt-in bfloat16 mode: two rounding pre-passes + the bf16 tensor-core kernel, all timed
    fn = lambda: pkg.blas.matmul(a8, b8, precision="bf16")
    for _ in range(2):
        fn()
    _, med = time_launches(torch, fn, 5)
    out["bf16_mode_8192"] = {"us": med * 1e3, "tflops": FLOP_PER_STEP / (med * 1e-3) / 1e12,
                             "frac_of_bf16_peak": FLOP_PER_STEP / (med * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    del a8, b8

    # cfg3 int8 (M=256) and the compute-bound int8 point (M=4096)
    for m in (256, 4096):
        nbytes = m * 4096 + 4096 * 4096 + 4 * m * 4096 + 4 * m + 4 * 4096
        sets = max(2, int(2 * l2_bytes // nbytes) + 1)
        ops = []
        for _ in range(sets):
            qa = to(rng.integers(0, 256, (m, 4096), dtype=np.uint8))
            qb = to(rng.integers(-127, 128, (4096, 4096), dtype=np.int8))
            ops.append((qa, qb, pkg.quantization.reduce_sum(qa, True),
                        pkg.quantization.reduce_sum(qb, False),
                        torch.empty((m, 4096), dtype=torch.int32, device=dev)))

        def make(qa, qb, ra, rb, c):
            def fn():
                st = lib.tfccb200_qgemm_u8s8s32(
                    torch.cuda.current_stream().cuda_stream, qa.data_ptr(), 0, ra.data_ptr(), 0,
                    -128, qb.data_ptr(), 0, rb.data_ptr(), 0, 0, c.data_ptr(), m * 4096, m, 4096,
                    4096, 1, sess.status_ptr)
                assert st == 0, st
            return fn
        calls = [make(*o) for o in ops]
        for c in calls[:2]:
            c()
        _, med = time_launches(torch, calls[0], 30, fl)
        train_us, _ = time_graph_train(torch, calls * max(1, 16 // len(calls)))
        ops_count = 2.0 * m * 4096 * 4096
        out[f"cfg3_int8_M{m}"] = {"us": med * 1e3, "train_us": train_us, "operand_sets": sets,
                                  "tops": ops_count / (train_us * 1e-6) / 1e12,
                                  "gbs": nbytes / (train_us * 1e-6) / 1e9,
                                  "hbm_frac": nbytes / (train_us * 1e-6) / 1e9 / peaks["hbm_gbs"]}
        if m == 256:
            qa, qb = ops[0][0], ops[0][1]
            f1 = lambda: pkg.quantization.reduce_sum(qa, True)
            f2 = lambda: pkg.quantization.reduce_sum(qb, False)
            for f, nm, nb in ((f1, "reduce_sum_rows_256x4096", m * 4096),
                              (f2, "reduce_sum_cols_4096x4096", 4096 * 4096)):
                for _ in range(3):
                    f()
                _, med = time_launches(torch, f, 20, fl)
                out[nm] = {"us": med * 1e3, "gbs": nb / (med * 1e-3) / 1e9}
        del ops, calls
    # int8 at the headline size: u8[8192,8192] x s8[8192,8192] -> s32 (13.8 waves of pair tiles)
    n8 = 8192
    ops = []
    for _ in range(2):
        qa = torch.randint(0, 256, (n8, n8), dtype=torch.uint8, device=dev)
        qb = torch.randint(-127, 128, (n8, n8), dtype=torch.int8, device=dev)
        ops.append((qa, qb, pkg.quantization.reduce_sum(qa, True),
                    pkg.quantization.reduce_sum(qb, False),
                    torch.empty((n8, n8), dtype=torch.int32, device=dev)))

    def make8(qa, qb, ra, rb, c):
        def fn():
            st = lib.tfccb200_qgemm_u8s8s32(
                torch.cuda.current_stream().cuda_stream, qa.data_ptr(), 0, ra.data_ptr(), 0, -128,
                qb.data_ptr(), 0, rb.data_ptr(), 0, 0, c.data_ptr(), n8 * n8, n8, n8, n8, 1,
                sess.status_ptr)
            assert st == 0, st
        return fn
    calls = [make8(*o) for o in ops]
    for c in calls:
        c()
    train_us, _ = time_graph_train(torch, calls * 3)
    out["int8_8192"] = {"train_us": train_us, "tops": 2.0 * n8 ** 3 / (train_us * 1e-6) / 1e12,
                        "frac_of_nominal_dense_int8": 2.0 * n8 ** 3 / (train_us * 1e-6) / 4.5e15}
    del ops, calls
    sess.sync()
    return out


def multi_gpu_extras(torch, dist, pkg, dev, world, rank, peaks):
    """The other shard-natural cases at N GPUs.  Every rank times its own share with CUDA events
    (mean of a train after warm-up); the job's figure uses the slowest rank.
    * config 2 split by batch: 96 attention batches / N per rank, no communication;
    * int8 u8[4096,4096] x s8[4096,4096] -> s32 split by columns of B: every rank keeps its
      column shard of C (the layout a following row-split layer consumes), and, separately,
      with an NCCL all-gather of the shards plus the panel interleave to the row-major C."""
    lib = pkg.lib
    sess = pkg.session.get_session(dev)
    out = {}

    def slowest(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def timed(fn, iters=20, warm=3):
        for _ in range(warm):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return slowest(e0.elapsed_time(e1) / iters)

    # ---- config 2, batch split
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    lo, hi = pkg.parallel.shard_range(96, world, rank)
    sets = 8  # rotate operand sets so that the train does not sit in L2 for free
    qs = [torch.randn((hi - lo, 128, 64), device=dev, generator=g) for _ in range(sets)]
    kts = [torch.randn((hi - lo, 64, 128), device=dev, generator=g) for _ in range(sets)]
    calls = [(lambda q=q, kt=kt: pkg.blas.matmul(q, kt)) for q, kt in zip(qs, kts)]
    dist.barrier()
    us, _ = time_graph_train(torch, calls * 2)  # graph replay: no host launch cost per step
    ms = slowest(us * 1e-3)
    out["cfg2_qk_batch_split"] = {"us_per_step": ms * 1e3, "batches_per_rank": hi - lo,
                                  "tflops_whole_job": 2.0 * 96 * 128 * 64 * 128 / (ms * 1e-3) / 1e12}
    del calls
    del qs, kts

    # ---- int8, column shards of B
    m = n = k = 4096
    ns = n // world
    rng = np.random.default_rng(7)  # same A on every rank
    qa = torch.from_numpy(rng.integers(0, 256, (m, k), dtype=np.uint8)).to(dev)
    qb_full = rng.integers(-127, 128, (k, n), dtype=np.int8)
    qb = torch.from_numpy(np.ascontiguousarray(qb_full[:, rank * ns:(rank + 1) * ns])).to(dev)
    ra = pkg.quantization.reduce_sum(qa, True)
    rb = pkg.quantization.reduce_sum(qb, False)
    c_shard = torch.empty((m, ns), dtype=torch.int32, device=dev)
    staging = torch.empty((world, m, ns), dtype=torch.int32, device=dev)
    c_full = torch.empty((m, n), dtype=torch.int32, device=dev)

    def local():
        st = lib.tfccb200_qgemm_u8s8s32(
            torch.cuda.current_stream().cuda_stream, qa.data_ptr(), 0, ra.data_ptr(), 0, -128,
            qb.data_ptr(), 0, rb.data_ptr(), 0, 0, c_shard.data_ptr(), m * ns, m, ns, k, 1,
            sess.status_ptr)
        assert st == 0, st

    def gathered():
        local()
        dist.all_gather_into_tensor(staging, c_shard)
        # bit copy of 32-bit words: the panel interleave does not care that they are integers
        pkg.parallel.interleave_panels(staging.view(torch.float32), c_full.view(torch.float32))

    ops = 2.0 * m * n * k
    ms = timed(local, iters=40)
    out["int8_4096_column_shards"] = {"us_per_step": ms * 1e3, "tops_whole_job": ops / (ms * 1e-3) / 1e12}
    ms = timed(gathered, iters=20)
    out["int8_4096_column_shards_gathered"] = {"us_per_step": ms * 1e3,
                                               "tops_whole_job": ops / (ms * 1e-3) / 1e12,
                                               "gathered_bytes_per_rank": 4 * m * (n - ns)}
    # exactness of the assembled matrix against the int64 product, on sampled rows
    gathered()
    torch.cuda.synchronize()
    rows = np.random.default_rng(0).choice(m, size=4, replace=False)
    a64 = qa[torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.int64) - 128
    truth = (a64 @ qb_full.astype(np.int64)).astype(np.int32)
    got = c_full[torch.from_numpy(rows).to(dev)].cpu().numpy()
    out["int8_4096_column_shards_gathered"]["sampled_rows_exact"] = bool(np.array_equal(got, truth))
    sess.sync()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    pkg = load_package()
    peaks = measured_peaks()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if args.profile_case:
        profile_case(torch, pkg, dev, args.profile_case)
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert N % world == 0
    ns = N // world

    # ---- synthetic operands (seed 4, U(-1,1)); every rank holds A and its column shard of B
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    a = torch.empty((M, K), dtype=torch.float32, device=dev).uniform_(-1, 1, generator=g)
    b_full = torch.empty((K, N), dtype=torch.float32, device=dev).uniform_(-1, 1, generator=g)
    b = b_full[:, rank * ns:(rank + 1) * ns].contiguous() if world > 1 else b_full
    if world > 1:
        del b_full
    staging = c_out = fused = None
    mode = "single GPU"
    if world > 1:
        if args.gather == "fused":
            try:
                fused = pkg.parallel.FusedNSplit(M, N, dev)
                mode = (f"N-split x{world}: B column shards; C tiles pushed to every rank from the "
                        f"GEMM epilogue over NVLink ({fused.how}) + barrier")
            except Exception as exc:  # peer mapping unavailable: NCCL gather of our local product
                print(f"[bench] fused N-split unavailable ({exc!r}); using NCCL all-gather",
                      file=sys.stderr)
                fused = None
        ok = torch.tensor([1.0 if fused is not None else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            fused = None
        if fused is None:
            staging = torch.empty((world, M, ns), dtype=torch.float32, device=dev)
            c_out = torch.empty((M, N), dtype=torch.float32, device=dev)
            mode = f"N-split x{world}: B column shards, NCCL all-gather of C + interleave kernel"
    sess = pkg.session.get_session(dev)

    def step():
        if world == 1:
            return pkg.blas.matmul(a, b)
        if fused is not None:
            return fused.matmul(a, b)
        return pkg.parallel.nsplit_matmul(a, b, staging=staging, out=c_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if world > 1 and args.check:
        # the assembled C must equal the product computed locally against the matching
        # shard of B, bit for bit (N-split does not touch the K order)
        full = step()
        barrier()
        bad = 0
        for r in range(world):
            g2 = torch.Generator(device=dev)
            g2.manual_seed(4)
            torch.empty((M, K), dtype=torch.float32, device=dev).uniform_(-1, 1, generator=g2)
            bf = torch.empty((K, N), dtype=torch.float32, device=dev).uniform_(-1, 1, generator=g2)
            ref = pkg.blas.matmul(a, bf[:, r * ns:(r + 1) * ns].contiguous())
            bad += int((ref != full[:, r * ns:(r + 1) * ns]).sum().item())
            del bf, ref
        print(f"[bench] rank {rank}: N-split check, mismatching elements = {bad}", file=sys.stderr)
        barrier()
    sampler = ClockSampler(local_rank)
    launches0 = pkg.launch_count()
    with sampler:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    launches = pkg.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    sess.sync()

    # device time of the GEMM launch alone for the roofline: at one GPU that is the step
    # itself; with shards, a train of local products between two events
    if world == 1:
        kern_mean_ms = ms_total / args.steps
    else:
        reps = max(3, min(args.steps, 20))
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(reps):
            pkg.blas.matmul(a, b)
        k1.record()
        torch.cuda.synchronize()
        kern_mean_ms = k0.elapsed_time(k1) / reps

    # ---- end to end: host buffers in, host buffer out, through the C-ABI host entry point
    e2e_steps = max(1, min(args.steps, 3))
    ha = torch.empty((M, K), dtype=torch.float32).pin_memory()
    hb = torch.empty((K, ns), dtype=torch.float32).pin_memory()
    hc = torch.empty((M, ns), dtype=torch.float32).pin_memory()
    ha.copy_(a.cpu())
    hb.copy_(b.cpu())
    h_full = torch.empty((M, N), dtype=torch.float32).pin_memory() if world > 1 else None

    def e2e_step():
        if world == 1:
            st = pkg.lib.tfccb200_sgemm_host(sess.stream_ptr, ha.data_ptr(), 0, hb.data_ptr(), 0,
                                             hc.data_ptr(), M * ns, None, M, ns, K, 1, 0)
            assert st == 0, st
        else:
            da = ha.to(dev, non_blocking=True)
            db = hb.to(dev, non_blocking=True)
            if fused is not None:
                full = fused.matmul(da, db)
            else:
                full = pkg.parallel.nsplit_matmul(da, db, staging=staging, out=c_out)
            h_full.copy_(full, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    h2d = 4 * (M * K + K * ns)
    d2h = 4 * (M * N if world > 1 else M * ns)

    # ---- max over ranks
    t = torch.tensor([ms_total, e2e_s * 1e3, float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms_total, e2e_ms, launches = float(tmax[0]), float(tmax[1]), int(tsum[2])
    else:
        e2e_ms = float(t[1])

    if rank == 0:
        ms_per_step = ms_total / args.steps
        value = FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
        e2e_value = FLOP_PER_STEP / (e2e_ms / e2e_steps * 1e-3) / 1e12
        kern_flop = FLOP_PER_STEP / world
        achieved = kern_flop / (kern_mean_ms * 1e-3) / 1e12
        # a kernel timed alone is judged against the burst figure, one timed inside a long
        # region (power-capped clocks) against the sustained one
        sustained = ms_total >= 250.0 and peaks.get("bf16_tflops_sustained")
        bf16_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        tensor_peak = bf16_peak / 2.0 / 3.0
        line = {
            "metric": f"fp32 matmul TFLOP/s ({M}^3)", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (3xTF32 tensor-core products, fp32 accumulation)",
            "data": "synthetic",
            "config": {
                "workload": f"cfg5-large: fp32 A[{M},{K}] x B[{K},{N}], U(-1,1), seed 4",
                "parallelism": mode,
                "l2": f"operands ({4 * M * K >> 20} MiB each) exceed the 126 MB L2; no flush between steps",
                "timing": "CUDA events on the launching stream, max over ranks"},
            "roofline": {
                "bound": "tensor", "kernel": "umma_gemm_kernel<TF32, split, cta_group::2, BN=256>",
                "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": achieved / tensor_peak,
                "peak_basis": f"of {peaks['source']}: bf16 {'sustained' if sustained else 'burst'} "
                              f"{bf16_peak} TFLOP/s / 2 (TF32 runs at half the bf16 rate) / 3 "
                              "(MMAs per fp32 product)",
                "frac_of_burst_peak": achieved / (peaks["bf16_tflops"] / 6.0),
                "executed_tf32_tflops": 3.0 * achieved,
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (world == 1 and M == 8192) else None,
                "algorithmic_bytes": 4 * (M * K + K * ns + M * ns)},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": sampler.summary(),
        }
        if world == 1:
            if not args.no_cpu:
                v, cores, sample = cpu_sgemm_panel()
                line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores,
                                        "kind": "port", "sample": sample}
            if not args.no_extra:
                line["extra"] = extra_measurements(torch, pkg, dev, peaks)
    if world > 1 and not args.no_extra:
        extra = multi_gpu_extras(torch, dist, pkg, dev, world, rank, peaks)
        if rank == 0:
            line["extra"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the secondary configurations (headline line only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--gather", choices=["fused", "nccl"], default="fused",
                    help="N > 1: push C tiles to peers from the GEMM epilogue, or NCCL all-gather")
    ap.add_argument("--profile-case", default="",
                    help="run only one small configuration (gemv_M1, int8_M256, int8_M4096, "
                         "attention_qk, ffn1) a few times and exit: the target of ncu captures")
    ap.add_argument("--check", action="store_true",
                    help="N > 1: verify the assembled C against the single-GPU product")
    ap.add_argument("--size", type=int, default=8192,
                    help="edge of the square GEMM (profiler captures use a smaller one)")
    args = ap.parse_args()
    global M, N, K, FLOP_PER_STEP
    M = N = K = args.size
    FLOP_PER_STEP = 2.0 * M * N * K
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
