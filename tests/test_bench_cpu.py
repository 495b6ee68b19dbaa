"""CPU-side pieces of bench.py: the batch description, the bounded CPU sample and the extra CPU
baseline figures (no GPU, no timing claims: only that they run and describe the same work)."""
import importlib.util
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_batch_descriptors_are_seeded(pkg, bench):
    a = bench.batch_descriptors(pkg, 24, 5)
    b = bench.batch_descriptors(pkg, 24, 5)
    c = bench.batch_descriptors(pkg, 24, 6)
    assert len(a) == 24
    for x, y in zip(a, b):
        assert x[:5] == y[:5] and np.array_equal(x[5], y[5])
    assert any(x[:5] != z[:5] or not np.array_equal(x[5], z[5]) for x, z in zip(a, c))
    shapes = {(M, K) for (M, K, N, sp, seed, ro) in a}
    assert shapes <= {(64, 64), (256, 256), (512, 2048), (2048, 512), (1024, 4096)}
    assert {N for (M, K, N, sp, seed, ro) in a} <= {256, 1024, 3136}


def test_cpu_sample_is_bounded_and_checked_work(pkg, oracle, bench):
    descs = bench.batch_descriptors(pkg, 32, 1)
    data, flops = bench.cpu_sample(pkg, descs, 3e8)
    assert 1 <= len(data) <= 32
    assert flops == sum(2.0 * ci.size * N for (M, K, N, ro, ci, vals, B) in data)
    assert flops <= 3e8 or len(data) == 1
    dt = bench.time_cpu(oracle, data, 2)
    extra = bench.cpu_variants(oracle, data, flops, dt, 2)
    assert extra["single_thread"]["value"] > 0
    assert extra["loops_interchanged"]["value"] > 0
    assert "value" in extra["o3_march_native"]
    # no oneMKL in this image: the row says so instead of inventing a number
    if extra["onemkl"]["value"] is None:
        assert "unavailable on this box" in extra["onemkl"]["why"] or "failed" in extra["onemkl"]["why"]


def test_interchanged_loop_has_the_same_bits(pkg, oracle):
    M, K, N = 50, 40, 36
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.3, 3)
    vals = pkg.gen_dense_host(int(ci.size), 3, 2)
    B = pkg.gen_dense_host(K * N, 3, 10).reshape(K, N)
    a = oracle.spmm(vals, ro, ci, B, M, N)
    b = oracle.spmm(vals, ro, ci, B, M, N, threads=3, fast_order=True)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_profile_summaries_keep_the_profiler_rules():
    """Every ncu command quoted under profiles/ leaves the GPU clocks alone and names one kernel."""
    import glob
    import os
    import re

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "profiles")
    files = sorted(glob.glob(os.path.join(root, "*.md")))
    assert files, "no profile summaries"
    for path in files:
        for line in open(path):
            if re.match(r"\s+ncu\s", line):
                assert "--clock-control none" in line, f"{os.path.basename(path)}: {line.strip()}"
                assert "--set full" not in line or " -k " in line, f"{os.path.basename(path)}: a full capture of every kernel"
