"""Grouped launch, host-buffer entry points, device generators and the multi-device layer."""
import numpy as np
import pytest

from cases import csr_bernoulli, csr_rowlen_normal, dense, spmm_case
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu

SHAPES = [(64, 64), (256, 256), (512, 2048), (2048, 512), (1024, 4096)]
SPARSITIES = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]


def make_problems(pkg, count, seed, widths=(256, 100, 33, 64, 1024, 6)):
    """Small problems drawn like the sweep grid (shapes scaled down), with mixed vector widths."""
    probs = []
    for i in range(count):
        h = pkg.rand_u64(seed, 50, i)
        M, K = SHAPES[h % 5]
        M, K = max(1, M // 8), max(1, K // 8)
        sp = SPARSITIES[(h >> 8) % 6]
        N = widths[(h >> 16) % len(widths)]
        ro, ci = csr_rowlen_normal(pkg, M, K, sp, seed * 1000 + i)
        vals = pkg.gen_dense_host(int(ci.size), seed * 1000 + i, 2)
        B = dense(pkg, K, N, seed * 1000 + i, 10)
        probs.append((M, K, N, ro, ci, vals, B))
    return probs


def check_all(oracle, probs, outs):
    for (M, K, N, ro, ci, vals, B), out in zip(probs, outs):
        ref = oracle.spmm(vals, ro, ci, B, M, N)
        scale = oracle.spmm_scale(vals, ro, ci, B, M, N)
        assert not np.isnan(out).any()
        bad, worst = oracle.violations(ref, out.reshape(M, N), scale, TOL)
        assert bad == 0, worst


@pytest.mark.parametrize("prepared", [False, True])
def test_batched_matches_oracle(pkg, oracle, ctx, dev, prepared):
    import torch

    probs = make_problems(pkg, 40, seed=3)
    # an empty problem and one without nonzeros in the middle of the batch
    probs.insert(5, (0, 8, 16, np.zeros(1, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32),
                     np.zeros((8, 16), np.float32)))
    probs.insert(9, (6, 8, 16, np.zeros(7, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32),
                     dense(pkg, 8, 16, 1, 10)))
    arr = pkg.ProblemArray(len(probs))
    outs = []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        Cd = torch.full((max(M * N, 1),), float("nan"), device=dev)[: M * N]
        outs.append(Cd)
        arr.set(i, M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev), Cd)
    if prepared:
        batch = ctx.batch_create(arr)
        batch.launch()
        batch.launch()  # a prepared batch can be launched repeatedly
        torch.cuda.synchronize()
        batch.close()
    else:
        ctx.spmm_batched(arr)
        torch.cuda.synchronize()
    check_all(oracle, probs, [o.cpu().numpy() for o in outs])


def test_batched_equals_single_launches(pkg, ctx, dev):
    """Same kernel body: the grouped launch gives the bits of one launch per problem."""
    import torch

    probs = make_problems(pkg, 12, seed=4)
    arr = pkg.ProblemArray(len(probs))
    outs, singles = [], []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        d = [to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev)]
        Cd = torch.empty(M * N, device=dev)
        Cs = torch.empty(M * N, device=dev)
        arr.set(i, M, K, N, int(ci.size), d[0], d[1], d[2], d[3], Cd)
        ctx.spmm(M, K, N, int(ci.size), d[0], d[1], d[2], d[3], Cs)
        outs.append(Cd)
        singles.append(Cs)
    ctx.spmm_batched(arr)
    torch.cuda.synchronize()
    for a, b in zip(outs, singles):
        assert torch.equal(a, b)


def test_host_entry_points(pkg, oracle, ctx):
    M, K, N = 300, 200, 96
    ro, ci, vals, B = spmm_case(pkg, M, K, N, 0.1, seed=5)
    out = np.full((M, N), np.nan, dtype=np.float32)
    ctx.spmm_host(M, K, N, int(ci.size), vals, ro, ci, B, out)
    bad, worst = oracle.violations(oracle.spmm(vals, ro, ci, B, M, N), out, oracle.spmm_scale(vals, ro, ci, B, M, N), TOL)
    assert bad == 0, worst

    lhs = dense(pkg, M, N, 5, 11)
    rhs = dense(pkg, K, N, 5, 12)
    s = np.full(ci.size, np.nan, dtype=np.float32)
    ctx.sddmm_host(M, K, N, int(ci.size), ro, ci, lhs, rhs, s)
    bad, worst = oracle.violations(oracle.sddmm(ro, ci, lhs, rhs, M, N), s, oracle.sddmm_scale(ro, ci, lhs, rhs, M, N), TOL)
    assert bad == 0, worst

    v = dense(pkg, K, N, 5, 13)
    e = np.full((M, N), np.nan, dtype=np.float32)
    ctx.fused_host(M, K, N, int(ci.size), ro, ci, lhs, rhs, v, e)
    ref, _ = oracle.fused(ro, ci, lhs, rhs, v, M, N)
    bad, worst = oracle.violations(ref, e, oracle.fused_scale(ro, ci, lhs, rhs, v, M, N), TOL)
    assert bad == 0, worst


def test_batched_host_with_pinned_memory(pkg, oracle, ctx):
    import torch

    probs = make_problems(pkg, 10, seed=6)
    arr = pkg.ProblemArray(len(probs))
    outs = []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        out = torch.full((M * N,), float("nan")).pin_memory()
        outs.append(out)
        arr.set(i, M, K, N, int(ci.size), torch.from_numpy(vals).pin_memory(), ro, ci,
                torch.from_numpy(B).pin_memory(), out, host=True)
    ctx.spmm_batched_host(arr)
    check_all(oracle, probs, [o.numpy() for o in outs])


def test_device_generators_match_host(pkg, ctx, dev):
    import torch

    # dense values: bit-identical for the two uniform kinds, close for the normal kind
    n = 100003
    for kind in (pkg.KIND_UNIFORM_PM1, pkg.KIND_UNIFORM_01):
        d = torch.empty(n, device=dev)
        ctx.gen_dense(d, 11, 7, first_index=5, kind=kind)
        h = pkg.gen_dense_host(n, 11, 7, first_index=5, kind=kind)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), h.view(np.uint32))
    d = torch.empty(n, device=dev)
    ctx.gen_dense(d, 11, 7, kind=pkg.KIND_NORMAL)
    np.testing.assert_allclose(d.cpu().numpy(), pkg.gen_dense_host(n, 11, 7, kind=pkg.KIND_NORMAL), rtol=1e-5, atol=1e-6)

    # sampled columns: same set, same order; includes empty rows, full rows and a row wider than
    # the shared-memory key cache
    for (M, K, sp) in [(64, 64, 0.9), (200, 333, 0.5), (50, 4096, 0.98), (3, 9000, 0.7)]:
        ro = pkg.gen_rowlen_normal_host(M, K, sp, 0.4, 13)
        ro = ro.copy()
        if M >= 3:  # force an empty and a full row
            lens = np.diff(ro)
            lens[0], lens[1] = 0, K
            ro[1:] = np.cumsum(lens)
        want = pkg.gen_sample_columns_host(M, K, ro, 13)
        got = torch.full((int(ro[-1]),), -1, dtype=torch.int32, device=dev)
        ctx.gen_sample_columns(M, K, to_dev(ro, dev), 13, got)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), want)

    # Bernoulli pattern in two steps
    M, K, density = 300, 1000, 0.07
    ro_h, ci_h = pkg.gen_bernoulli_csr_host(M, K, density, 17)
    counts = torch.zeros(M, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_count(M, K, density, 17, counts)
    assert np.array_equal(counts.cpu().numpy(), np.diff(ro_h))
    ci = torch.full((int(ro_h[-1]),), -1, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_fill(M, K, density, 17, to_dev(ro_h, dev), ci)
    assert np.array_equal(ci.cpu().numpy(), ci_h)


def test_plan_on_generated_pattern(pkg, oracle, ctx, dev):
    """Plan row order is a permutation: planned SpMM covers every row exactly once."""
    import torch

    M, K, N = 1000, 512, 64
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.95, seed=19)
    vals = pkg.gen_dense_host(int(ci.size), 19, 2)
    B = dense(pkg, K, N, 19, 10)
    Cd = torch.full((M, N), float("nan"), device=dev)
    d_ro, d_ci = to_dev(ro, dev), to_dev(ci, dev)
    plan = ctx.plan_create(M, K, int(ci.size), d_ro, d_ci)
    ctx.spmm_planned(plan, N, to_dev(vals, dev), d_ro, d_ci, to_dev(B, dev), Cd)
    torch.cuda.synchronize()
    out = Cd.cpu().numpy()
    assert not np.isnan(out).any()
    bad, worst = oracle.violations(oracle.spmm(vals, ro, ci, B, M, N), out, oracle.spmm_scale(vals, ro, ci, B, M, N), TOL)
    assert bad == 0, worst


def test_multi_device_layer(pkg, oracle):
    """dlspm_mg_* with every visible device (two contexts on device 0 when only one is visible)."""
    import torch

    n = torch.cuda.device_count()
    devices = list(range(n)) if n >= 2 else [0, 0]
    mg = pkg.MultiGpu(devices)
    assert mg.device_count() == len(devices)
    probs = make_problems(pkg, 17, seed=8)
    arr = pkg.ProblemArray(len(probs))
    outs = []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        out = np.full(M * N, np.nan, dtype=np.float32)
        outs.append(out)
        arr.set(i, M, K, N, int(ci.size), vals, ro, ci, B, out, host=True)
    mg.spmm_batched_host(arr)
    check_all(oracle, probs, outs)

    M, K, N = 3000, 700, 72
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.9, seed=23)
    vals = pkg.gen_dense_host(int(ci.size), 23, 2)
    B = dense(pkg, K, N, 23, 10)
    out = np.full((M, N), np.nan, dtype=np.float32)
    mg.spmm_rowshard_host(M, K, N, int(ci.size), vals, ro, ci, B, out)
    assert not np.isnan(out).any()
    bad, worst = oracle.violations(oracle.spmm(vals, ro, ci, B, M, N), out, oracle.spmm_scale(vals, ro, ci, B, M, N), TOL)
    assert bad == 0, worst
    mg.close()


def test_fp32_peak_probe(ctx):
    t = ctx.measure_fp32_peak()
    assert 10.0 < t < 200.0, t
