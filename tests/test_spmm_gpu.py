"""GPU parity of dlspm_spmm_csr_f32 (and its planned / strict variants) against the CPU oracle."""
import numpy as np
import pytest

from cases import csr_bernoulli, csr_from_lengths, csr_rowlen_normal, dense, shuffle_rows_columns, spmm_case
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=False, guard=64):
    """Runs the kernel into a NaN-prefilled, guard-banded output and returns C."""
    import torch

    nnz = int(ci.size)
    buf = torch.full((M * N + 2 * guard,), float("nan"), device=dev)
    Cd = buf[guard:guard + M * N]
    d_ro, d_ci, d_v, d_B = to_dev(ro, dev), to_dev(ci, dev), to_dev(vals, dev), to_dev(B, dev)
    if plan:
        p = ctx.plan_create(M, K, nnz, d_ro, d_ci)
        ctx.spmm_planned(p, N, d_v, d_ro, d_ci, d_B, Cd)
        torch.cuda.synchronize()
        p.close()
    else:
        ctx.spmm(M, K, N, nnz, d_v, d_ro, d_ci, d_B, Cd)
        torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert np.isnan(host[:guard]).all() and np.isnan(host[guard + M * N:]).all(), "wrote outside C"
    return host[guard:guard + M * N].reshape(M, N)


def check(oracle, ro, ci, vals, B, M, N, out):
    big = float(ci.size) * N > 2e8  # large cases: the same loop with its rows spread over the host threads
    threads = oracle.max_threads() if big else 1
    ref = oracle.spmm(vals, ro, ci, B, M, N, threads=threads)
    scale = oracle.spmm_scale(vals, ro, ci, B, M, N, threads=threads)
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, scale, TOL)
    assert bad == 0, f"{bad} elements beyond tolerance, worst ratio {worst:.3e}"


def test_config1_512x512_n128(pkg, oracle, ctx, dev):
    M, K, N = 512, 512, 128
    ro, ci, vals, B = spmm_case(pkg, M, K, N, 0.1, seed=1)
    check(oracle, ro, ci, vals, B, M, N, run_spmm(ctx, dev, M, K, N, ro, ci, vals, B))


@pytest.mark.parametrize("N", [1, 2, 3, 4, 6, 16, 17, 49, 64, 100, 128, 130, 196, 256, 260, 384, 512, 784, 1024, 1028, 3136])
def test_dense_widths(pkg, oracle, ctx, dev, N):
    M, K = 67, 96
    ro, ci, vals, B = spmm_case(pkg, M, K, N, 0.15, seed=100 + N)
    check(oracle, ro, ci, vals, B, M, N, run_spmm(ctx, dev, M, K, N, ro, ci, vals, B))


SWEEP_SHAPES = [(64, 64), (256, 256), (512, 2048), (2048, 512), (1024, 4096)]
SWEEP_SPARSITIES = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]
SWEEP_WIDTHS = [256, 1024, 3136]


def sweep_case(pkg, M, K, N, sparsity):
    seed = M * 7 + int(sparsity * 100) + N
    ro, ci = csr_rowlen_normal(pkg, M, K, sparsity, seed)
    vals = pkg.gen_dense_host(int(ci.size), seed, 2)
    B = dense(pkg, K, N, seed, 10)
    return ro, ci, vals, B


@pytest.mark.parametrize("N", SWEEP_WIDTHS)
@pytest.mark.parametrize("shape", SWEEP_SHAPES)
@pytest.mark.parametrize("sparsity", SWEEP_SPARSITIES)
def test_sweep_shapes(pkg, oracle, ctx, dev, shape, sparsity, N):
    """All 90 cases of the sweep configuration (5 shapes x 6 sparsities x 3 widths) at full size, as
    lone launches."""
    M, K = shape
    ro, ci, vals, B = sweep_case(pkg, M, K, N, sparsity)
    check(oracle, ro, ci, vals, B, M, N, run_spmm(ctx, dev, M, K, N, ro, ci, vals, B))


@pytest.mark.parametrize("kernel", [0, 2])
def test_sweep_shapes_one_prepared_batch(pkg, oracle, ctx, dev, kernel):
    """The same 90 cases at full size as ONE prepared grouped launch (the form the benchmark times):
    automatic kernel choice, and the tiled kernel wherever it applies."""
    import torch

    cases = [(M, K, N, sp) for (M, K) in SWEEP_SHAPES for sp in SWEEP_SPARSITIES for N in SWEEP_WIDTHS]
    arr = pkg.ProblemArray(len(cases))
    keep, outs = [], []
    for i, (M, K, N, sp) in enumerate(cases):
        ro, ci, vals, B = sweep_case(pkg, M, K, N, sp)
        d = (to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev))
        Cd = torch.full((M * N,), float("nan"), device=dev)
        arr.set(i, M, K, N, int(ci.size), *d, Cd)
        keep.append((ro, ci, vals, B, d))
        outs.append(Cd)
    ctx.set_option(pkg.OPT_SPMM_KERNEL, kernel)
    try:
        batch = ctx.batch_create(arr)
        batch.launch()
        torch.cuda.synchronize()
        assert batch.info(check_device=True)[2] == 0, "a bounded wait ran out"
        batch.close()
    finally:
        ctx.set_option(pkg.OPT_SPMM_KERNEL, 0)
    for (M, K, N, sp), (ro, ci, vals, B, _d), Cd in zip(cases, keep, outs):
        check(oracle, ro, ci, vals, B, M, N, Cd.cpu().numpy().reshape(M, N))


@pytest.mark.parametrize("N", [4, 8, 12, 16, 20, 32, 36, 48, 64])
def test_narrow_dense_operand_many_rows(pkg, oracle, ctx, dev, N):
    """Enough rows for the several-rows-per-warp kernel (N <= 64): 4, 8 and 16 lanes per row, widths
    that do not fill the lane group, empty rows and rows longer than one fetch round."""
    M, K = 40000, 96
    seed = 600 + N
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.8, seed, cov=0.8)
    assert (np.diff(ro) == 0).any() and np.diff(ro).max() > 32
    vals = pkg.gen_dense_host(int(ci.size), seed, 2)
    B = dense(pkg, K, N, seed, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    check(oracle, ro, ci, vals, B, M, N, out)
    planned = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=True)
    assert np.array_equal(out.view(np.uint32), planned.view(np.uint32))
    if N in (16, 32, 64):
        ctx.set_option(pkg.OPT_STRICT_FP32, 1)
        try:
            strict = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
        finally:
            ctx.set_option(pkg.OPT_STRICT_FP32, 0)
        assert np.array_equal(strict.view(np.uint32), oracle.spmm(vals, ro, ci, B, M, N).view(np.uint32))


@pytest.mark.parametrize("M,N", [(3000, 32), (4096, 28), (6000, 16), (2500, 64), (4500, 8), (3000, 36)])
def test_narrow_dense_operand_lane_groups_share_a_row(pkg, oracle, ctx, dev, M, N):
    """Narrow N with too few rows for a row per lane group: the groups of a warp share the row (its
    pairs dealt to them in turn, partial rows added at the end).  Empty rows, rows shorter than the
    number of groups and rows of several fetch rounds; with and without a plan."""
    K = 400
    seed = 700 + N
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.85, seed, cov=0.9)
    lengths = np.diff(ro)
    assert (lengths == 0).any() and (lengths < 4).any() and lengths.max() > 64
    vals = pkg.gen_dense_host(int(ci.size), seed, 2)
    B = dense(pkg, K, N, seed, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    check(oracle, ro, ci, vals, B, M, N, out)
    planned = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=True)
    assert np.array_equal(out.view(np.uint32), planned.view(np.uint32))
    ctx.set_option(pkg.OPT_STRICT_FP32, 1)  # strict mode keeps the CSR order (another kernel)
    try:
        strict = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    finally:
        ctx.set_option(pkg.OPT_STRICT_FP32, 0)
    assert np.array_equal(strict.view(np.uint32), oracle.spmm(vals, ro, ci, B, M, N).view(np.uint32))


def test_few_long_rows_shared_between_warps(pkg, oracle, ctx, dev):
    """Few rows with many nonzeros: 2, 4 or 8 warps share a row; strict mode keeps one warp per row."""
    for (M, K, N) in [(64, 4096, 256), (300, 2048, 132), (1024, 4096, 260), (9, 3000, 1024)]:
        seed = M + N
        ro, ci = csr_rowlen_normal(pkg, M, K, 0.7, seed)
        vals = pkg.gen_dense_host(int(ci.size), seed, 2)
        B = dense(pkg, K, N, seed, 10)
        out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
        check(oracle, ro, ci, vals, B, M, N, out)
        ctx.set_option(pkg.OPT_STRICT_FP32, 1)
        try:
            strict = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
        finally:
            ctx.set_option(pkg.OPT_STRICT_FP32, 0)
        assert np.array_equal(strict.view(np.uint32), oracle.spmm(vals, ro, ci, B, M, N).view(np.uint32))


def test_row_length_edges(pkg, oracle, ctx, dev):
    # empty rows first/last/in between, lengths around the 32-wide staging chunk, one full row
    K, N = 200, 132
    lengths = [0, 1, 0, 15, 16, 17, 31, 32, 33, 63, 64, 65, 96, 128, 200, 0, 5, 0]
    ro, ci = csr_from_lengths(pkg, K, lengths, seed=5)
    M = len(lengths)
    vals = pkg.gen_dense_host(int(ci.size), 5, 2)
    B = dense(pkg, K, N, 5, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    check(oracle, ro, ci, vals, B, M, N, out)
    for i, n in enumerate(lengths):
        if n == 0:
            assert (out[i] == 0).all(), "empty row must give zeros"


def test_all_rows_empty_and_degenerate_sizes(pkg, oracle, ctx, dev):
    import torch

    M, K, N = 9, 7, 20
    ro = np.zeros(M + 1, dtype=np.int32)
    ci = np.zeros(0, dtype=np.int32)
    vals = np.zeros(0, dtype=np.float32)
    B = dense(pkg, K, N, 1, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    assert (out == 0).all()
    # M = 0 and N = 0 are accepted and write nothing
    ctx.spmm(0, K, N, 0, None, to_dev(np.zeros(1, np.int32), dev), None, to_dev(B, dev), None)
    ctx.spmm(M, K, 0, 0, None, to_dev(ro, dev), None, None, None)
    torch.cuda.synchronize()


def test_single_row_single_column(pkg, oracle, ctx, dev):
    M, K, N = 1, 1, 5
    ro = np.array([0, 1], dtype=np.int32)
    ci = np.array([0], dtype=np.int32)
    vals = np.array([-0.75], dtype=np.float32)
    B = dense(pkg, K, N, 3, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    np.testing.assert_array_equal(out, vals[0] * B)


def test_unsorted_and_duplicate_columns(pkg, oracle, ctx, dev):
    M, K, N = 40, 64, 72
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=9)
    ci = shuffle_rows_columns(ro, ci, seed=9)
    # duplicates: repeat the first column of every non-empty row in its second slot
    for i in range(M):
        if ro[i + 1] - ro[i] >= 2:
            ci[ro[i] + 1] = ci[ro[i]]
    vals = pkg.gen_dense_host(int(ci.size), 9, 2)
    B = dense(pkg, K, N, 9, 10)
    check(oracle, ro, ci, vals, B, M, N, run_spmm(ctx, dev, M, K, N, ro, ci, vals, B))


@pytest.mark.parametrize("N", [128, 100, 33])
def test_strict_mode_is_bit_exact(pkg, oracle, ctx, dev, N):
    """Separate multiply and add in CSR order reproduces the fp32 host loop bit for bit."""
    M, K = 300, 257
    ro, ci, vals, B = spmm_case(pkg, M, K, N, 0.2, seed=21 + N)
    ctx.set_option(pkg.OPT_STRICT_FP32, 1)
    try:
        out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
        out_planned = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=True)
    finally:
        ctx.set_option(pkg.OPT_STRICT_FP32, 0)
    ref = oracle.spmm(vals, ro, ci, B, M, N)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(out_planned.view(np.uint32), ref.view(np.uint32))


def test_planned_equals_unplanned(pkg, oracle, ctx, dev):
    M, K, N = 777, 300, 260
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.8, seed=33)
    vals = pkg.gen_dense_host(int(ci.size), 33, 2)
    B = dense(pkg, K, N, 33, 10)
    a = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
    b = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=True)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    check(oracle, ro, ci, vals, B, M, N, b)


@pytest.mark.parametrize("M", [1, 255, 256, 777, 70001])
def test_plan_row_order_is_fixed_by_the_pattern(pkg, ctx, dev, M):
    """Rows come in bins by length (2^(b-1) <= length < 2^b, empty rows last), longest bin first,
    ascending row numbers inside a bin; nothing about it depends on the run."""
    K = 700
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.9, seed=M, cov=1.2)  # wide spread of lengths, empty rows included
    d_ro, d_ci = to_dev(ro, dev), to_dev(ci, dev)
    lengths = np.diff(ro)
    bins = np.where(lengths <= 0, 0, np.floor(np.log2(np.maximum(lengths, 1))).astype(np.int64) + 1)
    want = np.lexsort((np.arange(M), -bins)).astype(np.int32)  # by bin descending, then by row ascending
    for _ in range(3):
        plan = ctx.plan_create(M, K, int(ci.size), d_ro, d_ci)
        got = plan.row_order()
        plan.close()
        assert np.array_equal(got, want)


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_unaligned_dense_pointers(pkg, oracle, ctx, dev, offset):
    """B and C that do not start on a 16-byte boundary take the narrower vector path."""
    import torch

    M, K, N = 50, 60, 64
    ro, ci, vals, B = spmm_case(pkg, M, K, N, 0.2, seed=44)
    bufB = torch.zeros(K * N + 8, device=dev)
    bufB[offset:offset + K * N] = to_dev(B.ravel(), dev)
    bufC = torch.full((M * N + 8,), float("nan"), device=dev)
    ctx.spmm(M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev),
             bufB[offset:offset + K * N], bufC[offset:offset + M * N])
    torch.cuda.synchronize()
    host = bufC.cpu().numpy()
    assert np.isnan(host[:offset]).all() and np.isnan(host[offset + M * N:]).all()
    check(oracle, ro, ci, vals, B, M, N, host[offset:offset + M * N].reshape(M, N))


def test_invalid_arguments(pkg, ctx, dev):
    ro = to_dev(np.zeros(5, np.int32), dev)
    with pytest.raises(pkg.DlspmError) as e:
        ctx.spmm(-1, 4, 4, 0, None, ro, None, None, None)
    assert e.value.status == pkg.ERR_INVALID_ARGUMENT
    with pytest.raises(pkg.DlspmError):
        ctx.spmm(4, 4, 4, 3, None, ro, None, None, None)  # nnz > 0 without arrays


def test_full_size_row_sum_property(pkg, ctx, dev):
    """65536 x 65536 at 1 % density, N = 512: with B = 1 every element of row i of C equals the sum
    of row i's values (checked against a float64 prefix-sum on the device), and with unit values
    and B[k, :] = k it equals the sum of the row's column indices, which is exact in fp32 here."""
    import torch

    M = K = 65536
    N = 512
    density = 0.01
    counts = torch.zeros(M, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_count(M, K, density, 77, counts)
    ro = torch.zeros(M + 1, dtype=torch.int32, device=dev)
    ro[1:] = torch.cumsum(counts, 0).to(torch.int32)
    nnz = int(ro[-1].item())
    assert abs(nnz - M * K * density) < 0.01 * M * K * density
    ci = torch.empty(nnz, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_fill(M, K, density, 77, ro, ci)
    vals = torch.empty(nnz, device=dev)
    ctx.gen_dense(vals, 77, 2)
    B = torch.ones(K, N, device=dev)
    Cd = torch.full((M, N), float("nan"), device=dev)
    ctx.spmm(M, K, N, nnz, vals, ro, ci, B, Cd)
    torch.cuda.synchronize()
    csum = torch.zeros(nnz + 1, dtype=torch.float64, device=dev)
    csum[1:] = torch.cumsum(vals.double(), 0)
    row_sum = (csum[ro[1:].long()] - csum[ro[:-1].long()])
    abs_sum = torch.zeros(nnz + 1, dtype=torch.float64, device=dev)
    abs_sum[1:] = torch.cumsum(vals.double().abs(), 0)
    scale = (abs_sum[ro[1:].long()] - abs_sum[ro[:-1].long()])
    err = (Cd.double() - row_sum[:, None]).abs().max(dim=1).values
    assert bool((err <= TOL * torch.maximum(row_sum.abs(), scale)).all())
    # all columns of a row are identical
    assert bool((Cd == Cd[:, :1]).all())
    # unit values, B[k, :] = k  ->  sum of column indices (< 2^24 per partial sum is not needed:
    # compare with tolerance)
    vals.fill_(1.0)
    B.copy_(torch.arange(K, device=dev, dtype=torch.float32)[:, None].expand(K, N))
    ctx.spmm(M, K, N, nnz, vals, ro, ci, B, Cd)
    torch.cuda.synchronize()
    isum = torch.zeros(nnz + 1, dtype=torch.float64, device=dev)
    isum[1:] = torch.cumsum(ci.double(), 0)
    want = isum[ro[1:].long()] - isum[ro[:-1].long()]
    assert bool(((Cd[:, 0].double() - want).abs() <= TOL * want.clamp(min=1.0)).all())
    assert bool((Cd == Cd[:, :1]).all())


@pytest.mark.parametrize("K,density", [(40, 0.5), (100, 0.5), (600, 0.5)])
@pytest.mark.parametrize("N", [32, 50, 128, 256, 1024, 3136])
@pytest.mark.parametrize("plan", [False, True])
def test_few_rows_are_shared_between_warps(pkg, oracle, ctx, dev, K, density, N, plan):
    """A lone matrix with few rows runs with 2, 4 or 8 warps per row (about 20, 50 and 300 entries per
    row here), partial slabs combined through shared memory; empty and one-entry rows included, all
    slab widths and the scalar path (N = 50)."""
    M = 40
    ro, ci = csr_bernoulli(pkg, M, K, density, seed=51 + K)
    lengths = np.diff(ro).copy()
    lengths[2], lengths[9] = 0, 1
    keep = np.concatenate([np.arange(ro[i], ro[i] + min(lengths[i], ro[i + 1] - ro[i])) for i in range(M)]).astype(np.int64)
    ci = np.ascontiguousarray(ci[keep])
    ro = np.concatenate([[0], np.cumsum(np.minimum(lengths, np.diff(ro)))]).astype(np.int32)
    vals = pkg.gen_dense_host(int(ci.size), 51, 2)
    B = dense(pkg, K, N, 51, 10)
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=plan)
    check(oracle, ro, ci, vals, B, M, N, out)
    assert (out[2] == 0).all()


def test_strict_mode_keeps_csr_order_with_batched_loads(pkg, oracle, ctx, dev):
    """Strict mode never shares rows, and the narrow slabs' batched loads keep the order of the
    products: bits of the host loop for one-, two- and four-chunk slabs and ragged row lengths."""
    M, K = 70, 300
    ro, ci = csr_from_lengths(pkg, K, [0, 1, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 40, 63, 64, 65, 200, 300] + [11] * 50, seed=61)
    vals = pkg.gen_dense_host(int(ci.size), 61, 2)
    ctx.set_option(pkg.OPT_STRICT_FP32, 1)
    try:
        for N in (128, 100, 256, 1024):
            B = dense(pkg, K, N, 61, 10)
            out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B)
            ref = oracle.spmm(vals, ro, ci, B, M, N)
            assert np.array_equal(out.view(np.uint32), ref.view(np.uint32)), N
    finally:
        ctx.set_option(pkg.OPT_STRICT_FP32, 0)


def test_planned_launch_with_long_uneven_rows(pkg, oracle, ctx, dev):
    """A plan knows the longest row; long rows of uneven length then run with eight warps per row."""
    M, K, N = 96, 4000, 128
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.7, 71)  # mean 1200, spread 40 %
    vals = pkg.gen_dense_host(int(ci.size), 71, 2)
    B = dense(pkg, K, N, 71, 10)
    assert np.diff(ro).max() >= 1.3 * np.diff(ro).mean() >= 1.3 * 800
    out = run_spmm(ctx, dev, M, K, N, ro, ci, vals, B, plan=True)
    check(oracle, ro, ci, vals, B, M, N, out)
