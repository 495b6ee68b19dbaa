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
    """The grouped launch against one launch per problem.  Same kernel body, so the bits are equal
    unless the single launch shared long rows between warps (few-row matrices), which only changes
    the order of the partial sums."""
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
    equal = 0
    for a, b in zip(outs, singles):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-4)
        equal += int(torch.equal(a, b))
    assert equal >= len(outs) // 2


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


def test_batched_host_sends_one_pinned_arena_with_few_copies(pkg, oracle, ctx):
    """Inputs kept in one pinned arena in the staging order and spacing (and outputs in another) go
    as one copy per piece and direction; the same batch from separate arrays goes array by array;
    both give the oracle's result."""
    import torch

    probs = make_problems(pkg, 30, seed=11, widths=(256, 100, 64, 1024))

    def pad(nbytes):
        return (nbytes + 255) // 256 * 256

    in_bytes = sum(pad(4 * (M + 1)) + 2 * pad(4 * ci.size) + pad(4 * K * N) for (M, K, N, ro, ci, vals, B) in probs)
    out_bytes = sum(pad(4 * M * N) for (M, K, N, *_r) in probs)
    arena_in = torch.zeros(in_bytes, dtype=torch.uint8).pin_memory()
    arena_out = torch.zeros(out_bytes, dtype=torch.uint8).pin_memory()
    in_np, out_np = arena_in.numpy(), arena_out.numpy()
    arr = pkg.ProblemArray(len(probs))
    off, ooff, views = 0, 0, []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        ptrs = []
        for a in (ro.astype(np.int32), ci.astype(np.int32), vals.astype(np.float32), B.astype(np.float32).ravel()):
            in_np[off:off + a.nbytes] = a.view(np.uint8)
            ptrs.append(arena_in.data_ptr() + off)
            off += pad(a.nbytes)
        nnz = int(ci.size)
        arr.set_raw(i, M, K, N, nnz, ptrs[2] if nnz else None, ptrs[0], ptrs[1] if nnz else None, ptrs[3],
                    arena_out.data_ptr() + ooff)
        views.append((ooff, M * N))
        ooff += pad(4 * M * N)
    c0 = ctx.host_copy_count()
    ctx.spmm_batched_host(arr)
    assert ctx.host_copy_count() - c0 == 2, "one pinned arena per direction should be one copy each"
    outs = [out_np[o:o + 4 * n].view(np.float32).copy() for (o, n) in views]
    check_all(oracle, probs, outs)
    # separate (pageable) arrays: copied one by one, same bits
    arr2 = pkg.ProblemArray(len(probs))
    outs2 = []
    for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
        o = np.full(M * N, np.nan, dtype=np.float32)
        outs2.append(o)
        arr2.set(i, M, K, N, int(ci.size), vals, ro, ci, np.ascontiguousarray(B).ravel(), o, host=True)
    c0 = ctx.host_copy_count()
    ctx.spmm_batched_host(arr2)
    assert ctx.host_copy_count() - c0 > len(probs)
    for a, b in zip(outs, outs2):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


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


def _run_prepared(pkg, ctx, dev, probs, kernel, min_density=None):
    import torch

    ctx.set_option(pkg.OPT_SPMM_KERNEL, kernel)
    if min_density is not None:
        ctx.set_option(pkg.OPT_TILE_MIN_DENSITY, min_density)
    try:
        arr = pkg.ProblemArray(len(probs))
        outs = []
        for i, (M, K, N, ro, ci, vals, B) in enumerate(probs):
            Cd = torch.full((max(M * N, 1),), float("nan"), device=dev)[: M * N]
            outs.append(Cd)
            arr.set(i, M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev), Cd)
        batch = ctx.batch_create(arr)
        batch.launch()
        batch.launch()
        torch.cuda.synchronize()
        info = batch.info(check_device=True)
        batch.close()
    finally:
        ctx.set_option(pkg.OPT_SPMM_KERNEL, pkg.SPMM_KERNEL_AUTO)
        ctx.set_option(pkg.OPT_TILE_MIN_DENSITY, -1)  # back to the default
    return [o.cpu().numpy() for o in outs], info


def tiled_cases(pkg):
    """Shapes that exercise every edge of the 128 x 128 x 32 tiling."""
    from cases import csr_from_lengths

    cases = []
    for (M, K, N, sp, seed) in [(128, 64, 128, 0.5, 1), (256, 256, 256, 0.5, 2), (130, 70, 132, 0.3, 3),
                                (1, 33, 4, 0.5, 4), (64, 4096, 260, 0.7, 5), (300, 31, 1024, 0.2, 6),
                                (512, 2048, 256, 0.5, 7), (257, 100, 3136, 0.6, 8)]:
        ro, ci = csr_rowlen_normal(pkg, M, K, sp, 500 + seed)
        cases.append((M, K, N, ro, ci, pkg.gen_dense_host(int(ci.size), 500 + seed, 2), dense(pkg, K, N, 500 + seed, 10)))
    # empty rows, full rows, rows of exactly 32 and 33 entries
    K, N = 96, 64
    lengths = [0, 96, 32, 33, 1, 0, 95, 64, 0]
    ro, ci = csr_from_lengths(pkg, K, lengths, seed=9)
    cases.append((len(lengths), K, N, ro, ci, pkg.gen_dense_host(int(ci.size), 9, 2), dense(pkg, K, N, 9, 10)))
    return cases


def test_tiled_kernel_matches_gather_and_oracle(pkg, oracle, ctx, dev):
    probs = tiled_cases(pkg)
    tiled, info_t = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_TILED)
    gather, info_g = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_GATHER)
    assert info_t[1] == len(probs) and info_t[0] == 0 and info_t[2] == 0
    assert info_g[0] == len(probs) and info_g[1] == 0
    check_all(oracle, probs, tiled)
    check_all(oracle, probs, gather)
    # absent entries add fma(0, b, acc) = acc: the tiled kernel has the bits of the row-gather kernel
    for a, b in zip(tiled, gather):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # the variant that multiplies absent entries as zeros: same bits on finite data
    dense, info_d = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_TILED_DENSE)
    assert info_d[1] == len(probs) and info_d[2] == 0
    for a, b in zip(dense, gather):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_zero_filled_tiles_do_not_see_stale_rows(pkg, oracle, ctx, dev):
    """A block of the zero-filled variant that first stages a B full of infinities and then a tile
    whose K ends inside a 32-row chunk must not multiply the leftovers of the first one."""
    import torch

    Mh, Kh, N = 64, 64, 256
    roh, cih = csr_rowlen_normal(pkg, Mh, Kh, 0.5, 901)
    hot = [to_dev(a, dev) for a in (pkg.gen_dense_host(int(cih.size), 901, 2), roh, cih)]
    hotB = torch.full((Kh * N,), float("inf"), device=dev)
    Mc, Kc = 64, 33
    roc, cic = csr_rowlen_normal(pkg, Mc, Kc, 0.5, 902)
    valsc, Bc = pkg.gen_dense_host(int(cic.size), 902, 2), dense(pkg, Kc, N, 902, 10)
    cold = [to_dev(a, dev) for a in (valsc, roc, cic, Bc)]
    count = 1200  # several tiles per resident block
    ctx.set_option(pkg.OPT_SPMM_KERNEL, pkg.SPMM_KERNEL_TILED_DENSE)
    try:
        arr = pkg.ProblemArray(count)
        outs = torch.full((count, Mc * N), float("nan"), device=dev)
        for i in range(count):
            if i % 2 == 0:
                arr.set(i, Mh, Kh, N, int(cih.size), hot[0], hot[1], hot[2], hotB, outs[i])
            else:
                arr.set(i, Mc, Kc, N, int(cic.size), cold[0], cold[1], cold[2], cold[3], outs[i])
        batch = ctx.batch_create(arr)
        batch.launch()
        torch.cuda.synchronize()
        info = batch.info(check_device=True)
        batch.close()
    finally:
        ctx.set_option(pkg.OPT_SPMM_KERNEL, pkg.SPMM_KERNEL_AUTO)
    assert info[1] == count and info[2] == 0
    got = outs[1::2].cpu().numpy()
    ref = oracle.spmm(valsc, roc, cic, Bc, Mc, N)
    scale = oracle.spmm_scale(valsc, roc, cic, Bc, Mc, N)
    assert np.isfinite(got).all()
    for row in (0, got.shape[0] // 2, got.shape[0] - 1):
        bad, worst = oracle.violations(ref, got[row].reshape(Mc, N), scale, TOL)
        assert bad == 0, worst
    assert (got == got[0]).all()


def test_non_finite_rows_of_b_reach_only_the_rows_that_reference_them(pkg, oracle, ctx, dev):
    """The zero-filled tiled kernel multiplies absent entries as zeros, and 0 * inf is NaN: chunks of
    B that hold a non-finite value must therefore run under the presence masks.  One row of B that
    no row of A references is all infinities, another that some rows reference holds a NaN and an
    infinity: the result has the bits of the row-gather kernel, and rows that reference neither stay
    finite, as in the reference host loop."""
    M, K, N = 300, 200, 512
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.5, 4242)
    unused, used = 77, 130
    keep = ci != unused                      # drop column 77 from every row
    lengths = np.add.reduceat(keep.astype(np.int64), ro[:-1]) * (np.diff(ro) > 0)
    ci = ci[keep]
    ro = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    vals = pkg.gen_dense_host(int(ci.size), 4242, 2)
    B = dense(pkg, K, N, 4242, 10).copy()
    B[unused, :] = np.inf
    B[used, 5] = np.nan
    B[used, 300] = -np.inf
    probs = [(M, K, N, ro, ci, vals, B)]
    gather, _ = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_GATHER)
    for choice in (pkg.SPMM_KERNEL_TILED_DENSE, pkg.SPMM_KERNEL_TILED):
        tiled, info = _run_prepared(pkg, ctx, dev, probs, choice)
        assert info[1] == 1 and info[2] == 0
        assert np.array_equal(tiled[0].view(np.uint32), gather[0].view(np.uint32))
    out = gather[0].reshape(M, N)
    refs_used = np.array([used in ci[ro[i]:ro[i + 1]] for i in range(M)])
    assert refs_used.any() and not refs_used.all()
    assert np.isfinite(out[~refs_used]).all()
    assert np.isnan(out[refs_used][:, 5]).all() and np.isinf(out[refs_used][:, 300]).all()
    fin = np.ones(N, dtype=bool)
    fin[[5, 300]] = False
    assert np.isfinite(out[:, fin]).all()


def test_tiled_kernel_strict_mode_is_bit_exact(pkg, oracle, ctx, dev):
    probs = tiled_cases(pkg)[:4]
    ctx.set_option(pkg.OPT_STRICT_FP32, 1)
    try:
        tiled, info = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_TILED)
    finally:
        ctx.set_option(pkg.OPT_STRICT_FP32, 0)
    assert info[1] == len(probs)
    for (M, K, N, ro, ci, vals, B), out in zip(probs, tiled):
        ref = oracle.spmm(vals, ro, ci, B, M, N)
        assert np.array_equal(out.view(np.uint32), ref.ravel().view(np.uint32))


def test_automatic_choice_and_ineligible_problems(pkg, oracle, ctx, dev):
    """Unsorted rows, N % 4 != 0 and sparse patterns stay on the row-gather kernel; dense sorted
    patterns go to the tiled kernel; results are right either way."""
    from cases import shuffle_rows_columns

    dense_sorted = tiled_cases(pkg)[1]                       # 256 x 256, half full
    M, K, N, ro, ci, vals, B = tiled_cases(pkg)[6]
    unsorted = (M, K, N, ro, shuffle_rows_columns(ro, ci, 3), vals, B)
    ro2, ci2 = csr_rowlen_normal(pkg, 256, 256, 0.5, 77)
    odd_n = (256, 256, 130, ro2, ci2, pkg.gen_dense_host(int(ci2.size), 77, 2), dense(pkg, 256, 130, 77, 10))
    ro3, ci3 = csr_rowlen_normal(pkg, 512, 512, 0.98, 78)
    sparse = (512, 512, 256, ro3, ci3, pkg.gen_dense_host(int(ci3.size), 78, 2), dense(pkg, 512, 256, 78, 10))
    probs = [dense_sorted, unsorted, odd_n, sparse]
    outs, info = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_AUTO, min_density=150)
    assert info[0] == 3 and info[1] == 1 and info[2] == 0
    check_all(oracle, probs, outs)
    # forcing the tiled kernel still leaves the ineligible ones where they are
    outs, info = _run_prepared(pkg, ctx, dev, probs, pkg.SPMM_KERNEL_TILED)
    assert info[0] == 2 and info[1] == 2
    check_all(oracle, probs, outs)


def test_bounded_wait_reports_timeout_and_context_survives(pkg, oracle, ctx, dev):
    """A wait that nothing satisfies ends in a status, not in a hang; kernels run normally afterwards."""
    import torch

    st, timed_out = ctx.selftest_bounded_wait(2000)
    assert st == pkg.ERR_TIMEOUT and timed_out == 1
    assert "bounded wait" in pkg.strerror(st)
    M, K, N, ro, ci, vals, B = 64, 64, 32, *spmm_case(pkg, 64, 64, 32, 0.2, seed=3)
    Cd = torch.empty(M, N, device=dev)
    ctx.spmm(M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev), Cd)
    torch.cuda.synchronize()
    bad, worst = oracle.violations(oracle.spmm(vals, ro, ci, B, M, N), Cd.cpu().numpy(),
                                   oracle.spmm_scale(vals, ro, ci, B, M, N), TOL)
    assert bad == 0, worst


def test_device_side_csr_check(pkg, ctx, dev):
    """dlspm_sanity_check_csr validates CSR arrays that live on the device with the host check's rules
    and texts: a valid pattern passes; a column beyond K, a negative column, decreasing offsets, a
    wrong last offset and a wrong first offset are each reported."""
    M, K = 300, 200
    ro, ci = csr_bernoulli(pkg, M, K, 0.1, 77)
    nnz = int(ci.size)
    assert ctx.sanity_check_csr(M, K, nnz, to_dev(ro, dev), to_dev(ci, dev)) == (pkg.OK, "")
    empty = np.zeros(M + 1, dtype=np.int32)
    assert ctx.sanity_check_csr(M, K, 0, to_dev(empty, dev), None)[0] == pkg.OK
    bad = ci.copy(); bad[nnz // 2] = K
    st, why = ctx.sanity_check_csr(M, K, nnz, to_dev(ro, dev), to_dev(bad, dev))
    assert st == pkg.ERR_CSR and "a_column_indices[i] >= KSZ" in why and f"i = {nnz // 2}" in why
    bad = ci.copy(); bad[3] = -1
    assert ctx.sanity_check_csr(M, K, nnz, to_dev(ro, dev), to_dev(bad, dev))[0] == pkg.ERR_CSR
    bad = ro.copy(); bad[10], bad[11] = bad[11], bad[10] - 1
    st, why = ctx.sanity_check_csr(M, K, nnz, to_dev(bad, dev), to_dev(ci, dev))
    assert st == pkg.ERR_CSR and "a_row_offsets" in why
    bad = ro.copy(); bad[-1] += 1
    st, why = ctx.sanity_check_csr(M, K, nnz, to_dev(bad, dev), to_dev(ci, dev))
    assert st == pkg.ERR_CSR and why == "a_row_offsets[MSZ] != nnz."
    bad = ro.copy(); bad[0] = 1
    st, why = ctx.sanity_check_csr(M, K, nnz, to_dev(bad, dev), to_dev(ci, dev))
    assert st == pkg.ERR_CSR and "a_row_offsets[0] != 0" in why
    assert ctx.sanity_check_csr(2, 2, 5, to_dev(np.array([0, 2, 5], np.int32), dev), to_dev(np.zeros(5, np.int32), dev))[1] == "nnz is larger than matrix."


def test_check_input_option_rejects_bad_patterns_before_any_launch(pkg, oracle, ctx, dev):
    """DLSPM_OPT_CHECK_INPUT: with the option on, every entry point that takes a CSR pattern validates
    it first and returns DLSPM_ERR_CSR (reason in the error text) instead of launching a kernel that
    would read outside B; outputs stay untouched.  A valid pattern runs as usual.  Off by default."""
    import torch

    assert ctx.get_option(pkg.OPT_CHECK_INPUT) == 0
    M, K, N = 200, 150, 64
    ro, ci = csr_bernoulli(pkg, M, K, 0.1, 78)
    nnz = int(ci.size)
    bad = ci.copy()
    bad[nnz // 3] = K + 5  # would read beyond the last row of B
    vals = pkg.gen_dense_host(nnz, 78, 2)
    B = dense(pkg, K, N, 78, 10)
    A = dense(pkg, M, N, 78, 11)
    d_ro, d_ci, d_bad, d_v, d_B, d_A = (to_dev(x, dev) for x in (ro, ci, bad, vals, B, A))
    C = torch.full((M * N,), float("nan"), device=dev)
    out = torch.full((nnz,), float("nan"), device=dev)
    ctx.set_option(pkg.OPT_CHECK_INPUT, 1)
    try:
        calls = {
            "spmm": lambda c: ctx.spmm(M, K, N, nnz, d_v, d_ro, c, d_B, C),
            "sddmm": lambda c: ctx.sddmm(M, K, N, nnz, d_ro, c, d_A, d_B, out),
            "fused": lambda c: ctx.fused(M, K, N, nnz, d_ro, c, d_A, d_B, d_B, C),
        }
        for name, call in calls.items():
            with pytest.raises(pkg.DlspmError) as e:
                call(d_bad)
            assert e.value.status == pkg.ERR_CSR, name
            assert "a_column_indices[i] >= KSZ" in str(e.value) and f"i = {nnz // 3}" in str(e.value), name
        arr = pkg.ProblemArray(2)
        arr.set(0, M, K, N, nnz, d_v, d_ro, d_ci, d_B, C)
        arr.set(1, M, K, N, nnz, d_v, d_ro, d_bad, d_B, torch.empty(M * N, device=dev))
        for call in (lambda: ctx.spmm_batched(arr), lambda: ctx.batch_create(arr)):
            with pytest.raises(pkg.DlspmError) as e:
                call()
            assert e.value.status == pkg.ERR_CSR
        rows = pkg.RowProblemArray("sddmm", 1)
        rows.set_sddmm(0, M, K, N, nnz, d_ro, d_bad, d_A, d_B, out)
        with pytest.raises(pkg.DlspmError) as e:
            ctx.sddmm_batched(rows)
        assert e.value.status == pkg.ERR_CSR
        host = pkg.ProblemArray(1)
        Ch = np.full(M * N, np.nan, dtype=np.float32)
        host.set(0, M, K, N, nnz, vals, ro, bad, np.ascontiguousarray(B).ravel(), Ch, host=True)
        with pytest.raises(pkg.DlspmError) as e:
            ctx.spmm_batched_host(host)
        assert e.value.status == pkg.ERR_CSR
        torch.cuda.synchronize()
        assert torch.isnan(C).all() and torch.isnan(out).all() and np.isnan(Ch).all(), "a rejected call wrote output"
        # the valid pattern passes the check and gives the usual result
        calls["spmm"](d_ci)
        torch.cuda.synchronize()
    finally:
        ctx.set_option(pkg.OPT_CHECK_INPUT, 0)
    bad_count, worst = oracle.violations(oracle.spmm(vals, ro, ci, B, M, N), C.cpu().numpy().reshape(M, N),
                                         oracle.spmm_scale(vals, ro, ci, B, M, N), TOL)
    assert bad_count == 0, worst
