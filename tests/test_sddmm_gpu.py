"""GPU parity of dlspm_sddmm_csr_f32 against the CPU oracle (double-accumulating host loop)."""
import numpy as np
import pytest

from cases import csr_bernoulli, csr_from_lengths, dense, shuffle_rows_columns
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs, guard=64):
    import torch

    nnz = int(ci.size)
    buf = torch.full((nnz + 2 * guard,), float("nan"), device=dev)
    ctx.sddmm(M, K, N, nnz, to_dev(ro, dev), to_dev(ci, dev), to_dev(lhs, dev), to_dev(rhs, dev),
              buf[guard:guard + nnz])
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert np.isnan(host[:guard]).all() and np.isnan(host[guard + nnz:]).all(), "wrote outside the output"
    return host[guard:guard + nnz]


def check(oracle, ro, ci, lhs, rhs, M, N, out):
    ref = oracle.sddmm(ro, ci, lhs, rhs, M, N)
    scale = oracle.sddmm_scale(ro, ci, lhs, rhs, M, N)
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, scale, TOL)
    assert bad == 0, f"{bad} elements beyond tolerance, worst ratio {worst:.3e}"


def test_config2_2048x512_n128(pkg, oracle, ctx, dev):
    M, K, N = 2048, 512, 128
    ro, ci = csr_bernoulli(pkg, M, K, 0.2, seed=2)
    lhs = dense(pkg, M, N, 2, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 2, 12, kind=pkg.KIND_NORMAL)
    check(oracle, ro, ci, lhs, rhs, M, N, run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs))


# every (group width, chunks per lane) layout of the fast path, its ragged neighbours, the
# beyond-register path (N > 1024) and the narrow-vector paths (N % 4 != 0)
@pytest.mark.parametrize("N", [1, 2, 3, 4, 8, 12, 16, 28, 32, 36, 64, 100, 128, 132, 192, 256, 260,
                               512, 768, 1024, 1028, 2048, 49, 50, 127])
def test_inner_dimensions(pkg, oracle, ctx, dev, N):
    M, K = 61, 83
    ro, ci = csr_bernoulli(pkg, M, K, 0.25, seed=200 + N)
    lhs = dense(pkg, M, N, 200 + N, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 200 + N, 12, kind=pkg.KIND_NORMAL)
    check(oracle, ro, ci, lhs, rhs, M, N, run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs))


@pytest.mark.parametrize("N", [1028, 2048, 2052, 3136, 4100])
def test_long_inner_dimension_segments(pkg, oracle, ctx, dev, N):
    """Inner dimensions above 1024 run in segments (512 or 1024 floats) with a ragged last segment."""
    M, K = 70, 90
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=700 + N)
    lhs = dense(pkg, M, N, 700 + N, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 700 + N, 12, kind=pkg.KIND_NORMAL)
    check(oracle, ro, ci, lhs, rhs, M, N, run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs))


def test_row_length_edges(pkg, oracle, ctx, dev):
    K, N = 150, 64
    lengths = [0, 1, 0, 7, 8, 9, 31, 32, 33, 64, 65, 150, 0, 2, 0]
    ro, ci = csr_from_lengths(pkg, K, lengths, seed=6)
    M = len(lengths)
    lhs = dense(pkg, M, N, 6, 11)
    rhs = dense(pkg, K, N, 6, 12)
    check(oracle, ro, ci, lhs, rhs, M, N, run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs))


def test_empty_pattern_and_zero_inner_dimension(pkg, oracle, ctx, dev):
    import torch

    M, K, N = 5, 6, 32
    ro = np.zeros(M + 1, dtype=np.int32)
    ctx.sddmm(M, K, N, 0, to_dev(ro, dev), None, to_dev(dense(pkg, M, N, 1, 11), dev),
              to_dev(dense(pkg, K, N, 1, 12), dev), None)
    ro2, ci2 = csr_bernoulli(pkg, M, K, 0.5, seed=3)
    out = torch.full((int(ci2.size),), float("nan"), device=dev)
    ctx.sddmm(M, K, 0, int(ci2.size), to_dev(ro2, dev), to_dev(ci2, dev), None, None, out)
    torch.cuda.synchronize()
    assert bool((out == 0).all())


def test_unsorted_and_duplicate_columns(pkg, oracle, ctx, dev):
    M, K, N = 33, 40, 96
    ro, ci = csr_bernoulli(pkg, M, K, 0.4, seed=8)
    ci = shuffle_rows_columns(ro, ci, seed=8)
    for i in range(M):
        if ro[i + 1] - ro[i] >= 2:
            ci[ro[i] + 1] = ci[ro[i]]
    lhs = dense(pkg, M, N, 8, 11)
    rhs = dense(pkg, K, N, 8, 12)
    out = run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs)
    check(oracle, ro, ci, lhs, rhs, M, N, out)
    for i in range(M):
        if ro[i + 1] - ro[i] >= 2:
            assert out[ro[i]] == out[ro[i] + 1]


def test_deterministic(pkg, ctx, dev):
    """No atomics: two runs give identical bits."""
    M, K, N = 512, 256, 128
    ro, ci = csr_bernoulli(pkg, M, K, 0.2, seed=12)
    lhs = dense(pkg, M, N, 12, 11)
    rhs = dense(pkg, K, N, 12, 12)
    a = run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs)
    b = run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("offset", [1, 2])
def test_unaligned_dense_pointers(pkg, oracle, ctx, dev, offset):
    import torch

    M, K, N = 30, 20, 64
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=13)
    lhs = dense(pkg, M, N, 13, 11)
    rhs = dense(pkg, K, N, 13, 12)
    bufL = torch.zeros(M * N + 8, device=dev)
    bufL[offset:offset + M * N] = to_dev(lhs.ravel(), dev)
    out = torch.full((int(ci.size),), float("nan"), device=dev)
    ctx.sddmm(M, K, N, int(ci.size), to_dev(ro, dev), to_dev(ci, dev), bufL[offset:offset + M * N],
              to_dev(rhs, dev), out)
    torch.cuda.synchronize()
    check(oracle, ro, ci, lhs, rhs, M, N, out.cpu().numpy())


def test_full_size_outer_product_property(pkg, ctx, dev):
    """Rank-one inputs at a large size: lhs[i, :] = a_i * u and rhs[j, :] = b_j * u give
    out[p] = a_i * b_j * |u|^2, checked for every nonzero with torch on the device."""
    import torch

    M, K, N = 16384, 8192, 128
    density = 0.05
    counts = torch.zeros(M, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_count(M, K, density, 91, counts)
    ro = torch.zeros(M + 1, dtype=torch.int32, device=dev)
    ro[1:] = torch.cumsum(counts, 0).to(torch.int32)
    nnz = int(ro[-1].item())
    ci = torch.empty(nnz, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_fill(M, K, density, 91, ro, ci)
    a = torch.empty(M, device=dev)
    b = torch.empty(K, device=dev)
    u = torch.empty(N, device=dev)
    ctx.gen_dense(a, 91, 20)
    ctx.gen_dense(b, 91, 21)
    ctx.gen_dense(u, 91, 22)
    lhs = (a[:, None] * u[None, :]).contiguous()
    rhs = (b[:, None] * u[None, :]).contiguous()
    out = torch.full((nnz,), float("nan"), device=dev)
    ctx.sddmm(M, K, N, nnz, ro, ci, lhs, rhs, out)
    torch.cuda.synchronize()
    rows = torch.repeat_interleave(torch.arange(M, device=dev), counts.long())
    ld, rd = lhs.double(), rhs.double()
    step = 1 << 20  # bounds the temporary gathers to about 1 GiB each
    for s in range(0, nnz, step):
        e = min(nnz, s + step)
        x, y = ld[rows[s:e]], rd[ci[s:e].long()]
        w = (x * y).sum(dim=1)
        sc = (x.abs() * y.abs()).sum(dim=1)
        assert bool(((out[s:e].double() - w).abs() <= TOL * torch.maximum(w.abs(), sc)).all())


@pytest.mark.parametrize("N", [3, 64, 128, 130, 2048])
def test_mask_values_scale_the_products(pkg, oracle, ctx, dev, N):
    """dlspm_sddmm_csr_masked_f32: S_ij * (A_i . B_j); a NULL mask is the reference's all-ones mask.
    One kernel path per N here (scalar, two fast layouts, two-float vectors, segmented)."""
    import torch

    M, K = 90, 75
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=900 + N)
    nnz = int(ci.size)
    lhs = dense(pkg, M, N, 900 + N, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 900 + N, 12, kind=pkg.KIND_NORMAL)
    mask = pkg.gen_dense_host(nnz, 900 + N, 2)
    d = [to_dev(a, dev) for a in (ro, ci, mask, lhs, rhs)]
    plain = torch.full((nnz,), float("nan"), device=dev)
    masked = torch.full((nnz,), float("nan"), device=dev)
    nomask = torch.full((nnz,), float("nan"), device=dev)
    ctx.sddmm(M, K, N, nnz, d[0], d[1], d[3], d[4], plain)
    ctx.sddmm_masked(M, K, N, nnz, d[0], d[1], d[2], d[3], d[4], masked)
    ctx.sddmm_masked(M, K, N, nnz, d[0], d[1], None, d[3], d[4], nomask)
    torch.cuda.synchronize()
    plain, masked, nomask = plain.cpu().numpy(), masked.cpu().numpy(), nomask.cpu().numpy()
    assert np.array_equal(plain.view(np.uint32), nomask.view(np.uint32))
    assert np.array_equal(masked.view(np.uint32), (mask * plain).view(np.uint32))  # one rounding after the dot
    ref = oracle.sddmm(ro, ci, lhs, rhs, M, N).astype(np.float64) * mask
    scale = oracle.sddmm_scale(ro, ci, lhs, rhs, M, N) * np.abs(mask)
    bad, worst = oracle.violations(ref.astype(np.float32), masked, scale.astype(np.float32), TOL)
    assert bad == 0, worst


@pytest.mark.parametrize("M,K,N,density", [(64, 576, 3136, 0.1), (64, 64, 3136, 0.1), (128, 512, 784, 0.1),
                                           (512, 128, 784, 0.1), (256, 256, 64, 0.5), (2, 300, 128, 0.9),
                                           (64, 576, 32, 0.1), (2, 300, 16, 0.9), (128, 512, 32, 0.3), (16, 4096, 24, 0.5),
                                           (64, 576, 49, 0.1), (2, 300, 13, 0.9), (128, 512, 201, 0.2), (300, 700, 255, 0.3)])
def test_tiny_patterns_share_rows_and_passes(pkg, oracle, ctx, dev, M, K, N, density):
    """Layer-sized patterns (tens to hundreds of rows): warps share a row's passes and, where the
    device would still be mostly idle, the nonzeros inside a pass."""
    ro, ci = csr_bernoulli(pkg, M, K, density, seed=1000 + M + N)
    lhs = dense(pkg, M, N, 1000 + M, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 1000 + M, 12, kind=pkg.KIND_NORMAL)
    check(oracle, ro, ci, lhs, rhs, M, N, run_sddmm(ctx, dev, M, K, N, ro, ci, lhs, rhs))



@pytest.mark.parametrize("offset_floats", [0, 4])
def test_rows_of_32_floats_in_a_long_launch(pkg, oracle, ctx, dev, offset_floats):
    """N = 32 with 8192 rows or more: 32-byte aligned operands take the build with one 256-bit load per
    lane and nonzero; operands aligned to 16 bytes only (offset of four floats) must take the 16-byte
    build.  Both against the oracle, with empty rows and a ragged last pass in most rows."""
    import torch

    M, K, N = 9000, 700, 32
    ro, ci = csr_bernoulli(pkg, M, K, 0.07, seed=91)
    nnz = int(ci.size)
    lhs = dense(pkg, M, N, 91, 11, kind=pkg.KIND_NORMAL)
    rhs = dense(pkg, K, N, 91, 12, kind=pkg.KIND_NORMAL)
    d_lhs = torch.empty(M * N + 8, device=dev)[offset_floats:offset_floats + M * N]
    d_rhs = torch.empty(K * N + 8, device=dev)[offset_floats:offset_floats + K * N]
    d_lhs.copy_(torch.from_numpy(np.ascontiguousarray(lhs).ravel()))
    d_rhs.copy_(torch.from_numpy(np.ascontiguousarray(rhs).ravel()))
    assert d_rhs.data_ptr() % 32 == (16 if offset_floats else 0)
    out = torch.full((nnz,), float("nan"), device=dev)
    ctx.sddmm(M, K, N, nnz, to_dev(ro, dev), to_dev(ci, dev), d_lhs, d_rhs, out)
    torch.cuda.synchronize()
    check(oracle, ro, ci, lhs, rhs, M, N, out.cpu().numpy())
