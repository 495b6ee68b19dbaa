"""GPU parity of dlspm_fused_sddmm_spmm_f32 against the unfused CPU oracle (Sddmm then Spmm)."""
import numpy as np
import pytest

from cases import csr_bernoulli, csr_from_lengths, dense, shuffle_rows_columns
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def run_fused(ctx, dev, M, K, N, ro, ci, q, k, v, guard=64):
    import torch

    buf = torch.full((M * N + 2 * guard,), float("nan"), device=dev)
    ctx.fused(M, K, N, int(ci.size), to_dev(ro, dev), to_dev(ci, dev), to_dev(q, dev), to_dev(k, dev),
              to_dev(v, dev), buf[guard:guard + M * N])
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert np.isnan(host[:guard]).all() and np.isnan(host[guard + M * N:]).all(), "wrote outside E"
    return host[guard:guard + M * N].reshape(M, N)


def check(oracle, ro, ci, q, k, v, M, N, out):
    ref, _ = oracle.fused(ro, ci, q, k, v, M, N)
    scale = oracle.fused_scale(ro, ci, q, k, v, M, N)
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, scale, TOL)
    assert bad == 0, f"{bad} elements beyond tolerance, worst ratio {worst:.3e}"


def test_config4_band_mask_4096_d64(pkg, oracle, ctx, dev):
    M = K = 4096
    N = 64
    ro, ci = pkg.gen_band_csr_host(M, K, 32, 0.05, 4)
    q = dense(pkg, M, N, 4, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 4, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 4, 13, kind=pkg.KIND_NORMAL)
    check(oracle, ro, ci, q, k, v, M, N, run_fused(ctx, dev, M, K, N, ro, ci, q, k, v))


@pytest.mark.parametrize("N", [1, 3, 4, 8, 13, 16, 32, 36, 49, 64, 65, 100, 127, 128, 130, 201, 255, 256, 258, 384, 1024, 1040])
def test_feature_dimensions(pkg, oracle, ctx, dev, N):
    M, K = 45, 70
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=300 + N)
    q = dense(pkg, M, N, 300 + N, 11)
    k = dense(pkg, K, N, 300 + N, 12)
    v = dense(pkg, K, N, 300 + N, 13)
    check(oracle, ro, ci, q, k, v, M, N, run_fused(ctx, dev, M, K, N, ro, ci, q, k, v))


def test_row_length_edges_and_empty_rows(pkg, oracle, ctx, dev):
    K, N = 140, 64
    lengths = [0, 1, 0, 7, 8, 9, 31, 32, 33, 64, 65, 140, 0, 2, 0]
    ro, ci = csr_from_lengths(pkg, K, lengths, seed=7)
    M = len(lengths)
    q = dense(pkg, M, N, 7, 11)
    k = dense(pkg, K, N, 7, 12)
    v = dense(pkg, K, N, 7, 13)
    out = run_fused(ctx, dev, M, K, N, ro, ci, q, k, v)
    check(oracle, ro, ci, q, k, v, M, N, out)
    for i, n in enumerate(lengths):
        if n == 0:
            assert (out[i] == 0).all()


def test_unsorted_columns(pkg, oracle, ctx, dev):
    M, K, N = 37, 50, 32
    ro, ci = csr_bernoulli(pkg, M, K, 0.4, seed=15)
    ci = shuffle_rows_columns(ro, ci, seed=15)
    q = dense(pkg, M, N, 15, 11)
    k = dense(pkg, K, N, 15, 12)
    v = dense(pkg, K, N, 15, 13)
    check(oracle, ro, ci, q, k, v, M, N, run_fused(ctx, dev, M, K, N, ro, ci, q, k, v))


def test_matches_unfused_gpu_path(pkg, oracle, ctx, dev):
    """Fused result against SDDMM followed by SpMM on the GPU (the products written to memory)."""
    import torch

    M, K, N = 600, 500, 64
    ro, ci = csr_bernoulli(pkg, M, K, 0.1, seed=16)
    nnz = int(ci.size)
    q = dense(pkg, M, N, 16, 11)
    k = dense(pkg, K, N, 16, 12)
    v = dense(pkg, K, N, 16, 13)
    fused = run_fused(ctx, dev, M, K, N, ro, ci, q, k, v)
    d_ro, d_ci = to_dev(ro, dev), to_dev(ci, dev)
    s = torch.empty(nnz, device=dev)
    e = torch.empty(M, N, device=dev)
    ctx.sddmm(M, K, N, nnz, d_ro, d_ci, to_dev(q, dev), to_dev(k, dev), s)
    ctx.spmm(M, K, N, nnz, s, d_ro, d_ci, to_dev(v, dev), e)
    torch.cuda.synchronize()
    scale = oracle.fused_scale(ro, ci, q, k, v, M, N)
    bad, worst = oracle.violations(e.cpu().numpy(), fused, scale, TOL)
    assert bad == 0, worst


@pytest.mark.parametrize("K,density,N", [(100, 0.5, 64), (300, 0.4, 16), (600, 0.5, 128), (600, 0.5, 512)])
def test_few_long_rows_are_shared_between_warps(pkg, oracle, ctx, dev, K, density, N):
    """2, 4 or 8 warps per row (about 50, 120 and 300 entries per row) with their partial rows added
    through shared memory."""
    M = 40
    ro, ci = csr_bernoulli(pkg, M, K, density, seed=43)
    q = dense(pkg, M, N, 43, 11)
    k = dense(pkg, K, N, 43, 12)
    v = dense(pkg, K, N, 43, 13)
    check(oracle, ro, ci, q, k, v, M, N, run_fused(ctx, dev, M, K, N, ro, ci, q, k, v))


@pytest.mark.parametrize("offset_floats", [0, 4])
def test_rows_of_32_floats_in_a_long_launch(pkg, oracle, ctx, dev, offset_floats):
    """d = 32 with 8192 rows or more: 32-byte aligned operands take the build with 256-bit loads for
    the gathers of B and D; operands aligned to 16 bytes only must take the 16-byte build."""
    import torch

    M, K, N = 9000, 600, 32
    ro, ci = csr_bernoulli(pkg, M, K, 0.06, seed=92)
    q = dense(pkg, M, N, 92, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 92, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 92, 13, kind=pkg.KIND_NORMAL)

    def place(a):
        t = torch.empty(a.size + 8, device=dev)[offset_floats:offset_floats + a.size]
        t.copy_(torch.from_numpy(np.ascontiguousarray(a).ravel()))
        return t

    d_q, d_k, d_v = place(q), place(k), place(v)
    assert d_k.data_ptr() % 32 == (16 if offset_floats else 0)
    out = torch.full((M * N,), float("nan"), device=dev)
    ctx.fused(M, K, N, int(ci.size), to_dev(ro, dev), to_dev(ci, dev), d_q, d_k, d_v, out)
    torch.cuda.synchronize()
    check(oracle, ro, ci, q, k, v, M, N, out.cpu().numpy().reshape(M, N))
