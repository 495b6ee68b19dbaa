"""GPU parity of dlspm_fused_attention_f32 (scale and row softmax between the two products of the
fused chain) against the double-precision CPU restatement.  The reference has no code for these two
steps, so the checker is pinned only to numpy (tests/test_oracle_pins.py)."""
import numpy as np
import pytest

from cases import csr_bernoulli, csr_from_lengths, dense, shuffle_rows_columns
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, scale, softmax, guard=64):
    import torch

    buf = torch.full((M * N + 2 * guard,), float("nan"), device=dev)
    ctx.attention(M, K, N, int(ci.size), to_dev(ro, dev), to_dev(ci, dev), to_dev(q, dev), to_dev(k, dev),
                  to_dev(v, dev), buf[guard:guard + M * N], scale=scale,
                  flags=pkg.ATTN_SOFTMAX if softmax else 0)
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    assert np.isnan(host[:guard]).all() and np.isnan(host[guard + M * N:]).all(), "wrote outside O"
    return host[guard:guard + M * N].reshape(M, N)


def check(oracle, ro, ci, q, k, v, M, N, scale, softmax, out):
    ref, mag = oracle.attention(ro, ci, q, k, v, M, N, scale, softmax)
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, mag, TOL)
    assert bad == 0, f"{bad} elements beyond tolerance, worst ratio {worst:.3e}"


@pytest.mark.parametrize("softmax", [False, True])
def test_config4_band_mask_4096_d64(pkg, oracle, ctx, dev, softmax):
    M = K = 4096
    N = 64
    ro, ci = pkg.gen_band_csr_host(M, K, 32, 0.05, 4)
    q = dense(pkg, M, N, 4, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 4, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 4, 13, kind=pkg.KIND_NORMAL)
    scale = 1.0 / np.sqrt(N)
    check(oracle, ro, ci, q, k, v, M, N, scale, softmax,
          run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, scale, softmax))


@pytest.mark.parametrize("N", [1, 3, 4, 8, 13, 16, 32, 36, 49, 64, 65, 100, 127, 128, 130, 201, 255, 256, 258, 384, 1024, 1040])
@pytest.mark.parametrize("softmax", [False, True])
def test_feature_dimensions(pkg, oracle, ctx, dev, N, softmax):
    M, K = 45, 70
    ro, ci = csr_bernoulli(pkg, M, K, 0.3, seed=300 + N)
    q = dense(pkg, M, N, 300 + N, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 300 + N, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 300 + N, 13)
    scale = 1.0 / np.sqrt(N)
    check(oracle, ro, ci, q, k, v, M, N, scale, softmax,
          run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, scale, softmax))


@pytest.mark.parametrize("N", [64, 50])
def test_row_length_edges_and_empty_rows(pkg, oracle, ctx, dev, N):
    K = 140
    lengths = [0, 1, 0, 7, 8, 9, 31, 32, 33, 64, 65, 140, 0, 2, 0]
    ro, ci = csr_from_lengths(pkg, K, lengths, seed=7)
    ci = shuffle_rows_columns(ro, ci, seed=8)
    M = len(lengths)
    q = dense(pkg, M, N, 7, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 7, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 7, 13)
    out = run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, 0.25, True)
    check(oracle, ro, ci, q, k, v, M, N, 0.25, True, out)
    vmax, vmin = v.reshape(K, N).max(axis=0), v.reshape(K, N).min(axis=0)
    for i, n in enumerate(lengths):
        if n == 0:
            assert (out[i] == 0).all()
        elif n == 1:  # a single stored entry has weight 1
            assert np.array_equal(out[i], v.reshape(K, N)[ci[ro[i]]])
        else:         # a convex combination of rows of V
            assert (out[i] <= vmax + 1e-5).all() and (out[i] >= vmin - 1e-5).all()


def test_softmax_is_stable_for_large_scores(pkg, oracle, ctx, dev):
    """Scores near +-2000 overflow exp() unless the maximum is subtracted first; rows whose maximum
    arrives in a later pass exercise the rescaling of the partial row."""
    M, K, N = 64, 400, 32
    ro, ci = csr_bernoulli(pkg, M, K, 0.5, seed=21)
    q = dense(pkg, M, N, 21, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 21, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 21, 13)
    out = run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, 100.0, True)
    assert np.isfinite(out).all()
    ref, mag = oracle.attention(ro, ci, q, k, v, M, N, 100.0, True)
    # a score error of 1e-6 relative times a scale of 100 times |s| ~ 6 moves a weight by ~1e-3
    bad, worst = oracle.violations(ref, out, mag, 5e-3)
    assert bad == 0, worst


def test_scale_one_without_softmax_is_the_fused_chain(pkg, oracle, ctx, dev):
    import torch

    M, K, N = 300, 200, 64
    ro, ci = csr_bernoulli(pkg, M, K, 0.2, seed=31)
    q = dense(pkg, M, N, 31, 11)
    k = dense(pkg, K, N, 31, 12)
    v = dense(pkg, K, N, 31, 13)
    a = run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, 1.0, False)
    e = torch.empty(M, N, device=dev)
    ctx.fused(M, K, N, int(ci.size), to_dev(ro, dev), to_dev(ci, dev), to_dev(q, dev), to_dev(k, dev),
              to_dev(v, dev), e)
    assert np.array_equal(a.view(np.uint32), e.cpu().numpy().view(np.uint32))


def test_rejects_bad_arguments(pkg, ctx, dev):
    import torch

    z = torch.zeros(16, device=dev)
    zi = torch.zeros(5, dtype=torch.int32, device=dev)
    with pytest.raises(pkg.DlspmError):
        ctx.attention(4, 4, 4, 0, zi, zi, z, z, z, z, scale=float("nan"), flags=pkg.ATTN_SOFTMAX)
    with pytest.raises(pkg.DlspmError):
        ctx.attention(4, 4, 4, 0, zi, zi, z, z, z, z, scale=1.0, flags=8)


@pytest.mark.parametrize("K,density,N", [(100, 0.5, 64), (300, 0.4, 32), (600, 0.5, 128), (600, 0.5, 1024)])
@pytest.mark.parametrize("softmax", [False, True])
def test_few_long_rows_are_shared_between_warps(pkg, oracle, ctx, dev, K, density, N, softmax):
    """With few rows, 2, 4 or 8 warps share a row (about 50, 120 and 300 entries per row here) and
    their partial rows, maxima and sums are combined; a few rows are emptied and a few shortened so
    that some of the sharing warps have no pass at all."""
    M = 40
    ro, ci = csr_bernoulli(pkg, M, K, density, seed=41)
    lengths = np.diff(ro).copy()
    lengths[3] = 0
    lengths[7] = 1
    lengths[11] = 33
    keep = np.concatenate([np.arange(ro[i], ro[i] + min(lengths[i], ro[i + 1] - ro[i])) for i in range(M)]).astype(np.int64)
    ci = np.ascontiguousarray(ci[keep])
    ro = np.concatenate([[0], np.cumsum(np.minimum(lengths, np.diff(ro)))]).astype(np.int32)
    q = dense(pkg, M, N, 41, 11, kind=pkg.KIND_NORMAL)
    k = dense(pkg, K, N, 41, 12, kind=pkg.KIND_NORMAL)
    v = dense(pkg, K, N, 41, 13)
    scale = 1.0 / np.sqrt(N)
    out = run_attention(pkg, ctx, dev, M, K, N, ro, ci, q, k, v, scale, softmax)
    check(oracle, ro, ci, q, k, v, M, N, scale, softmax, out)
    assert (out[3] == 0).all()
