"""dlspm_spmm_batched_f32_static: the grouped SpMM for callers that cannot allocate device memory
(for example a plug-in whose host application owns the device heap).  Its tables live in a fixed
device array inside the library instead of cudaMalloc'ed scratch, so its results must equal those
of dlspm_spmm_batched_f32 exactly; the array is shared by all calls and keeps the previous call's
contents, so two calls in a row with different batches are checked.

This file is collected last on purpose: a failure here does not hide the other tests in a run that
stops at the first failure.  It creates its own context so that it behaves the same alone and after
the rest of the suite.
"""
import numpy as np
import pytest

from cases import csr_rowlen_normal, dense
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def build_batch(pkg, dev, seed, count, widths):
    import torch

    shapes = [(8, 8), (32, 32), (64, 256), (256, 64), (128, 512)]
    sparsities = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]
    tensors, ref_out, new_out = [], [], []
    a = pkg.ProblemArray(count)
    b = pkg.ProblemArray(count)
    for i in range(count):
        h = pkg.rand_u64(seed, 60, i)
        M, K = shapes[h % 5]
        N = widths[(h >> 16) % len(widths)]
        ro, ci = csr_rowlen_normal(pkg, M, K, sparsities[(h >> 8) % 6], seed * 100 + i)
        vals = pkg.gen_dense_host(int(ci.size), seed * 100 + i, 2)
        B = dense(pkg, K, N, seed * 100 + i, 10)
        d = (to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev))
        c_ref = torch.full((M * N,), float("nan"), device=dev)
        c_new = torch.full((M * N,), float("nan"), device=dev)
        a.set(i, M, K, N, int(ci.size), *d, c_ref)
        b.set(i, M, K, N, int(ci.size), *d, c_new)
        tensors.append(d)
        ref_out.append(c_ref)
        new_out.append(c_new)
    return a, b, ref_out, new_out


def test_static_scratch_variant_matches_allocating_entry_point(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    ctx = pkg.Context(0)
    try:
        # two different batches back to back: the second call finds the first call's tables and
        # counter in the shared array and must not be affected by them
        for seed, count, widths in ((1, 37, (256, 100, 33)), (2, 9, (64, 1024, 6))):
            a, b, ref_out, new_out = build_batch(pkg, dev, seed, count, widths)
            ctx.spmm_batched(a)
            ctx.spmm_batched_static(b)
            torch.cuda.synchronize()
            for r, n in zip(ref_out, new_out):
                r_h, n_h = r.cpu().numpy(), n.cpu().numpy()
                assert not np.isnan(n_h).any(), "output not fully written"
                np.testing.assert_allclose(n_h, r_h, rtol=TOL, atol=0.0)
                assert np.array_equal(n_h.view(np.uint32), r_h.view(np.uint32))
        # same batch again through the static entry point only: identical bits once more
        ctx.spmm_batched_static(b)
        torch.cuda.synchronize()
        for r, n in zip(ref_out, new_out):
            assert torch.equal(r, n)
        # beyond the fixed limit: a clear error, nothing launched
        big = pkg.ProblemArray(1025)
        for i in range(1025):
            big.set_raw(i, 0, 1, 1, 0, None, None, None, None, None)
        with pytest.raises(pkg.DlspmError) as e:
            ctx.spmm_batched_static(big)
        assert e.value.status == pkg.ERR_UNSUPPORTED and "1024" in str(e.value)
    finally:
        ctx.close()
