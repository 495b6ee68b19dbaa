"""dlspm_spmm_batched_f32_static: the grouped SpMM for callers that cannot allocate device memory
(for example a plug-in whose host application owns the device heap).  Its tables live in a fixed
device array inside the library instead of cudaMalloc'ed scratch, so its results must equal those
of dlspm_spmm_batched_f32 exactly; the array is shared by all calls and keeps the previous call's
contents, so two calls in a row with different batches are checked.  The test also checks the one
property the entry point exists for: once the first call on a device has looked up the array's
address, further calls leave the amount of free device memory unchanged.

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
    host, ref_out, new_out = [], [], []
    a = pkg.ProblemArray(count)
    b = pkg.ProblemArray(count)
    keep = []
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
        keep.append(d)
        host.append((M, K, N, ro, ci, vals, B))
        ref_out.append(c_ref)
        new_out.append(c_new)
    return a, b, ref_out, new_out, host, keep


def test_static_scratch_variant_matches_allocating_entry_point(pkg, oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    dev = torch.device("cuda:0")
    # every device buffer of the test exists before the first reading of free memory
    batches = [build_batch(pkg, dev, seed, count, widths)
               for seed, count, widths in ((1, 37, (256, 100, 33)), (2, 9, (64, 1024, 6)))]
    big = pkg.ProblemArray(1025)
    for i in range(1025):
        big.set_raw(i, 0, 1, 1, 0, None, None, None, None, None)
    ctx = pkg.Context(0)        # only ever makes static calls: nothing else may grow its scratch
    ctx_alloc = pkg.Context(0)  # the allocating entry point runs on a context of its own
    try:
        # the first call on the device looks up the array's address; it is the warm-up
        ctx.spmm_batched_static(batches[0][1])
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        # two different batches back to back: the second call finds the first call's tables and
        # counter in the shared array and must not be affected by them
        for (a, b, ref_out, new_out, host, _keep) in batches:
            for c in new_out:
                c.fill_(float("nan"))
            ctx.spmm_batched_static(b)
        # same batch again through the static entry point only
        ctx.spmm_batched_static(batches[1][1])
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "a static call changed the free device memory"
        for (a, b, ref_out, new_out, host, _keep) in batches:
            ctx_alloc.spmm_batched(a)
            torch.cuda.synchronize()
            for (M, K, N, ro, ci, vals, B), r, n in zip(host, ref_out, new_out):
                r_h, n_h = r.cpu().numpy(), n.cpu().numpy()
                assert not np.isnan(n_h).any(), "output not fully written"
                np.testing.assert_allclose(n_h, r_h, rtol=TOL, atol=0.0)
                assert np.array_equal(n_h.view(np.uint32), r_h.view(np.uint32))
                # and against the CPU oracle, like every other kernel
                ref = oracle.spmm(vals, ro, ci, B, M, N)
                scale = oracle.spmm_scale(vals, ro, ci, B, M, N)
                bad, worst = oracle.violations(ref, n_h.reshape(M, N), scale, TOL)
                assert bad == 0, worst
        # beyond the fixed limit: a clear error, nothing launched
        with pytest.raises(pkg.DlspmError) as e:
            ctx.spmm_batched_static(big)
        assert e.value.status == pkg.ERR_UNSUPPORTED and "1024" in str(e.value)
    finally:
        ctx.close()
        ctx_alloc.close()


def test_one_shot_grouped_launches_refuse_a_capturing_stream(pkg):
    """Both one-shot grouped launches copy their tables from host memory that dies with the call, so
    a CUDA graph that recorded them would replay garbage: on a capturing stream they must return
    DLSPM_ERR_UNSUPPORTED before anything is enqueued.  Nothing is launched by this test."""
    import torch

    dev = torch.device("cuda:0")
    a, b, _r, _n, _h, _keep = build_batch(pkg, dev, 3, 5, (64,))
    ctx = pkg.Context(0)
    try:
        ctx.spmm_batched_static(b)  # address lookup outside any capture
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            graph.capture_begin()
            try:
                for call, arr in ((ctx.spmm_batched_static, b), (ctx.spmm_batched, a)):
                    with pytest.raises(pkg.DlspmError) as e:
                        call(arr, stream=side)
                    assert e.value.status == pkg.ERR_UNSUPPORTED and "captur" in str(e.value)
            finally:
                graph.capture_end()
        torch.cuda.synchronize()
        ctx.spmm_batched_static(b)  # the context is still usable
        torch.cuda.synchronize()
    finally:
        ctx.close()
