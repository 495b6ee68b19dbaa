"""dlspm_spmm_csr_f32_scatter: the row-sharded SpMM whose epilogue stores every finished row into
all destination buffers (fused compute + gather)."""
import numpy as np
import pytest

from cases import csr_rowlen_normal, dense
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu


def _case(pkg, M=500, K=160, N=72, seed=31):
    ro, ci = csr_rowlen_normal(pkg, M, K, 0.85, seed)
    vals = pkg.gen_dense_host(int(ci.size), seed, 2)
    B = dense(pkg, K, N, seed, 10)
    return M, K, N, ro, ci, vals, B


@pytest.mark.parametrize("N", [72, 256, 33])
def test_scatter_writes_row_block_into_every_destination(pkg, oracle, ctx, dev, N):
    import importlib
    import torch

    import __graft_entry__ as entry

    sharding = importlib.import_module(entry.PKG_NAME + ".sharding")
    M, K, N, ro, ci, vals, B = _case(pkg, N=N)
    ref = oracle.spmm(vals, ro, ci, B, M, N)
    scale = oracle.spmm_scale(vals, ro, ci, B, M, N)
    parts = 3
    dsts = [torch.full((M, N), float("nan"), device=dev) for _ in range(2)]
    d_B = to_dev(B, dev)
    bounds = pkg.partition_rows_by_nnz(ro, parts)
    for p in range(parts):  # the three row blocks one after the other, as three ranks would
        r0, r1 = int(bounds[p]), int(bounds[p + 1])
        lo, hi = int(ro[r0]), int(ro[r1])
        ctx.spmm_scatter(r1 - r0, K, N, hi - lo, to_dev(vals[lo:hi], dev), to_dev(sharding.rebase_offsets(ro, r0, r1), dev),
                         to_dev(ci[lo:hi], dev), d_B, [d.data_ptr() for d in dsts], r0)
    torch.cuda.synchronize()
    for d in dsts:
        out = d.cpu().numpy()
        assert not np.isnan(out).any()
        bad, worst = oracle.violations(ref, out, scale, TOL)
        assert bad == 0, worst
    assert torch.equal(dsts[0], dsts[1])
    # same bits as the plain kernel in strict mode (both accumulate in CSR order; the default lone
    # launch may share a row between warps, which reorders the partial sums)
    plain = torch.empty(M, N, device=dev)
    ctx.spmm(M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), d_B, plain)
    torch.cuda.synchronize()
    assert torch.allclose(plain, dsts[0], rtol=1e-5, atol=1e-5)


def test_scatter_strict_mode_reproduces_the_host_loop_bits(pkg, oracle, ctx, dev):
    """With DLSPM_OPT_STRICT_FP32 the scatter form multiplies and adds with separate roundings in
    CSR order, like dlspm_spmm_csr_f32: every destination holds the oracle's bits."""
    import torch

    M, K, N, ro, ci, vals, B = _case(pkg, M=300, K=200, N=132, seed=41)
    dsts = [torch.full((M, N), float("nan"), device=dev) for _ in range(3)]
    ctx.set_option(pkg.OPT_STRICT_FP32, 1)
    try:
        ctx.spmm_scatter(M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev),
                         [d.data_ptr() for d in dsts], 0)
        torch.cuda.synchronize()
    finally:
        ctx.set_option(pkg.OPT_STRICT_FP32, 0)
    ref = oracle.spmm(vals, ro, ci, B, M, N)
    for d in dsts:
        assert np.array_equal(d.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_scatter_rejects_bad_destination_lists(pkg, ctx, dev):
    import torch

    M, K, N, ro, ci, vals, B = _case(pkg, M=8, K=8, N=8)
    args = (M, K, N, int(ci.size), to_dev(vals, dev), to_dev(ro, dev), to_dev(ci, dev), to_dev(B, dev))
    c = torch.empty(M, N, device=dev)
    with pytest.raises(pkg.DlspmError):
        ctx.spmm_scatter(*args, [], 0)
    with pytest.raises(pkg.DlspmError):
        ctx.spmm_scatter(*args, [c.data_ptr()] * 9, 0)


def test_scatter_between_two_gpus_in_one_process(pkg, oracle):
    """Each GPU computes its row block and stores it into its own C and into the peer's C."""
    import importlib
    import torch

    import __graft_entry__ as entry

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sharding = importlib.import_module(entry.PKG_NAME + ".sharding")
    M, K, N, ro, ci, vals, B = _case(pkg, M=4000, K=512, N=260, seed=37)
    ctxs = [pkg.Context(0), pkg.Context(1)]
    ctxs[0].enable_peer_access(1)
    ctxs[1].enable_peer_access(0)
    devs = [torch.device("cuda:0"), torch.device("cuda:1")]
    full = [torch.full((M, N), float("nan"), device=d) for d in devs]
    bounds = pkg.partition_rows_by_nnz(ro, 2)
    for r in range(2):
        r0, r1 = int(bounds[r]), int(bounds[r + 1])
        lo, hi = int(ro[r0]), int(ro[r1])
        with torch.cuda.device(devs[r]):
            ctxs[r].spmm_scatter(r1 - r0, K, N, hi - lo, to_dev(vals[lo:hi], devs[r]),
                                 to_dev(sharding.rebase_offsets(ro, r0, r1), devs[r]), to_dev(ci[lo:hi], devs[r]),
                                 to_dev(B, devs[r]), [full[r].data_ptr(), full[1 - r].data_ptr()], r0)
    for d in devs:
        torch.cuda.synchronize(d)
    ref = oracle.spmm(vals, ro, ci, B, M, N)
    scale = oracle.spmm_scale(vals, ro, ci, B, M, N)
    for f in full:
        out = f.cpu().numpy()
        assert not np.isnan(out).any()
        bad, worst = oracle.violations(ref, out, scale, TOL)
        assert bad == 0, worst
    assert torch.equal(full[0].cpu(), full[1].cpu())
    for c in ctxs:
        c.close()
