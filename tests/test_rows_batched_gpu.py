"""Grouped launches over many independent SDDMMs and fused SDDMM -> SpMM chains
(dlspm_sddmm_batched_f32, dlspm_fused_batched_f32 and their host-pointer forms) against the CPU
oracle: mixed shapes and inner dimensions (every register layout, plus inner dimensions that fall
back to the single-matrix kernels), empty problems, problems without entries, empty rows."""
import numpy as np
import pytest

from cases import csr_rowlen_normal, dense
from conftest import TOL, to_dev

pytestmark = pytest.mark.gpu

SHAPES = [(8, 8), (61, 83), (64, 256), (256, 64), (300, 512)]
SPARSITIES = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]
# one inner dimension per layout (4x1, 4x2, 8x2, 8x4, 16x4, 32x4, 32x8), scalar fall-backs, long rows in segments
WIDTHS = [16, 32, 64, 128, 256, 512, 1024, 100, 50, 33, 1028, 3136, 8, 24]


def make_problems(pkg, count, seed, widths=WIDTHS):
    probs = []
    for i in range(count):
        h = pkg.rand_u64(seed, 70, i)
        M, K = SHAPES[h % 5]
        N = widths[(h >> 16) % len(widths)]
        s = seed * 1000 + i
        ro, ci = csr_rowlen_normal(pkg, M, K, SPARSITIES[(h >> 8) % 6], s, cov=0.8)
        probs.append(dict(M=M, K=K, N=N, ro=ro, ci=ci, a=dense(pkg, M, N, s, 11, kind=pkg.KIND_NORMAL),
                          b=dense(pkg, K, N, s, 12, kind=pkg.KIND_NORMAL), d=dense(pkg, K, N, s, 13, kind=pkg.KIND_NORMAL),
                          mask=pkg.gen_dense_host(int(ci.size), s, 14) if i % 3 == 0 else None))
    # a problem with no rows and one whose rows are all empty, in the middle of the batch
    z = np.zeros
    probs.insert(3, dict(M=0, K=8, N=16, ro=z(1, np.int32), ci=z(0, np.int32), a=z((0, 16), np.float32),
                         b=z((8, 16), np.float32), d=z((8, 16), np.float32), mask=None))
    probs.insert(7, dict(M=6, K=8, N=16, ro=z(7, np.int32), ci=z(0, np.int32), a=dense(pkg, 6, 16, 1, 11),
                         b=dense(pkg, 8, 16, 1, 12), d=dense(pkg, 8, 16, 1, 13), mask=None))
    return probs


def check_sddmm(oracle, p, out):
    nnz = int(p["ci"].size)
    if nnz == 0:
        return
    ref = oracle.sddmm(p["ro"], p["ci"], p["a"], p["b"], p["M"], p["N"])
    scale = oracle.sddmm_scale(p["ro"], p["ci"], p["a"], p["b"], p["M"], p["N"])
    if p["mask"] is not None:
        ref, scale = ref * p["mask"], scale * np.abs(p["mask"])
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, scale, TOL)
    assert bad == 0, f"M={p['M']} K={p['K']} N={p['N']}: {bad} beyond tolerance, worst {worst:.3e}"


def check_fused(oracle, p, out):
    if p["M"] == 0:
        return
    ref, _ = oracle.fused(p["ro"], p["ci"], p["a"], p["b"], p["d"], p["M"], p["N"])
    scale = oracle.fused_scale(p["ro"], p["ci"], p["a"], p["b"], p["d"], p["M"], p["N"])
    out = out.reshape(p["M"], p["N"])
    assert not np.isnan(out).any(), "output not fully written"
    bad, worst = oracle.violations(ref, out, scale, TOL)
    assert bad == 0, f"M={p['M']} K={p['K']} N={p['N']}: {bad} beyond tolerance, worst {worst:.3e}"
    empty = np.diff(p["ro"]) == 0
    assert (out[empty] == 0).all(), "rows without entries must give zeros"


def test_sddmm_batched_matches_oracle_and_single_launches(pkg, oracle, ctx, dev):
    import torch

    probs = make_problems(pkg, 60, seed=5)
    arr = pkg.RowProblemArray("sddmm", len(probs))
    outs, singles = [], []
    for i, p in enumerate(probs):
        nnz = int(p["ci"].size)
        o = torch.full((max(nnz, 1),), float("nan"), device=dev)[:nnz]
        outs.append(o)
        d = [to_dev(p[k], dev) for k in ("ro", "ci", "a", "b")]
        m = to_dev(p["mask"], dev) if p["mask"] is not None else None
        arr.set_sddmm(i, p["M"], p["K"], p["N"], nnz, d[0], d[1], d[2], d[3], o, mask_values=m)
        s = torch.full((max(nnz, 1),), float("nan"), device=dev)[:nnz]
        ctx.sddmm_masked(p["M"], p["K"], p["N"], nnz, d[0], d[1], m, d[2], d[3], s)
        singles.append(s)
    ctx.sddmm_batched(arr)
    ctx.sddmm_batched(arr)  # the tables in the context's scratch are rebuilt by every call
    torch.cuda.synchronize()
    for p, o, s in zip(probs, outs, singles):
        check_sddmm(oracle, p, o.cpu().numpy())
        # a row is processed exactly as by the single-matrix kernel whenever that kernel gives one
        # warp the whole row (it may share long rows of small patterns between warps, same sums)
        assert torch.allclose(o, s, rtol=1e-5, atol=1e-6)


def test_fused_batched_matches_oracle(pkg, oracle, ctx, dev):
    import torch

    probs = make_problems(pkg, 50, seed=6)
    arr = pkg.RowProblemArray("fused", len(probs))
    outs = []
    for i, p in enumerate(probs):
        o = torch.full((max(p["M"] * p["N"], 1),), float("nan"), device=dev)[: p["M"] * p["N"]]
        outs.append(o)
        arr.set_fused(i, p["M"], p["K"], p["N"], int(p["ci"].size), to_dev(p["ro"], dev), to_dev(p["ci"], dev),
                      to_dev(p["a"], dev), to_dev(p["b"], dev), to_dev(p["d"], dev), o)
    ctx.fused_batched(arr)
    torch.cuda.synchronize()
    for p, o in zip(probs, outs):
        check_fused(oracle, p, o.cpu().numpy())


def test_batched_host_forms(pkg, oracle, ctx):
    probs = make_problems(pkg, 25, seed=7)
    sd = pkg.RowProblemArray("sddmm", len(probs), host=True)
    fu = pkg.RowProblemArray("fused", len(probs), host=True)
    souts, fouts = [], []
    for i, p in enumerate(probs):
        nnz = int(p["ci"].size)
        so = np.full(nnz, np.nan, dtype=np.float32)
        fo = np.full(p["M"] * p["N"], np.nan, dtype=np.float32)
        souts.append(so)
        fouts.append(fo)
        flat = {k: np.ascontiguousarray(p[k]).ravel() for k in ("a", "b", "d")}
        sd.set_sddmm(i, p["M"], p["K"], p["N"], nnz, p["ro"], p["ci"], flat["a"], flat["b"], so, mask_values=p["mask"])
        fu.set_fused(i, p["M"], p["K"], p["N"], nnz, p["ro"], p["ci"], flat["a"], flat["b"], flat["d"], fo)
    ctx.sddmm_batched_host(sd)
    ctx.fused_batched_host(fu)
    for p, so, fo in zip(probs, souts, fouts):
        check_sddmm(oracle, p, so)
        check_fused(oracle, p, fo)


def test_batched_rejects_bad_problems_and_capturing_streams(pkg, ctx, dev):
    import torch

    arr = pkg.RowProblemArray("sddmm", 1)
    ro = torch.zeros(5, dtype=torch.int32, device=dev)
    arr.set_sddmm(0, 4, 4, 8, 3, ro, None, None, None, None)  # entries but no arrays
    with pytest.raises(pkg.DlspmError) as e:
        ctx.sddmm_batched(arr)
    assert e.value.status == pkg.ERR_INVALID_ARGUMENT
    good = pkg.RowProblemArray("fused", 1)
    t = torch.zeros(32, device=dev)
    good.set_fused(0, 4, 4, 8, 0, ro, None, t, t, t, torch.empty(32, device=dev))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        graph.capture_begin()
        try:
            with pytest.raises(pkg.DlspmError) as e:
                ctx.fused_batched(good, stream=side)
            assert e.value.status == pkg.ERR_UNSUPPORTED
        finally:
            graph.capture_end()
    torch.cuda.synchronize()
    ctx.fused_batched(good)
    torch.cuda.synchronize()
