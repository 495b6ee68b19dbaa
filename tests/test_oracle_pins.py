"""Pins the CPU oracle: (1) against golden vectors produced by the reference's own object code
(tests/golden/*.npz, made by tests/golden/make_golden.py), always; (2) against that object code
itself when oracle/_ref/ is present.  All comparisons are bit for bit."""
import glob
import hashlib
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = sorted(glob.glob(os.path.join(HERE, "golden", "*.npz")))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).ravel().view(np.uint32)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def inputs_of(pkg, g):
    M, K, N, seed, vkind = (int(g[k]) for k in ("M", "K", "N", "seed", "vkind"))
    if int(g["full"]):
        return M, K, N, g["row_offsets"], g["column_indices"], g["values"], g["c"], g["b"], g["d"]
    param = g["pattern_param"]
    if str(g["pattern_kind"]) == "bernoulli":
        ro, ci = pkg.gen_bernoulli_csr_host(M, K, float(param[0]), seed)
    else:
        ro, ci = pkg.gen_band_csr_host(M, K, int(param[0]), float(param[1]), seed)
    vals = pkg.gen_dense_host(int(ci.size), seed, 2, kind=vkind)
    c = pkg.gen_dense_host(M * N, seed, 11, kind=vkind).reshape(M, N)
    b = pkg.gen_dense_host(K * N, seed, 12, kind=vkind).reshape(K, N)
    d = pkg.gen_dense_host(K * N, seed, 13, kind=vkind).reshape(K, N)
    return M, K, N, ro, ci, vals, c, b, d


def expect(g, key, got):
    got = np.ascontiguousarray(got, dtype=np.float32).ravel()
    assert got.size == int(g[f"{key}__n"])
    sample = got if int(g["full"]) else got[:: int(g["stride"])]
    assert np.array_equal(bits(sample), bits(g[f"{key}__data"])), f"{key}: sampled bits differ"
    assert np.float64(got.astype(np.float64).sum()) == g[f"{key}__sum"], f"{key}: checksum differs"
    assert np.float64((got.astype(np.float64) ** 2).sum()) == g[f"{key}__sumsq"], f"{key}: checksum differs"


def test_golden_files_exist():
    assert len(GOLDEN) >= 6


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_reproduces_reference_vectors(pkg, oracle, path):
    g = np.load(path)
    M, K, N, ro, ci, vals, c, b, d = inputs_of(pkg, g)
    assert int(ci.size) == int(g["nnz"])
    assert digest(ro, ci, vals, c, b, d) == str(g["input_digest"]), "seeded inputs changed, not the oracle"
    s = oracle.sddmm(ro, ci, c, b, M, N)
    expect(g, "sddmm", s)                                                   # reference Sddmm
    expect(g, "spmm_f64acc", oracle.spmm_f64acc(vals, ro, ci, d, M, N))     # reference Spmm (double)
    expect(g, "spmm_f32", oracle.spmm(vals, ro, ci, d, M, N))               # reference SpmmEsimdCPU
    expect(g, "spmm_f32", oracle.spmm(vals, ro, ci, d, M, N, threads=4))    # threaded variant, same bits
    expect(g, "spmm_f32", oracle.spmm(vals, ro, ci, d, M, N, threads=4, fast_order=True))
    e, s2 = oracle.fused(ro, ci, c, b, d, M, N)
    expect(g, "unfused", e)                                                 # Sddmm -> Spmm
    assert np.array_equal(bits(s), bits(s2))
    e_mt, _ = oracle.fused(ro, ci, c, b, d, M, N, threads=3)
    expect(g, "unfused", e_mt)
    expect(g, "fused_order", oracle.fused_order(ro, ci, c, b, d, M, N))     # reference FusedEsimdCPU
    expect(g, "sddmm", oracle.sddmm(ro, ci, c, b, M, N, threads=5))


REF_SHAPES = [(64, 48, 32), (256, 256, 64), (512, 512, 32), (512, 512, 128)]


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("seed", [7, 8])
def test_oracle_equals_reference_object_code(pkg, oracle, shape, seed):
    M, K, N = shape
    if not oracle.ref_available(M, K, N):
        pytest.skip("oracle/_ref not built on this machine (needs the reference checkout)")
    ref = oracle.RefObject(M, K, N)
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.15 + 0.1 * (seed % 2), seed)
    assert (np.diff(ro) > 0).all()
    vals = pkg.gen_dense_host(int(ci.size), seed, 2)
    c = pkg.gen_dense_host(M * N, seed, 11).reshape(M, N)
    b = pkg.gen_dense_host(K * N, seed, 12).reshape(K, N)
    d = pkg.gen_dense_host(K * N, seed, 13).reshape(K, N)
    assert np.array_equal(bits(oracle.sddmm(ro, ci, c, b, M, N)), bits(ref.sddmm(ro, ci, c, b)))
    assert np.array_equal(bits(oracle.spmm_f64acc(vals, ro, ci, d, M, N)), bits(ref.spmm_f64acc(vals, ro, ci, d)))
    assert np.array_equal(bits(oracle.spmm(vals, ro, ci, d, M, N)), bits(ref.spmm_f32(vals, ro, ci, d)))
    assert np.array_equal(bits(oracle.fused_order(ro, ci, c, b, d, M, N)), bits(ref.fused_order(ro, ci, c, b, d)))
    e, _ = oracle.fused(ro, ci, c, b, d, M, N)
    assert np.array_equal(bits(e), bits(ref.spmm_f64acc(ref.sddmm(ro, ci, c, b), ro, ci, d)))


def test_oracle_spmm_matches_numpy_float64(pkg, oracle):
    """Independent check of the restated loops against dense float64 arithmetic."""
    M, K, N = 40, 30, 17
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.3, 5)
    vals = pkg.gen_dense_host(int(ci.size), 5, 2)
    B = pkg.gen_dense_host(K * N, 5, 10).reshape(K, N)
    A = np.zeros((M, K))
    for i in range(M):
        A[i, ci[ro[i]:ro[i + 1]]] = vals[ro[i]:ro[i + 1]]
    np.testing.assert_allclose(oracle.spmm(vals, ro, ci, B, M, N), A @ B.astype(np.float64), rtol=1e-5, atol=1e-5)
    lhs = pkg.gen_dense_host(M * N, 5, 11).reshape(M, N)
    rhs = pkg.gen_dense_host(K * N, 5, 12).reshape(K, N)
    full = lhs.astype(np.float64) @ rhs.astype(np.float64).T
    want = np.concatenate([full[i, ci[ro[i]:ro[i + 1]]] for i in range(M)])
    np.testing.assert_allclose(oracle.sddmm(ro, ci, lhs, rhs, M, N), want, rtol=1e-6, atol=1e-6)
    e, s = oracle.fused(ro, ci, lhs, rhs, B[:, :N] if False else rhs, M, N)
    S = np.zeros((M, K))
    for i in range(M):
        S[i, ci[ro[i]:ro[i + 1]]] = s[ro[i]:ro[i + 1]]
    np.testing.assert_allclose(e, S @ rhs.astype(np.float64), rtol=1e-5, atol=1e-5)


def test_oracle_attention_matches_numpy_float64(pkg, oracle):
    """The scale / row-softmax steps have no reference code; the restatement is checked against a
    dense float64 masked softmax."""
    M, K, N = 33, 41, 12
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.25, 8)
    ro = ro.copy()
    q = pkg.gen_dense_host(M * N, 8, 11).reshape(M, N).astype(np.float64)
    k = pkg.gen_dense_host(K * N, 8, 12).reshape(K, N).astype(np.float64)
    v = pkg.gen_dense_host(K * N, 8, 13).reshape(K, N).astype(np.float64)
    scores = 0.7 * (q @ k.T)
    mask = np.zeros((M, K), dtype=bool)
    for i in range(M):
        mask[i, ci[ro[i]:ro[i + 1]]] = True
    want_scaled = np.where(mask, scores, 0.0) @ v
    e = np.where(mask, np.exp(scores - np.where(mask, scores, -np.inf).max(axis=1, keepdims=True, initial=-1e300)), 0.0)
    denom = e.sum(axis=1, keepdims=True)
    want_soft = np.divide(e, denom, out=np.zeros_like(e), where=denom > 0) @ v
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    got, mag = oracle.attention(ro, ci, f32(q), f32(k), f32(v), M, N, 0.7, False)
    np.testing.assert_allclose(got, want_scaled, rtol=1e-5, atol=1e-5)
    got, mag = oracle.attention(ro, ci, f32(q), f32(k), f32(v), M, N, 0.7, True)
    np.testing.assert_allclose(got, want_soft, rtol=1e-5, atol=1e-5)
    assert (mag + 1e-6 >= np.abs(got)).all()
    for i in range(M):
        if ro[i] == ro[i + 1]:
            assert (got[i] == 0).all()


def test_violation_counter(oracle):
    ref = np.array([1.0, 0.0, 2.0, 0.0], dtype=np.float32)
    out = np.array([1.00005, 1e-6, 2.1, 0.0], dtype=np.float32)
    scale = np.array([1.0, 1.0, 2.0, 0.0], dtype=np.float32)
    bad, worst = oracle.violations(ref, out, scale, 1e-4)
    assert bad == 1 and 0.04 < worst < 0.06
    bad, _ = oracle.violations(ref, np.array([1.0, 0.0, 2.0, np.nan], dtype=np.float32), scale, 1e-4)
    assert bad == 1
