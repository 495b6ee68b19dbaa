"""Seeded test matrices built with the library's host generators (shared by CPU and GPU tests)."""
import numpy as np


def csr_bernoulli(pkg, M, K, density, seed):
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, density, seed)
    return ro, ci


def csr_rowlen_normal(pkg, M, K, sparsity, seed, cov=0.4):
    ro = pkg.gen_rowlen_normal_host(M, K, sparsity, cov, seed)
    ci = pkg.gen_sample_columns_host(M, K, ro, seed)
    return ro, ci


def csr_from_lengths(pkg, K, lengths, seed):
    """Rows with exactly the given lengths, columns sampled without replacement."""
    lengths = np.asarray(lengths, dtype=np.int64)
    ro = np.zeros(lengths.size + 1, dtype=np.int32)
    ro[1:] = np.cumsum(lengths)
    ci = pkg.gen_sample_columns_host(int(lengths.size), K, ro, seed)
    return ro, ci


def dense(pkg, rows, cols, seed, stream, kind=0):
    return pkg.gen_dense_host(rows * cols, seed, stream, kind=kind).reshape(rows, cols)


def spmm_case(pkg, M, K, N, density, seed, signed=True):
    ro, ci = csr_bernoulli(pkg, M, K, density, seed)
    vals = pkg.gen_dense_host(int(ci.size), seed, 2, kind=0 if signed else 1)
    B = dense(pkg, K, N, seed, 10, kind=0 if signed else 1)
    return ro, ci, vals, B


def shuffle_rows_columns(ro, ci, seed):
    """Same pattern with the entries of every row in a random (unsorted) order."""
    rng = np.random.default_rng(seed)
    out = ci.copy()
    for i in range(ro.size - 1):
        s, e = ro[i], ro[i + 1]
        out[s:e] = rng.permutation(out[s:e])
    return out
