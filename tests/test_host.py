"""CPU-only tests of the host side of the library: ABI surface, .smtx reader, CSR validation,
seeded generators and the partitioners.  No kernel is launched."""
import glob
import os
import re

import numpy as np
import pytest


# ---- ABI surface -----------------------------------------------------------------------------------

def declared_functions(header_path):
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dlspm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    import ctypes

    names = declared_functions(pkg.HEADER_PATH)
    assert len(names) >= 40
    lib = ctypes.CDLL(pkg.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in dlspm.h but not exported: {missing}"
    # and the Python binding covers the same set
    assert sorted(pkg.exported_names()) == names


def test_python_constants_match_the_header(pkg):
    """Option numbers and status codes of the ctypes binding are the header's."""
    text = open(pkg.HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    enums = {name: int(value) for name, value in re.findall(r"\b(DLSPM_[A-Z0-9_]+)\s*=\s*(-?\d+)", text)}
    options = {k: v for k, v in enums.items() if k.startswith("DLSPM_OPT_")}
    assert len(options) == 4
    for name, value in options.items():
        assert getattr(pkg, name[len("DLSPM_"):]) == value, name
    for name, value in enums.items():
        if name.startswith("DLSPM_ERR_") or name == "DLSPM_OK":
            assert getattr(pkg, name[len("DLSPM_"):]) == value, name


def test_strerror_and_no_device_failure(pkg):
    assert pkg.strerror(pkg.OK) == "ok"
    assert pkg.strerror(pkg.ERR_IO) == "Error opening file!"  # the reference's exception text
    import torch

    if not torch.cuda.is_available():
        # there is no CPU fallback: creating a context without a GPU must fail loudly
        with pytest.raises(pkg.DlspmError) as e:
            pkg.Context(0)
        assert e.value.status == pkg.ERR_NO_DEVICE


# ---- .smtx reader ------------------------------------------------------------------------------------

def test_smtx_round_trip(pkg, oracle, tmp_path):
    ro, ci = pkg.gen_bernoulli_csr_host(37, 53, 0.2, 3)
    p = str(tmp_path / "a.smtx")
    pkg.write_smtx(p, 37, 53, ro, ci)
    M, K, nnz, ro2, ci2 = pkg.read_smtx(p)
    assert (M, K, nnz) == (37, 53, ci.size)
    assert np.array_equal(ro, ro2) and np.array_equal(ci, ci2)
    # the oracle reader (fscanf, as the reference) sees the same integers
    M3, K3, nnz3, ro3, ci3 = oracle.read_smtx(p)
    assert (M3, K3, nnz3) == (M, K, nnz) and np.array_equal(ro3, ro) and np.array_equal(ci3, ci)


def test_smtx_dataset_layout_and_whitespace(pkg, oracle, tmp_path):
    # the layout of the DLMC files: "M, K, nnz" then two long lines; also tabs / CRLF / no final newline
    texts = {
        "dlmc": "3, 4, 5\n0 2 2 5\n0 3 1 2 3\n",
        "crlf": "3, 4, 5\r\n0 2 2 5\r\n0 3 1 2 3\r\n",
        "tabs": "3,4,5\n0\t2\t2\t5\n0 3\n1 2 3",
        "multi": "3,\n4,\n5 0 2 2 5 0 3 1 2 3",
    }
    for name, text in texts.items():
        p = tmp_path / f"{name}.smtx"
        p.write_bytes(text.encode())
        M, K, nnz, ro, ci = pkg.read_smtx(str(p))
        assert (M, K, nnz) == (3, 4, 5), name
        assert ro.tolist() == [0, 2, 2, 5] and ci.tolist() == [0, 3, 1, 2, 3], name
        assert oracle.read_smtx(str(p))[3].tolist() == ro.tolist()


def test_smtx_empty_matrix(pkg, tmp_path):
    p = tmp_path / "e.smtx"
    p.write_text("2, 3, 0\n0 0 0\n\n")
    M, K, nnz, ro, ci = pkg.read_smtx(str(p))
    assert (M, K, nnz) == (2, 3, 0) and ro.tolist() == [0, 0, 0] and ci.size == 0


@pytest.mark.parametrize("text", ["", "3 4 5\n0 1 2 3\n", "3, 4\n", "2, 2, 2\n0 1\n", "2, 2, 2\n0 1 2\n0\n",
                                  "2, 2, x\n", "2, 2, 2\n0 1 2\n0 a\n", "-1, 2, 0\n0\n"])
def test_smtx_malformed(pkg, tmp_path, text):
    p = tmp_path / "bad.smtx"
    p.write_text(text)
    with pytest.raises(pkg.DlspmError) as e:
        pkg.read_smtx(str(p))
    assert e.value.status == pkg.ERR_FORMAT


def test_smtx_missing_file(pkg, tmp_path):
    with pytest.raises(pkg.DlspmError) as e:
        pkg.read_smtx(str(tmp_path / "nope.smtx"))
    assert e.value.status == pkg.ERR_IO


def test_smtx_with_values_round_trip(pkg, oracle, tmp_path):
    ro, ci = pkg.gen_bernoulli_csr_host(29, 41, 0.3, 5)
    vals = pkg.gen_dense_host(int(ci.size), 5, 2, kind=pkg.KIND_NORMAL)
    vals[:3] = [np.float32(1e-38), np.float32(-3.4e38), np.float32(1) / np.float32(3)]
    p = str(tmp_path / "v.smtx")
    pkg.write_smtx_values(p, 29, 41, ro, ci, vals)
    M, K, nnz, ro2, ci2, v2 = pkg.read_smtx_values(p)
    assert (M, K, nnz) == (29, 41, ci.size) and np.array_equal(ro, ro2) and np.array_equal(ci, ci2)
    assert np.array_equal(vals.view(np.uint32), v2.view(np.uint32))  # nine digits: every bit comes back
    # the plain readers (this library's and the fscanf one) take it as a pattern file
    assert np.array_equal(pkg.read_smtx(p)[4], ci)
    assert np.array_equal(oracle.read_smtx(p)[4], ci)
    # a plain file has no values
    q = str(tmp_path / "plain.smtx")
    pkg.write_smtx(q, 29, 41, ro, ci)
    assert pkg.read_smtx_values(q)[5] is None
    # a values block that is too short or not numeric is a format error
    for tail in ("0.5 0.25\n", "0.5 x\n"):
        bad = tmp_path / "short.smtx"
        bad.write_text("2, 2, 3\n0 1 3\n0 0 1\n" + tail)
        with pytest.raises(pkg.DlspmError) as e:
            pkg.read_smtx_values(str(bad))
        assert e.value.status == pkg.ERR_FORMAT


@pytest.mark.parametrize("with_values", [False, True])
def test_csr_cache_round_trip_and_corruption(pkg, tmp_path, with_values):
    M, K = 61, 47
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.15, 6)
    vals = pkg.gen_dense_host(int(ci.size), 6, 2) if with_values else None
    p = str(tmp_path / "m.csrbin")
    pkg.write_csr_cache(p, M, K, ro, ci, vals)
    M2, K2, nnz2, ro2, ci2, v2 = pkg.read_csr_cache(p)
    assert (M2, K2, nnz2) == (M, K, ci.size) and np.array_equal(ro, ro2) and np.array_equal(ci, ci2)
    assert (v2 is None) == (vals is None)
    if with_values:
        assert np.array_equal(vals.view(np.uint32), v2.view(np.uint32))
    blob = bytearray(open(p, "rb").read())
    assert len(blob) % 8 == 0 and blob[:8] == b"DLSPMCSR"

    def expect_format_error(data):
        bad = str(tmp_path / "bad.csrbin")
        open(bad, "wb").write(bytes(data))
        with pytest.raises(pkg.DlspmError) as e:
            pkg.read_csr_cache(bad)
        assert e.value.status == pkg.ERR_FORMAT

    flipped = bytearray(blob)
    flipped[48 + 4 * 7] ^= 0x10                      # one bit of a row offset
    expect_format_error(flipped)
    expect_format_error(blob[:-8])                   # truncated
    expect_format_error(blob + b"\0" * 8)            # trailing bytes
    expect_format_error(b"NOTACSR!" + bytes(blob[8:]))
    huge = bytearray(blob)
    huge[24:28] = (2**31 - 1).to_bytes(4, "little")  # nnz far beyond the file: rejected before allocation
    expect_format_error(huge)
    with pytest.raises(pkg.DlspmError) as e:
        pkg.read_csr_cache(str(tmp_path / "absent.csrbin"))
    assert e.value.status == pkg.ERR_IO


def test_csr_cache_empty_matrix(pkg, tmp_path):
    p = str(tmp_path / "e.csrbin")
    pkg.write_csr_cache(p, 3, 5, np.zeros(4, dtype=np.int32), np.zeros(0, dtype=np.int32))
    M, K, nnz, ro, ci, v = pkg.read_csr_cache(p)
    assert (M, K, nnz) == (3, 5, 0) and ro.tolist() == [0, 0, 0, 0] and ci.size == 0 and v is None


def test_reader_matches_fscanf_reader_on_dataset_files(pkg, oracle):
    """Bit-exact index handling on real pattern files, where the dataset checkout is present."""
    import __graft_entry__ as entry

    root = os.path.join(entry.REFERENCE_DIR, "dlmc")
    files = sorted(glob.glob(os.path.join(root, "rn50", "*", "*", "*.smtx")))
    files += sorted(glob.glob(os.path.join(root, "transformer", "*", "*", "*.smtx")))
    if not files:
        pytest.skip("pattern data set not present on this machine")
    files = [f for f in files if os.path.getsize(f) < 600_000]
    picks = files[:: max(1, len(files) // 40)][:40]
    empty_rows = 0
    for f in picks:
        a = pkg.read_smtx(f)
        b = oracle.read_smtx(f)
        assert a[:3] == b[:3]
        assert np.array_equal(a[3], b[3]) and np.array_equal(a[4], b[4])
        st, why = pkg.sanity_check(a[0], a[1], 16, a[2], a[3], a[4])
        assert st == pkg.OK, (f, why)
        empty_rows += int((np.diff(a[3]) == 0).sum())
    assert len(picks) >= 20


# ---- SanityCheck ---------------------------------------------------------------------------------------

def test_sanity_check_agrees_with_reference_texts(pkg, oracle):
    M, K = 4, 5
    good_ro = np.array([0, 2, 2, 4, 5], dtype=np.int32)
    good_ci = np.array([0, 4, 1, 2, 3], dtype=np.int32)
    cases = [
        (good_ro, good_ci, 5, ""),
        (np.array([0, 5, 10, 15, 21], np.int32), np.zeros(21, np.int32), 21, "nnz is larger than matrix."),
        (np.array([0, 2, 2, 4, 4], np.int32), good_ci, 5, "a_row_offsets[MSZ] != nnz."),
        (np.array([0, 3, 2, 4, 5], np.int32), good_ci, 5, "a_row_offsets[i+1] < a_row_offsets[i]"),
        (np.array([0, 0, 0, 0, 6], np.int32), np.zeros(6, np.int32), 6, "a_row_offsets[i + 1] - a_row_offsets[i] > KSZ"),
        (good_ro, np.array([0, 5, 1, 2, 3], np.int32), 5, "a_column_indices[i] >= KSZ"),
    ]
    for ro, ci, nnz, text in cases:
        st, why = pkg.sanity_check(M, K, 8, nnz, ro, ci)
        code, why_ref = oracle.sanity_check(M, K, 8, nnz, ro, ci)
        assert why == text == why_ref
        assert (st == pkg.OK) == (code == 0)
        assert st in (pkg.OK, pkg.ERR_CSR)
    # the two checks the reference leaves out
    st, why = pkg.sanity_check(M, K, 8, 5, good_ro, np.array([0, 4, -1, 2, 3], np.int32))
    assert st == pkg.ERR_CSR and why == "a_column_indices[i] < 0"
    st, why = pkg.sanity_check(2, 5, 8, 2, np.array([1, 1, 2], np.int32), np.array([0, 1], np.int32))
    assert st == pkg.ERR_CSR and why == "a_row_offsets[0] != 0"


# ---- generators ----------------------------------------------------------------------------------------

def test_counter_rng_is_deterministic_and_stream_separated(pkg):
    a = pkg.gen_dense_host(1000, 1, 2)
    assert np.array_equal(a, pkg.gen_dense_host(1000, 1, 2))
    assert np.array_equal(a[100:200], pkg.gen_dense_host(100, 1, 2, first_index=100))
    assert not np.array_equal(a, pkg.gen_dense_host(1000, 1, 3))
    assert not np.array_equal(a, pkg.gen_dense_host(1000, 2, 2))
    assert pkg.rand_u64(1, 2, 3) == pkg.rand_u64(1, 2, 3) != pkg.rand_u64(1, 2, 4)


def test_dense_distributions(pkg):
    n = 1 << 20
    u = pkg.gen_dense_host(n, 9, 1, kind=pkg.KIND_UNIFORM_PM1)
    assert u.min() >= -1.0 and u.max() < 1.0
    assert abs(u.mean()) < 4 * (1 / np.sqrt(3)) / np.sqrt(n) and abs(u.std() - 1 / np.sqrt(3)) < 2e-3
    v = pkg.gen_dense_host(n, 9, 1, kind=pkg.KIND_UNIFORM_01)
    assert v.min() >= 0.0 and v.max() < 1.0 and abs(v.mean() - 0.5) < 2e-3
    z = pkg.gen_dense_host(n, 9, 1, kind=pkg.KIND_NORMAL)
    assert abs(z.mean()) < 5 / np.sqrt(n) and abs(z.std() - 1.0) < 5e-3
    assert abs((np.abs(z) < 1).mean() - 0.6827) < 3e-3 and abs(((z ** 4).mean()) - 3.0) < 0.05


def test_bernoulli_pattern(pkg):
    M, K, p = 512, 512, 0.1
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, p, 1)
    assert pkg.sanity_check(M, K, 1, int(ci.size), ro, ci)[0] == pkg.OK
    lens = np.diff(ro)
    # Binomial(512, 0.1): mean 51.2, variance 46.1
    assert abs(lens.mean() - 51.2) < 1.0 and abs(lens.var() - 46.1) < 8.0
    for i in range(M):
        row = ci[ro[i]:ro[i + 1]]
        assert (np.diff(row) > 0).all()
    # column marginal is uniform
    hist = np.bincount(ci, minlength=K)
    assert abs(hist.mean() - 51.2) < 1.0 and hist.min() > 20 and hist.max() < 90
    assert pkg.gen_bernoulli_csr_host(8, 8, 0.0, 1)[1].size == 0
    assert pkg.gen_bernoulli_csr_host(8, 8, 1.0, 1)[1].size == 64


def test_rowlen_normal_and_sampled_columns(pkg):
    M, K, sp = 1024, 4096, 0.9
    ro = pkg.gen_rowlen_normal_host(M, K, sp, 0.4, 7)
    lens = np.diff(ro)
    mu = K * (1 - sp)
    assert lens.min() >= 0 and lens.max() <= K
    assert abs(lens.mean() - mu) < 0.05 * mu and abs(lens.std() / lens.mean() - 0.4) < 0.05
    ci = pkg.gen_sample_columns_host(M, K, ro, 7)
    assert ci.size == ro[-1]
    assert pkg.sanity_check(M, K, 1, int(ci.size), ro, ci)[0] == pkg.OK
    for i in range(0, M, 37):
        row = ci[ro[i]:ro[i + 1]]
        assert (np.diff(row) > 0).all() and (row >= 0).all() and (row < K).all()
    hist = np.bincount(ci, minlength=K)
    assert hist.min() > 0.5 * hist.mean() and hist.max() < 1.6 * hist.mean()
    # clipping: very sparse rows hit zero, dense rows hit K
    lens98 = np.diff(pkg.gen_rowlen_normal_host(4096, 64, 0.98, 0.4, 7))
    assert lens98.min() == 0 and (lens98 == 0).sum() > 0
    full = pkg.gen_rowlen_normal_host(16, 8, 0.0, 0.0, 7)
    assert (np.diff(full) == 8).all()
    assert pkg.gen_sample_columns_host(16, 8, full, 7).reshape(16, 8).tolist() == [list(range(8))] * 16


def test_band_pattern(pkg):
    M = K = 256
    ro, ci = pkg.gen_band_csr_host(M, K, 8, 0.05, 3)
    for i in (0, 5, 100, 255):
        row = set(ci[ro[i]:ro[i + 1]].tolist())
        assert set(range(max(0, i - 8), min(K, i + 9))) <= row
        assert (np.diff(ci[ro[i]:ro[i + 1]]) > 0).all()
    extra = ci.size - sum(min(K, i + 9) - max(0, i - 8) for i in range(M))
    assert 0.03 * M * K < extra < 0.07 * M * K


# ---- partitioners -----------------------------------------------------------------------------------------

@pytest.mark.parametrize("parts", [1, 2, 4, 8])
def test_lpt_partition(pkg, parts):
    rng = np.random.default_rng(parts)
    w = rng.pareto(1.5, 8192) + 0.01
    owner = pkg.partition_lpt(w, parts)
    assert owner.min() >= 0 and owner.max() < parts
    loads = np.bincount(owner, weights=w, minlength=parts)
    # greedy LPT bound: max load <= mean + largest item
    assert loads.max() <= w.sum() / parts + w.max() + 1e-9
    if parts > 1:
        assert loads.max() / loads.mean() < 1.02 or w.max() > 0.5 * loads.mean()
    assert np.array_equal(owner, pkg.partition_lpt(w, parts))  # deterministic
    # ties go to the lower index / lower part
    assert pkg.partition_lpt(np.ones(4), 2).tolist() == [0, 1, 0, 1]
    assert pkg.partition_lpt(np.array([5, 3, 3, 2, 2, 1.0]), 2).tolist() == [0, 1, 1, 0, 1, 0]
    assert pkg.partition_lpt(np.zeros(0), 3).size == 0


@pytest.mark.parametrize("parts", [1, 2, 4, 8])
def test_row_partition_by_nnz(pkg, parts):
    M, K = 4096, 512
    ro = pkg.gen_rowlen_normal_host(M, K, 0.9, 0.4, 11)
    bounds = pkg.partition_rows_by_nnz(ro, parts)
    assert bounds[0] == 0 and bounds[-1] == M and (np.diff(bounds) >= 0).all()
    per = np.diff(ro[bounds])
    assert per.sum() == ro[-1]
    assert per.max() - per.min() <= 2 * np.diff(ro).max()
    # skewed: all nonzeros in the last rows
    skew = np.zeros(101, dtype=np.int32)
    skew[91:] = np.arange(1, 11) * 1000
    b = pkg.partition_rows_by_nnz(skew, 4)
    assert b[0] == 0 and b[-1] == 100 and (np.diff(b) >= 0).all() and b[1] >= 90
    # no nonzeros: rows split evenly
    assert pkg.partition_rows_by_nnz(np.zeros(9, dtype=np.int32), 4).tolist() == [0, 2, 4, 6, 8]
