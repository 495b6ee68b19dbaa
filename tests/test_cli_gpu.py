"""The command-line drivers (the reference's `./app <file>.smtx <N>` programs): report lines, CSV
columns and the printed CPU-vs-GPU difference."""
import os
import re
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(pkg, name, *args):
    exe = os.path.join(pkg.PKG_DIR, "bin", name)
    assert os.path.exists(exe), f"{exe} not built"
    p = subprocess.run([exe, *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert p.returncode == 0, p.stdout
    return p.stdout


def _value(text, pattern):
    m = re.search(pattern, text)
    assert m, f"{pattern!r} not found in:\n{text}"
    return float(m.group(1))


def test_spmm_fromfile(pkg, tmp_path):
    ro, ci = pkg.gen_bernoulli_csr_host(300, 200, 0.1, 5)
    smtx = str(tmp_path / "a.smtx")
    csv = str(tmp_path / "out.csv")
    pkg.write_smtx(smtx, 300, 200, ro, ci)
    out = _run(pkg, "spmm-fromfile", smtx, 64, "--csv", csv)
    assert f"MSZ: 300, KSZ: 200, NSZ: 64, nnz: {ci.size}" in out
    assert "Total kernel time was" in out and "GFLOPS:" in out
    # inputs in [0,1): outputs of order nnz/row * 0.25, differences at rounding level
    assert _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-4
    cpu, gpu = _value(out, r"checksum_cpu = ([0-9.e+-]+)"), _value(out, r"checksum_gpu = ([0-9.e+-]+)")
    assert abs(cpu - gpu) <= 1e-5 * cpu
    row = open(csv).read().strip().split(",")
    assert len(row) == 7 and [int(row[0]), int(row[1]), int(row[2])] == [300, 64, 200]  # M,N,K,density,gflops,max_diff,opcount
    # planned and signed variants give a report as well
    out = _run(pkg, "spmm-fromfile", smtx, 100, "--planned", "--signed", "--cold")
    assert "cold-L2 median ms" in out and _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-4
    assert _value(out, r"plan \(rows binned by length\) created in ([0-9.e+-]+) ms") > 0
    # per-launch time from 100 launches captured in one CUDA graph (what counts for kernels of a few us)
    out = _run(pkg, "spmm-fromfile", smtx, 64, "--graph")
    assert 0 < _value(out, r"graph of 100 launches: ([0-9.e+-]+) ms per launch") < 1.0
    assert _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-4


def test_spmm_fromfile_cache_and_file_values(pkg, tmp_path):
    """--cache writes a binary copy on the first run and reads it on the second; a values block in
    the file replaces the generated values (same report either way)."""
    ro, ci = pkg.gen_bernoulli_csr_host(200, 150, 0.1, 8)
    vals = pkg.gen_dense_host(int(ci.size), 8, 2)
    smtx = str(tmp_path / "v.smtx")
    pkg.write_smtx_values(smtx, 200, 150, ro, ci, vals)
    first = _run(pkg, "spmm-fromfile", smtx, 32, "--cache")
    assert f"wrote {smtx}.csrbin" in first and os.path.exists(smtx + ".csrbin")
    second = _run(pkg, "spmm-fromfile", smtx, 32, "--cache")
    assert f"read {smtx}.csrbin" in second
    plain = str(tmp_path / "p.smtx")
    pkg.write_smtx(plain, 200, 150, ro, ci)
    generated = _run(pkg, "spmm-fromfile", plain, 32)
    sums = [_value(o, r"checksum_gpu = ([0-9.e+-]+)") for o in (first, second, generated)]
    assert sums[0] == sums[1] and sums[0] != sums[2]
    for o in (first, second):
        assert _value(o, r"max_diff = ([0-9.e+-]+)") < 1e-4
    M, K, nnz, ro2, ci2, v2 = pkg.read_csr_cache(smtx + ".csrbin")
    assert np.array_equal(ci2, ci) and np.array_equal(v2.view(np.uint32), vals.view(np.uint32))


def test_spmm_fromfile_errors(pkg, tmp_path):
    out = _run(pkg, "spmm-fromfile")
    assert "Usage: ./app <filename>.smtx <batchsize>" in out
    exe = os.path.join(pkg.PKG_DIR, "bin", "spmm-fromfile")
    p = subprocess.run([exe, str(tmp_path / "missing.smtx"), "16"], stdout=subprocess.PIPE, text=True)
    assert "Error opening file!" in p.stdout
    bad = tmp_path / "bad.smtx"
    bad.write_text("2, 2, 2\n0 1 2\n0 5\n")
    p = subprocess.run([exe, str(bad), "16"], stdout=subprocess.PIPE, text=True)
    assert "a_column_indices[i] >= KSZ" in p.stdout


def test_sddmm_fromfile_and_fused(pkg, tmp_path):
    ro, ci = pkg.gen_bernoulli_csr_host(256, 128, 0.2, 6)
    smtx = str(tmp_path / "b.smtx")
    csv = str(tmp_path / "s.csv")
    pkg.write_smtx(smtx, 256, 128, ro, ci)
    out = _run(pkg, "sddmm-fromfile", smtx, 128, "--csv", csv)
    assert "GFLOPS :" in out and _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-3
    row = open(csv).read().strip().split(",")
    assert len(row) == 7 and [int(row[0]), int(row[1]), int(row[2])] == [256, 128, 128]  # M,K,N,density,gflops,flops,max_diff
    out = _run(pkg, "fused", 512, 512, 32, 0.1, "--graph")
    assert "GFLOPS/s :" in out and "checksum_e using gpu" in out and "graph of 100 launches" in out
    assert _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-7
    out = _run(pkg, "fused", 256, 256, 64, 0.05, "--band", 8)
    assert _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-7
    out = _run(pkg, "fused", 256, 256, 64, 0.05, "--band", 8, "--signed", "--scale", 2000, "--softmax")
    assert _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-7
    assert _value(out, r"checksum_e using gpu = ([0-9.e+-]+)") > 0


def test_sweep_drivers_single_case(pkg):
    out = _run(pkg, "spmm-allbenchs", 1024, 1024, 32, 0.1)
    assert "GFLOPS:" in out and _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-4
    out = _run(pkg, "sddmm-allbench", 1024, 1024, 32, 0.1)
    assert "GFLOPS :" in out and _value(out, r"max_diff = ([0-9.e+-]+)") < 1e-4


def test_batch_scripts_walk_a_tree_in_one_process(pkg, tmp_path):
    """batch-run-*_fromfile over a small DLMC-style tree: one driver process runs every file of the
    tree (--list), widths come from the "<name>,<N>" table, the host check covers a sample of the
    rows (--check-rows), and the CSV has one row per file."""
    tree = tmp_path / "dlmc" / "rn50" / "magnitude_pruning"
    names = ["layer_a", "layer_b", "layer_c"]
    for sp in ("0.5", "0.9"):
        (tree / sp).mkdir(parents=True)
        for i, n in enumerate(names):
            ro, ci = pkg.gen_bernoulli_csr_host(128 + 64 * i, 96, 1.0 - float(sp), 20 + i)
            pkg.write_smtx(str(tree / sp / f"{n}.smtx"), 128 + 64 * i, 96, ro, ci)
    table = tmp_path / "widths.txt"
    table.write_text("layer_a,64\nlayer_b,49\nlayer_c,256\n")
    for op, cols in (("spmm", 7), ("sddmm", 7)):
        script = os.path.join(pkg.PKG_DIR, "cli", f"batch-run-{op}_fromfile")
        p = subprocess.run(["bash", script, str(tmp_path / "dlmc" / "rn50"), str(table), "--check-rows", "16"],
                           cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
        assert p.returncode == 0, p.stdout
        csvs = [f for f in os.listdir(tmp_path) if f.startswith(f"{op}-fromfile_") and f.endswith(".csv")]
        reports = [f for f in os.listdir(tmp_path) if f.startswith(f"summary-perf-{op}-")]
        assert len(csvs) == 1 and len(reports) == 1
        rows = [r.split(",") for r in open(tmp_path / csvs[0]).read().strip().splitlines()]
        assert len(rows) == 6 and all(len(r) == cols for r in rows)
        text = open(tmp_path / reports[0]).read()
        assert text.count("Filename = ") == 6 and "host check on every" in text
        for m in re.finditer(r"max_diff = ([0-9.e+-]+)", text):
            assert float(m.group(1)) < 1e-3
    # a table with the single line "*,<N>" gives every file that width
    table.write_text("*,32\n")
    script = os.path.join(pkg.PKG_DIR, "cli", "batch-run-spmm_fromfile")
    p = subprocess.run(["bash", script, str(tmp_path / "dlmc" / "rn50"), str(table), "--no-check"], cwd=tmp_path,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout
    report = [f for f in os.listdir(tmp_path) if f.startswith("summary-perf-spmm-")][0]
    assert open(tmp_path / report).read().count("NSZ: 32") == 6
