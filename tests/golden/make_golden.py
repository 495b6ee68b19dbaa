"""Generates the golden vectors under tests/golden/ from the REFERENCE's own object code.

Run where a checkout of zubair23517/dlspm-esimd is available:

    python -c "import __graft_entry__ as g; g.build()"     # also compiles oracle/_ref/*.so
    python tests/golden/make_golden.py

Every expected value written here is produced by FUSED/fused.cpp of the reference, compiled
unchanged (see oracle/Makefile, target `ref`): Sddmm, Spmm (double accumulator), SpmmEsimdCPU (fp32,
CSR order) and FusedEsimdCPU.  Inputs come from the library's seeded host generators; a SHA-256
digest of the input bytes is stored so that a generator change is reported as such instead of as a
kernel mismatch.  Small cases store inputs and outputs in full, large ones a strided sample of the
output plus float64 checksums.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

# (name, M, K, N, pattern kind, pattern parameter, seed, value kind, store everything?)
CASES = [
    ("tiny_64x48_n32", 64, 48, 32, "bernoulli", 0.3, 101, 0, True),
    ("band_256x256_n64", 256, 256, 64, "band", (8, 0.05), 102, 2, False),
    ("cfg1_512x512_n128", 512, 512, 128, "bernoulli", 0.1, 1, 0, False),
    ("fused_512x512_n32", 512, 512, 32, "bernoulli", 0.1, 103, 1, False),
    ("cfg2_2048x512_n128", 2048, 512, 128, "bernoulli", 0.2, 2, 2, False),
    ("cfg4_4096x4096_n64", 4096, 4096, 64, "band", (32, 0.05), 4, 2, False),
]
STRIDE = 61  # sampled outputs keep every 61st element


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_inputs(pkg, M, K, N, kind, param, seed, vkind):
    if kind == "bernoulli":
        ro, ci = pkg.gen_bernoulli_csr_host(M, K, param, seed)
    else:
        ro, ci = pkg.gen_band_csr_host(M, K, param[0], param[1], seed)
    vals = pkg.gen_dense_host(int(ci.size), seed, 2, kind=vkind)
    c = pkg.gen_dense_host(M * N, seed, 11, kind=vkind).reshape(M, N)
    b = pkg.gen_dense_host(K * N, seed, 12, kind=vkind).reshape(K, N)
    d = pkg.gen_dense_host(K * N, seed, 13, kind=vkind).reshape(K, N)
    return ro, ci, vals, c, b, d


def summarize(x, full):
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = {"sum": np.float64(x.astype(np.float64).sum()), "sumsq": np.float64((x.astype(np.float64) ** 2).sum()),
           "n": np.int64(x.size)}
    out["data"] = x.copy() if full else x[::STRIDE].copy()
    return out


def main():
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    for name, M, K, N, kind, param, seed, vkind, full in CASES:
        if not oracle.ref_available(M, K, N):
            raise SystemExit(f"oracle/_ref has no object for {M}x{K}x{N}; run build() with the reference present")
        ref = oracle.RefObject(M, K, N)
        ro, ci, vals, c, b, d = make_inputs(pkg, M, K, N, kind, param, seed, vkind)
        assert (np.diff(ro) > 0).all(), "the reference's order-emulating loops misread empty rows"
        sddmm = ref.sddmm(ro, ci, c, b)
        outputs = {
            "sddmm": sddmm,                                    # Sddmm
            "spmm_f64acc": ref.spmm_f64acc(vals, ro, ci, d),   # Spmm on random values
            "spmm_f32": ref.spmm_f32(vals, ro, ci, d),         # SpmmEsimdCPU
            "unfused": ref.spmm_f64acc(sddmm, ro, ci, d),      # Sddmm -> Spmm, the fused oracle
            "fused_order": ref.fused_order(ro, ci, c, b, d),   # FusedEsimdCPU
        }
        blob = {"M": M, "K": K, "N": N, "seed": seed, "vkind": vkind, "full": int(full), "stride": STRIDE,
                "pattern_kind": kind, "pattern_param": np.atleast_1d(np.asarray(param, dtype=np.float64)),
                "input_digest": digest(ro, ci, vals, c, b, d), "nnz": int(ci.size)}
        if full:
            blob.update(row_offsets=ro, column_indices=ci, values=vals, c=c, b=b, d=d)
        for key, arr in outputs.items():
            for k2, v in summarize(arr, full).items():
                blob[f"{key}__{k2}"] = v
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **blob)
        print(f"{name}: nnz={ci.size} -> {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
