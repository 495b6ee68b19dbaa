"""Python access to the CPU oracle (oracle.c) and to the reference's own object code (_ref/).

TEST INFRASTRUCTURE ONLY: the test suite, the smoke check and the benchmark's CPU-baseline /
reference arm load this module to CHECK the CUDA library.  Nothing in the product package imports
it, and the product has no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(ORACLE_DIR, "liboracle.so")
REF_DIR = os.path.join(ORACLE_DIR, "_ref")

_lib: Optional[C.CDLL] = None
_P, _I, _LL, _D = C.c_void_p, C.c_int, C.c_longlong, C.c_double


def build(reference_dir: Optional[str] = None) -> None:
    """Compiles liboracle.so and, if a checkout of the reference is given, the _ref objects."""
    subprocess.run(["make", "-C", ORACLE_DIR, "all"], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if reference_dir and os.path.exists(os.path.join(reference_dir, "FUSED", "fused.cpp")):
        subprocess.run(["make", "-C", ORACLE_DIR, "ref", f"REF={reference_dir}"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        l = C.CDLL(LIB_PATH)
        l.oracle_spmm_f32.argtypes = [_P, _P, _P, _P, _P, _I, _I]
        l.oracle_spmm_f32_mt.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I]
        l.oracle_spmm_f32_rowmajor_mt.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I]
        l.oracle_spmm_f64acc.argtypes = [_P, _P, _P, _P, _P, _I, _I]
        l.oracle_sddmm.argtypes = [_P, _P, _P, _P, _P, _I, _I]
        l.oracle_sddmm_mt.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I]
        l.oracle_fused.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I]
        l.oracle_fused_mt.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I]
        l.oracle_attention.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I, C.c_float, _I]
        l.oracle_fused_order.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I]
        l.oracle_spmm_scale.argtypes = [_P, _P, _P, _P, _P, _I, _I]
        l.oracle_sddmm_scale.argtypes = [_P, _P, _P, _P, _P, _I, _I]
        l.oracle_fused_scale.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I, _I]
        l.oracle_sanity_check.argtypes = [_I, _I, _I, _I, _P, _P, C.c_char_p, C.c_size_t]
        l.oracle_sanity_check.restype = _I
        l.oracle_read_smtx.argtypes = [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I),
                                       C.POINTER(C.POINTER(_I)), C.POINTER(C.POINTER(_I))]
        l.oracle_read_smtx.restype = _I
        l.oracle_free.argtypes = [_P]
        l.oracle_checksum_rms.argtypes = [_P, _LL]
        l.oracle_checksum_rms.restype = _D
        l.oracle_validate.argtypes = [_P, _P, _LL, C.POINTER(_D), C.POINTER(_LL), C.POINTER(_D)]
        l.oracle_count_violations.argtypes = [_P, _P, _P, _LL, _D, C.POINTER(_D)]
        l.oracle_count_violations.restype = _LL
        l.oracle_max_threads.restype = _I
        _lib = l
    return _lib


class SpeedBuild:
    """The same oracle.c compiled for speed (-O3 -march=native) on the machine that runs it, for the
    benchmark's CPU baseline only; the parity checks always use the -O2 -ffp-contract=off build."""

    def __init__(self):
        import shutil
        import tempfile

        cc = shutil.which("gcc")
        if cc is None:
            raise RuntimeError("no gcc on this machine")
        self._dir = tempfile.mkdtemp(prefix="oracle_speed_")
        path = os.path.join(self._dir, "liboracle_speed.so")
        subprocess.run([cc, "-O3", "-march=native", "-fPIC", "-pthread", "-std=gnu11", "-shared", "-o", path,
                        os.path.join(ORACLE_DIR, "oracle.c"), "-lm"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
        self._lib = C.CDLL(path)
        self._lib.oracle_spmm_f32_mt.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I]

    def spmm(self, values, row_offsets, cols, B, M, N, threads: int) -> np.ndarray:
        values, row_offsets, cols, B = _f32(values), _i32(row_offsets), _i32(cols), _f32(B)
        out = np.zeros((M, N), dtype=np.float32)
        self._lib.oracle_spmm_f32_mt(_p(values), _p(row_offsets), _p(cols), _p(B), _p(out), M, N, threads)
        return out


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a: np.ndarray):
    return a.ctypes.data if a.size else None


def max_threads() -> int:
    return lib().oracle_max_threads()


def spmm(values, row_offsets, cols, B, M, N, threads: int = 1, fast_order: bool = False) -> np.ndarray:
    """fp32-accumulating CPU SpMM (the reference's host loop)."""
    values, row_offsets, cols, B = _f32(values), _i32(row_offsets), _i32(cols), _f32(B)
    out = np.zeros((M, N), dtype=np.float32)
    if fast_order:
        lib().oracle_spmm_f32_rowmajor_mt(_p(values), _p(row_offsets), _p(cols), _p(B), _p(out), M, N, threads)
    elif threads > 1:
        lib().oracle_spmm_f32_mt(_p(values), _p(row_offsets), _p(cols), _p(B), _p(out), M, N, threads)
    else:
        lib().oracle_spmm_f32(_p(values), _p(row_offsets), _p(cols), _p(B), _p(out), M, N)
    return out


def spmm_f64acc(values, row_offsets, cols, D, M, N) -> np.ndarray:
    values, row_offsets, cols, D = _f32(values), _i32(row_offsets), _i32(cols), _f32(D)
    out = np.zeros((M, N), dtype=np.float32)
    lib().oracle_spmm_f64acc(_p(values), _p(row_offsets), _p(cols), _p(D), _p(out), M, N)
    return out


def sddmm(row_offsets, cols, lhs, rhs, M, N, threads: int = 1) -> np.ndarray:
    row_offsets, cols, lhs, rhs = _i32(row_offsets), _i32(cols), _f32(lhs), _f32(rhs)
    out = np.zeros(cols.size, dtype=np.float32)
    if threads > 1:
        lib().oracle_sddmm_mt(_p(row_offsets), _p(cols), _p(lhs), _p(rhs), _p(out), M, N, threads)
    else:
        lib().oracle_sddmm(_p(row_offsets), _p(cols), _p(lhs), _p(rhs), _p(out), M, N)
    return out


def fused(row_offsets, cols, c, b, d, M, N, threads: int = 1):
    """Unfused CPU reference of the fused kernel; returns (E, sddmm_values)."""
    row_offsets, cols, c, b, d = _i32(row_offsets), _i32(cols), _f32(c), _f32(b), _f32(d)
    e = np.zeros((M, N), dtype=np.float32)
    a = np.zeros(max(cols.size, 1), dtype=np.float32)
    if threads > 1:
        lib().oracle_fused_mt(_p(row_offsets), _p(cols), _p(c), _p(b), _p(d), _p(e), _p(a), M, N, threads)
    else:
        lib().oracle_fused(_p(row_offsets), _p(cols), _p(c), _p(b), _p(d), _p(e), _p(a), M, N)
    return e, a[: cols.size]


def attention(row_offsets, cols, q, k, v, M, N, scale: float, softmax: bool):
    """Double-precision sparse attention (scale, optional row softmax); returns (O, magnitude)."""
    o = np.empty((M, N), dtype=np.float32)
    mag = np.empty((M, N), dtype=np.float32)
    lib().oracle_attention(_p(row_offsets), _p(cols), _p(q), _p(k), _p(v), _p(o), _p(mag), M, N,
                           C.c_float(scale), int(bool(softmax)))
    return o, mag


def fused_order(row_offsets, cols, c, b, d, M, N) -> np.ndarray:
    row_offsets, cols, c, b, d = _i32(row_offsets), _i32(cols), _f32(c), _f32(b), _f32(d)
    e = np.zeros((M, N), dtype=np.float32)
    lib().oracle_fused_order(_p(row_offsets), _p(cols), _p(c), _p(b), _p(d), _p(e), M, N)
    return e


def spmm_scale(values, row_offsets, cols, B, M, N, threads: int = 1) -> np.ndarray:
    """Sum of |products| behind every output element (the magnitude term of the tolerance).  With
    threads > 1 it is formed as the fp32 product of |A| and |B| on all threads, which is accurate to
    a few ulp: more than enough for a magnitude."""
    values, row_offsets, cols, B = _f32(values), _i32(row_offsets), _i32(cols), _f32(B)
    if threads > 1:
        return spmm(np.abs(values), row_offsets, cols, np.abs(B), M, N, threads=threads, fast_order=True)
    out = np.zeros((M, N), dtype=np.float32)
    lib().oracle_spmm_scale(_p(values), _p(row_offsets), _p(cols), _p(B), _p(out), M, N)
    return out


def sddmm_scale(row_offsets, cols, lhs, rhs, M, N) -> np.ndarray:
    row_offsets, cols, lhs, rhs = _i32(row_offsets), _i32(cols), _f32(lhs), _f32(rhs)
    out = np.zeros(cols.size, dtype=np.float32)
    lib().oracle_sddmm_scale(_p(row_offsets), _p(cols), _p(lhs), _p(rhs), _p(out), M, N)
    return out


def fused_scale(row_offsets, cols, c, b, d, M, N) -> np.ndarray:
    row_offsets, cols, c, b, d = _i32(row_offsets), _i32(cols), _f32(c), _f32(b), _f32(d)
    out = np.zeros((M, N), dtype=np.float32)
    tmp = np.zeros(max(cols.size, 1), dtype=np.float32)
    lib().oracle_fused_scale(_p(row_offsets), _p(cols), _p(c), _p(b), _p(d), _p(out), _p(tmp), M, N)
    return out


def sanity_check(M, K, N, nnz, row_offsets, cols):
    """Returns (code, reason): 0 = passes, otherwise the number of the failing reference check."""
    row_offsets, cols = _i32(row_offsets), _i32(cols)
    why = C.create_string_buffer(128)
    code = lib().oracle_sanity_check(M, K, N, nnz, _p(row_offsets), _p(cols), why, 128)
    return code, why.value.decode()


def read_smtx(path: str):
    M, K, nnz = _I(), _I(), _I()
    ro, ci = C.POINTER(_I)(), C.POINTER(_I)()
    rc = lib().oracle_read_smtx(path.encode(), C.byref(M), C.byref(K), C.byref(nnz), C.byref(ro), C.byref(ci))
    if rc:
        raise RuntimeError(f"oracle_read_smtx({path}) failed with code {rc}")
    try:
        row_offsets = np.ctypeslib.as_array(ro, shape=(M.value + 1,)).copy()
        cols = np.ctypeslib.as_array(ci, shape=(max(nnz.value, 1),))[: nnz.value].copy()
    finally:
        lib().oracle_free(ro)
        lib().oracle_free(ci)
    return M.value, K.value, nnz.value, row_offsets, cols


def checksum_rms(x) -> float:
    x = _f32(x).ravel()
    return lib().oracle_checksum_rms(_p(x), x.size)


def validate(gold, x):
    """Returns (max_abs_diff, index, max_rel_diff) as the reference drivers report them."""
    gold, x = _f32(gold).ravel(), _f32(x).ravel()
    md, mi, mr = _D(), _LL(), _D()
    lib().oracle_validate(_p(gold), _p(x), gold.size, C.byref(md), C.byref(mi), C.byref(mr))
    return md.value, mi.value, mr.value


def violations(ref, out, scale, tol: float):
    """Elements with |out-ref| > tol*max(|ref|, scale); returns (count, worst_ratio)."""
    ref, out, scale = _f32(ref).ravel(), _f32(out).ravel(), _f32(scale).ravel()
    assert ref.size == out.size == scale.size
    worst = _D()
    n = lib().oracle_count_violations(_p(ref), _p(out), _p(scale), ref.size, tol, C.byref(worst))
    return n, worst.value


# ---- the reference's own object code (FUSED/fused.cpp compiled unchanged, one .so per shape) ---------

class RefObject:
    """Functions of the reference's plain-C++ file for one compile-time (M, K, N)."""

    def __init__(self, M: int, K: int, N: int):
        path = os.path.join(REF_DIR, f"libfused_ref_{M}_{K}_{N}.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.M, self.K, self.N = M, K, N
        so = C.CDLL(path)
        # C++ symbols (Itanium mangling) of Sddmm, Spmm, FusedEsimdCPU, SpmmEsimdCPU
        self._sddmm = so._Z5SddmmPKiS0_PKfS2_Pf
        self._spmm = so._Z4SpmmPKfPKiS2_S0_Pf
        self._fused_cpu = so._Z13FusedEsimdCPUPKiS0_PKfS2_S2_Pf
        self._spmm_cpu = so._Z12SpmmEsimdCPUPKfPKiS2_S0_Pf
        for f, n in ((self._sddmm, 5), (self._spmm, 5), (self._fused_cpu, 6), (self._spmm_cpu, 5)):
            f.argtypes = [_P] * n
            f.restype = None

    def sddmm(self, row_offsets, cols, c, b) -> np.ndarray:
        row_offsets, cols, c, b = _i32(row_offsets), _i32(cols), _f32(c), _f32(b)
        out = np.zeros(cols.size, dtype=np.float32)
        self._sddmm(_p(row_offsets), _p(cols), _p(c), _p(b), _p(out))
        return out

    def spmm_f64acc(self, values, row_offsets, cols, d) -> np.ndarray:
        values, row_offsets, cols, d = _f32(values), _i32(row_offsets), _i32(cols), _f32(d)
        out = np.zeros((self.M, self.N), dtype=np.float32)
        self._spmm(_p(values), _p(row_offsets), _p(cols), _p(d), _p(out))
        return out

    def spmm_f32(self, values, row_offsets, cols, d) -> np.ndarray:
        """SpmmEsimdCPU: fp32 accumulation in CSR order."""
        values, row_offsets, cols, d = _f32(values), _i32(row_offsets), _i32(cols), _f32(d)
        out = np.zeros((self.M, self.N), dtype=np.float32)
        self._spmm_cpu(_p(values), _p(row_offsets), _p(cols), _p(d), _p(out))
        return out

    def fused_order(self, row_offsets, cols, c, b, d) -> np.ndarray:
        row_offsets, cols, c, b, d = _i32(row_offsets), _i32(cols), _f32(c), _f32(b), _f32(d)
        out = np.zeros((self.M, self.N), dtype=np.float32)
        self._fused_cpu(_p(row_offsets), _p(cols), _p(c), _p(b), _p(d), _p(out))
        return out


def ref_available(M: int, K: int, N: int) -> bool:
    return os.path.exists(os.path.join(REF_DIR, f"libfused_ref_{M}_{K}_{N}.so"))
