"""ctypes binding of libdlspm.so (the sm_100a CSR SpMM / SDDMM / fused SDDMM->SpMM library).

This package is plumbing for the tests and the benchmark: it loads the C-ABI shared library that
`include/dlspm.h` declares and passes device pointers of torch tensors (or host pointers of numpy
arrays) straight through.  There is no Python or CPU implementation of any kernel here; if the
shared library is missing, `load_library()` raises.

The directory name contains a hyphen, so it is imported through `importlib` under the module name
``dlspm_esimd_b200`` (see `__graft_entry__.load_package`).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libdlspm.so")
HEADER_PATH = os.path.join(os.path.dirname(PKG_DIR), "include", "dlspm.h")

OK = 0
(ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_IO, ERR_FORMAT, ERR_CSR, ERR_NOMEM, ERR_UNSUPPORTED, ERR_NO_DEVICE,
 ERR_TIMEOUT) = range(1, 10)
OPT_STRICT_FP32, OPT_SPMM_KERNEL, OPT_TILE_MIN_DENSITY, OPT_CHECK_INPUT = 0, 1, 2, 3
SPMM_KERNEL_AUTO, SPMM_KERNEL_GATHER, SPMM_KERNEL_TILED, SPMM_KERNEL_TILED_DENSE = 0, 1, 2, 3
ATTN_SOFTMAX = 1
KIND_UNIFORM_PM1, KIND_UNIFORM_01, KIND_NORMAL = 0, 1, 2


class DlspmError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status} ({strerror(status)}){' - ' + detail if detail else ''}")


class Problem(C.Structure):
    """Mirror of `dlspm_problem`."""

    _fields_ = [
        ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("nnz", C.c_int),
        ("values", C.c_void_p), ("row_offsets", C.c_void_p), ("column_indices", C.c_void_p),
        ("B", C.c_void_p), ("C", C.c_void_p),
    ]


class SddmmProblem(C.Structure):
    """Mirror of `dlspm_sddmm_problem`."""

    _fields_ = [
        ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("nnz", C.c_int),
        ("row_offsets", C.c_void_p), ("column_indices", C.c_void_p), ("mask_values", C.c_void_p),
        ("lhs", C.c_void_p), ("rhs", C.c_void_p), ("out_values", C.c_void_p),
    ]


class FusedProblem(C.Structure):
    """Mirror of `dlspm_fused_problem`."""

    _fields_ = [
        ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("nnz", C.c_int),
        ("row_offsets", C.c_void_p), ("column_indices", C.c_void_p),
        ("C", C.c_void_p), ("B", C.c_void_p), ("D", C.c_void_p), ("E", C.c_void_p),
    ]


_lib: Optional[C.CDLL] = None

_P = C.c_void_p
_I = C.c_int
_SIGNATURES = {
    "dlspm_create": (_I, [C.POINTER(_P), _I]),
    "dlspm_destroy": (_I, [_P]),
    "dlspm_strerror": (C.c_char_p, [_I]),
    "dlspm_last_error": (C.c_char_p, [_P]),
    "dlspm_device_info": (_I, [_P, C.c_char_p, C.c_size_t, C.POINTER(_I), C.POINTER(C.c_size_t)]),
    "dlspm_set_option": (_I, [_P, _I, _I]),
    "dlspm_get_option": (_I, [_P, _I, C.POINTER(_I)]),
    "dlspm_spmm_csr_f32": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "dlspm_spmm_csr_f32_planned": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, _P]),
    "dlspm_sddmm_csr_f32": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "dlspm_sddmm_csr_masked_f32": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "dlspm_fused_sddmm_spmm_f32": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "dlspm_fused_attention_f32": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, C.c_float, C.c_uint, _P]),
    "dlspm_plan_create": (_I, [_P, _I, _I, _I, _P, _P, _P, C.POINTER(_P)]),
    "dlspm_plan_destroy": (_I, [_P]),
    "dlspm_plan_row_order": (_I, [_P, _P, _P]),
    "dlspm_spmm_batched_f32": (_I, [_P, _I, C.POINTER(Problem), _P]),
    "dlspm_sddmm_batched_f32": (_I, [_P, _I, C.POINTER(SddmmProblem), _P]),
    "dlspm_fused_batched_f32": (_I, [_P, _I, C.POINTER(FusedProblem), _P]),
    "dlspm_sddmm_batched_f32_host": (_I, [_P, _I, C.POINTER(SddmmProblem)]),
    "dlspm_fused_batched_f32_host": (_I, [_P, _I, C.POINTER(FusedProblem)]),
    "dlspm_spmm_batched_f32_static": (_I, [_P, _I, C.POINTER(Problem), _P]),
    "dlspm_batch_create": (_I, [_P, _I, C.POINTER(Problem), C.POINTER(_P)]),
    "dlspm_batch_launch": (_I, [_P, _P, _P]),
    "dlspm_batch_launch_part": (_I, [_P, _P, _I, _P]),
    "dlspm_batch_info": (_I, [_P, _P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(C.c_double)]),
    "dlspm_batch_destroy": (_I, [_P]),
    "dlspm_spmm_csr_f32_host": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "dlspm_sddmm_csr_f32_host": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "dlspm_fused_sddmm_spmm_f32_host": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "dlspm_spmm_batched_f32_host": (_I, [_P, _I, C.POINTER(Problem)]),
    "dlspm_read_smtx_host": (_I, [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I),
                                  C.POINTER(C.POINTER(_I)), C.POINTER(C.POINTER(_I))]),
    "dlspm_write_smtx_host": (_I, [C.c_char_p, _I, _I, _I, _P, _P]),
    "dlspm_read_smtx_values_host": (_I, [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I),
                                         C.POINTER(C.POINTER(_I)), C.POINTER(C.POINTER(_I)),
                                         C.POINTER(C.POINTER(C.c_float))]),
    "dlspm_write_smtx_values_host": (_I, [C.c_char_p, _I, _I, _I, _P, _P, _P]),
    "dlspm_read_csr_cache_host": (_I, [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I),
                                       C.POINTER(C.POINTER(_I)), C.POINTER(C.POINTER(_I)),
                                       C.POINTER(C.POINTER(C.c_float))]),
    "dlspm_write_csr_cache_host": (_I, [C.c_char_p, _I, _I, _I, _P, _P, _P]),
    "dlspm_free_host": (None, [_P]),
    "dlspm_sanity_check_csr_host": (_I, [_I, _I, _I, _I, _P, _P, C.c_char_p, C.c_size_t]),
    "dlspm_rand_u64": (C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint64]),
    "dlspm_gen_dense_host": (_I, [_P, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, _I]),
    "dlspm_gen_dense": (_I, [_P, _P, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, _I, _P]),
    "dlspm_gen_bernoulli_csr_host": (_I, [_I, _I, C.c_double, C.c_uint64, _P, _P, C.c_size_t, C.POINTER(_I)]),
    "dlspm_gen_rowlen_normal_host": (_I, [_I, _I, C.c_double, C.c_double, C.c_uint64, _P]),
    "dlspm_gen_sample_columns_host": (_I, [_I, _I, _P, C.c_uint64, _P]),
    "dlspm_gen_sample_columns": (_I, [_P, _I, _I, _P, C.c_uint64, _P, _P]),
    "dlspm_gen_band_csr_host": (_I, [_I, _I, _I, C.c_double, C.c_uint64, _P, _P, C.c_size_t, C.POINTER(_I)]),
    "dlspm_gen_bernoulli_count": (_I, [_P, _I, _I, _I, C.c_double, C.c_uint64, _P, _P]),
    "dlspm_gen_bernoulli_fill": (_I, [_P, _I, _I, _I, C.c_double, C.c_uint64, _P, _P, _P]),
    "dlspm_partition_lpt_host": (_I, [_I, _P, _I, _P]),
    "dlspm_partition_rows_by_nnz_host": (_I, [_I, _P, _I, _P]),
    "dlspm_mg_create": (_I, [C.POINTER(_P), _I, _P]),
    "dlspm_mg_destroy": (_I, [_P]),
    "dlspm_mg_device_count": (_I, [_P]),
    "dlspm_mg_spmm_batched_f32_host": (_I, [_P, _I, C.POINTER(Problem)]),
    "dlspm_mg_spmm_rowshard_f32_host": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "dlspm_measure_fp32_peak": (_I, [_P, C.POINTER(C.c_double)]),
    "dlspm_measure_fp32_peaks": (_I, [_P, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "dlspm_host_copy_count": (_I, [_P, C.POINTER(C.c_longlong)]),
    "dlspm_sanity_check_csr": (_I, [_P, _I, _I, _I, _P, _P, C.c_char_p, C.c_size_t, _P]),
    "dlspm_selftest_bounded_wait": (_I, [_P, C.c_uint, C.POINTER(_I)]),
    "dlspm_spmm_csr_f32_scatter": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _I, C.POINTER(_P), C.c_longlong, _P]),
    "dlspm_enable_peer_access": (_I, [_P, _I]),
    "dlspm_peer_alloc": (_I, [_P, C.c_size_t, C.POINTER(_P), C.c_char_p]),
    "dlspm_peer_open": (_I, [_P, C.c_char_p, C.POINTER(_P)]),
    "dlspm_peer_close": (_I, [_P, _P]),
    "dlspm_peer_free": (_I, [_P, _P]),
}


def exported_names() -> Sequence[str]:
    """Names this binding expects the shared library to export."""
    return tuple(_SIGNATURES)


def build(verbose: bool = False) -> None:
    """Compiles libdlspm.so and the drivers in-tree with nvcc for sm_100a (no GPU needed)."""
    cmd = ["make", "-C", PKG_DIR, "-j", str(os.cpu_count() or 4), "all"]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        print(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("building libdlspm.so failed")


def load_library() -> C.CDLL:
    """Loads libdlspm.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C {PKG_DIR}` (no fallback exists)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def strerror(status: int) -> str:
    return load_library().dlspm_strerror(status).decode()


def _check(status: int, what: str, ctx: "Optional[Context]" = None) -> None:
    if status != OK:
        detail = ""
        if ctx is not None and ctx.handle:
            detail = load_library().dlspm_last_error(ctx.handle).decode()
        raise DlspmError(status, what, detail)


# ---- pointer helpers -----------------------------------------------------------------------------

def _dev_ptr(t, dtype, what: str) -> Optional[int]:
    """Device pointer of a contiguous CUDA torch tensor of the given dtype (None passes NULL)."""
    if t is None:
        return None
    import torch

    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{what}: expected a CUDA torch tensor")
    if t.dtype != dtype or not t.is_contiguous():
        raise TypeError(f"{what}: expected contiguous {dtype}, got {t.dtype} contiguous={t.is_contiguous()}")
    return t.data_ptr() if t.numel() else None


def _host_ptr(a, dtype, what: str) -> Optional[int]:
    """Host pointer of a C-contiguous numpy array or CPU torch tensor (pinned or not)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        if a.dtype != dtype or not a.flags["C_CONTIGUOUS"]:
            raise TypeError(f"{what}: expected C-contiguous {dtype}, got {a.dtype}")
        return a.ctypes.data if a.size else None
    import torch

    if isinstance(a, torch.Tensor) and not a.is_cuda:
        want = {np.float32: torch.float32, np.int32: torch.int32, np.float64: torch.float64}[dtype]
        if a.dtype != want or not a.is_contiguous():
            raise TypeError(f"{what}: expected contiguous {want}")
        return a.data_ptr() if a.numel() else None
    raise TypeError(f"{what}: expected a numpy array or CPU tensor")


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream or None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


# ---- context ----------------------------------------------------------------------------------------

class Context:
    """One `dlspm_ctx` (one device)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        self.handle = _P()
        self.device = device
        _check(self.lib.dlspm_create(C.byref(self.handle), device), "dlspm_create")

    def close(self) -> None:
        if self.handle:
            self.lib.dlspm_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def device_info(self):
        name = C.create_string_buffer(256)
        sms = _I()
        mem = C.c_size_t()
        _check(self.lib.dlspm_device_info(self.handle, name, 256, C.byref(sms), C.byref(mem)), "dlspm_device_info")
        return name.value.decode(), sms.value, mem.value

    def set_option(self, option: int, value: int) -> None:
        _check(self.lib.dlspm_set_option(self.handle, option, value), "dlspm_set_option")

    def get_option(self, option: int) -> int:
        v = _I()
        _check(self.lib.dlspm_get_option(self.handle, option, C.byref(v)), "dlspm_get_option")
        return v.value

    # device-pointer entry points (torch CUDA tensors)
    def spmm(self, M, K, N, nnz, values, row_offsets, column_indices, B, Cout, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_spmm_csr_f32(
            self.handle, M, K, N, nnz, _dev_ptr(values, torch.float32, "values"),
            _dev_ptr(row_offsets, torch.int32, "row_offsets"), _dev_ptr(column_indices, torch.int32, "column_indices"),
            _dev_ptr(B, torch.float32, "B"), _dev_ptr(Cout, torch.float32, "C"), _stream_ptr(stream)),
            "dlspm_spmm_csr_f32", self)

    def sddmm(self, M, K, N, nnz, row_offsets, column_indices, lhs, rhs, out, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_sddmm_csr_f32(
            self.handle, M, K, N, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"), _dev_ptr(lhs, torch.float32, "lhs"),
            _dev_ptr(rhs, torch.float32, "rhs"), _dev_ptr(out, torch.float32, "out"), _stream_ptr(stream)),
            "dlspm_sddmm_csr_f32", self)

    def sddmm_masked(self, M, K, N, nnz, row_offsets, column_indices, mask_values, lhs, rhs, out, stream=None) -> None:
        """out[p] = mask_values[p] * dot(lhs[i], rhs[col_p]); mask_values None means 1."""
        import torch

        _check(self.lib.dlspm_sddmm_csr_masked_f32(
            self.handle, M, K, N, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"),
            _dev_ptr(mask_values, torch.float32, "mask_values") if mask_values is not None else None,
            _dev_ptr(lhs, torch.float32, "lhs"), _dev_ptr(rhs, torch.float32, "rhs"),
            _dev_ptr(out, torch.float32, "out"), _stream_ptr(stream)), "dlspm_sddmm_csr_masked_f32", self)

    def fused(self, M, K, N, nnz, row_offsets, column_indices, Cq, Bk, Dv, Eo, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_fused_sddmm_spmm_f32(
            self.handle, M, K, N, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"), _dev_ptr(Cq, torch.float32, "C"),
            _dev_ptr(Bk, torch.float32, "B"), _dev_ptr(Dv, torch.float32, "D"), _dev_ptr(Eo, torch.float32, "E"),
            _stream_ptr(stream)), "dlspm_fused_sddmm_spmm_f32", self)

    def attention(self, M, K, N, nnz, row_offsets, column_indices, Q, Kmat, V, O, scale=1.0, flags=0,
                  stream=None) -> None:
        """O = softmax_rows(scale * pattern .* (Q Kmat^T)) V (flags=ATTN_SOFTMAX) or the scaled chain."""
        import torch

        _check(self.lib.dlspm_fused_attention_f32(
            self.handle, M, K, N, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"), _dev_ptr(Q, torch.float32, "Q"),
            _dev_ptr(Kmat, torch.float32, "Kmat"), _dev_ptr(V, torch.float32, "V"), _dev_ptr(O, torch.float32, "O"),
            float(scale), int(flags), _stream_ptr(stream)), "dlspm_fused_attention_f32", self)

    def plan_create(self, M, K, nnz, row_offsets, column_indices, stream=None) -> "Plan":
        import torch

        h = _P()
        _check(self.lib.dlspm_plan_create(
            self.handle, M, K, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"), _stream_ptr(stream), C.byref(h)),
            "dlspm_plan_create", self)
        return Plan(self, h, M)

    def spmm_planned(self, plan, N, values, row_offsets, column_indices, B, Cout, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_spmm_csr_f32_planned(
            self.handle, plan.handle, N, _dev_ptr(values, torch.float32, "values"),
            _dev_ptr(row_offsets, torch.int32, "row_offsets"), _dev_ptr(column_indices, torch.int32, "column_indices"),
            _dev_ptr(B, torch.float32, "B"), _dev_ptr(Cout, torch.float32, "C"), _stream_ptr(stream)),
            "dlspm_spmm_csr_f32_planned", self)

    def spmm_batched(self, problems: "ProblemArray", stream=None) -> None:
        _check(self.lib.dlspm_spmm_batched_f32(self.handle, len(problems), problems.array, _stream_ptr(stream)),
               "dlspm_spmm_batched_f32", self)

    def spmm_batched_static(self, problems: "ProblemArray", stream=None) -> None:
        """Grouped launch that allocates nothing (tables in a fixed device array, <= 1024 problems)."""
        _check(self.lib.dlspm_spmm_batched_f32_static(self.handle, len(problems), problems.array,
                                                      _stream_ptr(stream)),
               "dlspm_spmm_batched_f32_static", self)

    def sddmm_batched(self, problems: "RowProblemArray", stream=None) -> None:
        _check(self.lib.dlspm_sddmm_batched_f32(self.handle, len(problems), problems.array, _stream_ptr(stream)),
               "dlspm_sddmm_batched_f32", self)

    def fused_batched(self, problems: "RowProblemArray", stream=None) -> None:
        _check(self.lib.dlspm_fused_batched_f32(self.handle, len(problems), problems.array, _stream_ptr(stream)),
               "dlspm_fused_batched_f32", self)

    def sddmm_batched_host(self, problems: "RowProblemArray") -> None:
        _check(self.lib.dlspm_sddmm_batched_f32_host(self.handle, len(problems), problems.array),
               "dlspm_sddmm_batched_f32_host", self)

    def fused_batched_host(self, problems: "RowProblemArray") -> None:
        _check(self.lib.dlspm_fused_batched_f32_host(self.handle, len(problems), problems.array),
               "dlspm_fused_batched_f32_host", self)

    def batch_create(self, problems: "ProblemArray") -> "Batch":
        h = _P()
        _check(self.lib.dlspm_batch_create(self.handle, len(problems), problems.array, C.byref(h)),
               "dlspm_batch_create", self)
        return Batch(self, h, problems)

    # host-pointer entry points (numpy arrays or CPU tensors, pinned or pageable)
    def spmm_host(self, M, K, N, nnz, values, row_offsets, column_indices, B, Cout) -> None:
        _check(self.lib.dlspm_spmm_csr_f32_host(
            self.handle, M, K, N, nnz, _host_ptr(values, np.float32, "values"),
            _host_ptr(row_offsets, np.int32, "row_offsets"), _host_ptr(column_indices, np.int32, "column_indices"),
            _host_ptr(B, np.float32, "B"), _host_ptr(Cout, np.float32, "C")), "dlspm_spmm_csr_f32_host", self)

    def sddmm_host(self, M, K, N, nnz, row_offsets, column_indices, lhs, rhs, out) -> None:
        _check(self.lib.dlspm_sddmm_csr_f32_host(
            self.handle, M, K, N, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
            _host_ptr(column_indices, np.int32, "column_indices"), _host_ptr(lhs, np.float32, "lhs"),
            _host_ptr(rhs, np.float32, "rhs"), _host_ptr(out, np.float32, "out")), "dlspm_sddmm_csr_f32_host", self)

    def fused_host(self, M, K, N, nnz, row_offsets, column_indices, Cq, Bk, Dv, Eo) -> None:
        _check(self.lib.dlspm_fused_sddmm_spmm_f32_host(
            self.handle, M, K, N, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
            _host_ptr(column_indices, np.int32, "column_indices"), _host_ptr(Cq, np.float32, "C"),
            _host_ptr(Bk, np.float32, "B"), _host_ptr(Dv, np.float32, "D"), _host_ptr(Eo, np.float32, "E")),
            "dlspm_fused_sddmm_spmm_f32_host", self)

    def spmm_batched_host(self, problems: "ProblemArray") -> None:
        _check(self.lib.dlspm_spmm_batched_f32_host(self.handle, len(problems), problems.array),
               "dlspm_spmm_batched_f32_host", self)

    def measure_fp32_peaks(self):
        """(TFLOP/s with scalar FMAs, TFLOP/s with packed two-wide FMAs)."""
        a, b = C.c_double(), C.c_double()
        _check(self.lib.dlspm_measure_fp32_peaks(self.handle, C.byref(a), C.byref(b)), "dlspm_measure_fp32_peaks", self)
        return a.value, b.value

    def sanity_check_csr(self, M, K, nnz, row_offsets, column_indices, stream=None):
        """Device-side CSR validation: (status, reason)."""
        import torch

        why = C.create_string_buffer(256)
        st = self.lib.dlspm_sanity_check_csr(self.handle, M, K, nnz, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
                                             _dev_ptr(column_indices, torch.int32, "column_indices"), why, 256,
                                             _stream_ptr(stream))
        return st, why.value.decode()

    def host_copy_count(self) -> int:
        """cudaMemcpyAsync calls issued so far by spmm_batched_host on this context."""
        v = C.c_longlong()
        _check(self.lib.dlspm_host_copy_count(self.handle, C.byref(v)), "dlspm_host_copy_count", self)
        return v.value

    # device generators
    def gen_dense(self, out, seed, stream_id, first_index=0, kind=KIND_UNIFORM_PM1, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_gen_dense(self.handle, _dev_ptr(out, torch.float32, "out"), out.numel(), seed,
                                        stream_id, first_index, kind, _stream_ptr(stream)), "dlspm_gen_dense", self)

    def gen_sample_columns(self, M, K, row_offsets, seed, column_indices, stream=None) -> None:
        import torch

        _check(self.lib.dlspm_gen_sample_columns(
            self.handle, M, K, _dev_ptr(row_offsets, torch.int32, "row_offsets"), seed,
            _dev_ptr(column_indices, torch.int32, "column_indices"), _stream_ptr(stream)),
            "dlspm_gen_sample_columns", self)

    def gen_bernoulli_count(self, M, K, density, seed, counts, stream=None, first_row=0) -> None:
        import torch

        _check(self.lib.dlspm_gen_bernoulli_count(self.handle, M, K, first_row, density, seed,
                                                  _dev_ptr(counts, torch.int32, "counts"), _stream_ptr(stream)),
               "dlspm_gen_bernoulli_count", self)

    def gen_bernoulli_fill(self, M, K, density, seed, row_offsets, column_indices, stream=None, first_row=0) -> None:
        import torch

        _check(self.lib.dlspm_gen_bernoulli_fill(
            self.handle, M, K, first_row, density, seed, _dev_ptr(row_offsets, torch.int32, "row_offsets"),
            _dev_ptr(column_indices, torch.int32, "column_indices"), _stream_ptr(stream)),
            "dlspm_gen_bernoulli_fill", self)

    # fused SpMM + gather over peer memory
    def spmm_scatter(self, M, K, N, nnz, values, row_offsets, column_indices, B, dst_ptrs, first_row, stream=None):
        """dst_ptrs: integer device addresses of the full-size C buffers (local first, then peers)."""
        import torch

        arr = (_P * len(dst_ptrs))(*dst_ptrs)
        _check(self.lib.dlspm_spmm_csr_f32_scatter(
            self.handle, M, K, N, nnz, _dev_ptr(values, torch.float32, "values"),
            _dev_ptr(row_offsets, torch.int32, "row_offsets"), _dev_ptr(column_indices, torch.int32, "column_indices"),
            _dev_ptr(B, torch.float32, "B"), len(dst_ptrs), arr, first_row, _stream_ptr(stream)),
            "dlspm_spmm_csr_f32_scatter", self)

    def enable_peer_access(self, peer_device: int) -> None:
        _check(self.lib.dlspm_enable_peer_access(self.handle, peer_device), "dlspm_enable_peer_access", self)

    def peer_alloc(self, nbytes: int):
        """Returns (device address, 64-byte IPC handle)."""
        ptr = _P()
        handle = C.create_string_buffer(64)
        _check(self.lib.dlspm_peer_alloc(self.handle, nbytes, C.byref(ptr), handle), "dlspm_peer_alloc", self)
        return ptr.value, handle.raw

    def peer_open(self, handle: bytes) -> int:
        ptr = _P()
        _check(self.lib.dlspm_peer_open(self.handle, handle, C.byref(ptr)), "dlspm_peer_open", self)
        return ptr.value

    def peer_close(self, ptr: int) -> None:
        _check(self.lib.dlspm_peer_close(self.handle, ptr), "dlspm_peer_close", self)

    def peer_free(self, ptr: int) -> None:
        _check(self.lib.dlspm_peer_free(self.handle, ptr), "dlspm_peer_free", self)

    def selftest_bounded_wait(self, polls: int = 1000):
        """(status, timed_out) of the bounded-wait self-test; the context stays usable afterwards."""
        t = _I()
        st = self.lib.dlspm_selftest_bounded_wait(self.handle, polls, C.byref(t))
        return st, t.value

    def measure_fp32_peak(self) -> float:
        v = C.c_double()
        _check(self.lib.dlspm_measure_fp32_peak(self.handle, C.byref(v)), "dlspm_measure_fp32_peak", self)
        return v.value


class DeviceArray:
    """Zero-copy torch view of a raw device allocation (through __cuda_array_interface__)."""

    def __init__(self, ptr: int, shape, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}

    def tensor(self, device):
        import torch

        return torch.as_tensor(self, device=device)


class Plan:
    def __init__(self, ctx: Context, handle, M: int = 0):
        self.ctx, self.handle, self.M = ctx, handle, M

    def row_order(self, stream=None) -> np.ndarray:
        """The plan's row order as a host array (dlspm_plan_row_order)."""
        out = np.empty(self.M, dtype=np.int32)
        if self.M:
            _check(self.ctx.lib.dlspm_plan_row_order(self.handle, out.ctypes.data_as(_P), _stream_ptr(stream)),
                   "dlspm_plan_row_order", self.ctx)
        return out

    def close(self) -> None:
        if self.handle:
            self.ctx.lib.dlspm_plan_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ProblemArray:
    """A host array of `dlspm_problem`; keeps the tensors it points to alive."""

    def __init__(self, n: int):
        self.array = (Problem * max(n, 1))()
        self.n = n
        self.keep = []

    def __len__(self) -> int:
        return self.n

    def set(self, i, M, K, N, nnz, values, row_offsets, column_indices, B, Cout, host=False) -> None:
        p = self.array[i]
        p.M, p.K, p.N, p.nnz = M, K, N, nnz
        if host:
            p.values = _host_ptr(values, np.float32, "values")
            p.row_offsets = _host_ptr(row_offsets, np.int32, "row_offsets")
            p.column_indices = _host_ptr(column_indices, np.int32, "column_indices")
            p.B = _host_ptr(B, np.float32, "B")
            p.C = _host_ptr(Cout, np.float32, "C")
        else:
            import torch

            p.values = _dev_ptr(values, torch.float32, "values")
            p.row_offsets = _dev_ptr(row_offsets, torch.int32, "row_offsets")
            p.column_indices = _dev_ptr(column_indices, torch.int32, "column_indices")
            p.B = _dev_ptr(B, torch.float32, "B")
            p.C = _dev_ptr(Cout, torch.float32, "C")
        self.keep.append((values, row_offsets, column_indices, B, Cout))

    def set_raw(self, i, M, K, N, nnz, values, row_offsets, column_indices, B, Cout) -> None:
        """Raw integer addresses (the caller keeps the memory alive)."""
        p = self.array[i]
        p.M, p.K, p.N, p.nnz = M, K, N, nnz
        p.values, p.row_offsets, p.column_indices, p.B, p.C = values, row_offsets, column_indices, B, Cout


class RowProblemArray:
    """A host array of `dlspm_sddmm_problem` (kind "sddmm") or `dlspm_fused_problem` (kind "fused");
    keeps the arrays it points to alive.  `host=True`: numpy / CPU tensors instead of CUDA tensors."""

    def __init__(self, kind: str, n: int, host: bool = False):
        assert kind in ("sddmm", "fused")
        self.kind, self.n, self.host = kind, n, host
        self.array = ((SddmmProblem if kind == "sddmm" else FusedProblem) * max(n, 1))()
        self.keep = []

    def __len__(self) -> int:
        return self.n

    def _ptr(self, a, dtype_np, what):
        if self.host:
            return _host_ptr(a, dtype_np, what)
        import torch

        return _dev_ptr(a, torch.int32 if dtype_np == np.int32 else torch.float32, what)

    def set_sddmm(self, i, M, K, N, nnz, row_offsets, column_indices, lhs, rhs, out_values, mask_values=None) -> None:
        p = self.array[i]
        p.M, p.K, p.N, p.nnz = M, K, N, nnz
        p.row_offsets = self._ptr(row_offsets, np.int32, "row_offsets")
        p.column_indices = self._ptr(column_indices, np.int32, "column_indices")
        p.mask_values = self._ptr(mask_values, np.float32, "mask_values")
        p.lhs = self._ptr(lhs, np.float32, "lhs")
        p.rhs = self._ptr(rhs, np.float32, "rhs")
        p.out_values = self._ptr(out_values, np.float32, "out_values")
        self.keep.append((row_offsets, column_indices, mask_values, lhs, rhs, out_values))

    def set_fused(self, i, M, K, N, nnz, row_offsets, column_indices, Cq, Bk, Dv, Eo) -> None:
        p = self.array[i]
        p.M, p.K, p.N, p.nnz = M, K, N, nnz
        p.row_offsets = self._ptr(row_offsets, np.int32, "row_offsets")
        p.column_indices = self._ptr(column_indices, np.int32, "column_indices")
        p.C = self._ptr(Cq, np.float32, "C")
        p.B = self._ptr(Bk, np.float32, "B")
        p.D = self._ptr(Dv, np.float32, "D")
        p.E = self._ptr(Eo, np.float32, "E")
        self.keep.append((row_offsets, column_indices, Cq, Bk, Dv, Eo))


class Batch:
    def __init__(self, ctx: Context, handle, problems: ProblemArray):
        self.ctx, self.handle, self.problems = ctx, handle, problems

    def launch(self, stream=None) -> None:
        _check(self.ctx.lib.dlspm_batch_launch(self.ctx.handle, self.handle, _stream_ptr(stream)),
               "dlspm_batch_launch", self.ctx)

    def info(self, check_device: bool = False):
        """(problems on the row-gather kernel, problems on the tiled kernel, device error word or None)."""
        g, t, e = _I(), _I(), _I()
        self.stats = (C.c_double * 4)()
        _check(self.ctx.lib.dlspm_batch_info(self.ctx.handle, self.handle, C.byref(g), C.byref(t),
                                             C.byref(e) if check_device else None, self.stats),
               "dlspm_batch_info", self.ctx)
        return g.value, t.value, (e.value if check_device else None)

    def launch_part(self, part: int, stream=None) -> None:
        """1 = row-gather problems only, 2 = tiled problems only, 0 = all."""
        _check(self.ctx.lib.dlspm_batch_launch_part(self.ctx.handle, self.handle, part, _stream_ptr(stream)),
               "dlspm_batch_launch_part", self.ctx)

    def close(self) -> None:
        if self.handle:
            self.ctx.lib.dlspm_batch_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultiGpu:
    """One host process driving several devices (`dlspm_mg`)."""

    def __init__(self, devices: Sequence[int]):
        self.lib = load_library()
        self.handle = _P()
        arr = (C.c_int * len(devices))(*devices)
        _check(self.lib.dlspm_mg_create(C.byref(self.handle), len(devices), arr), "dlspm_mg_create")

    def device_count(self) -> int:
        return self.lib.dlspm_mg_device_count(self.handle)

    def spmm_batched_host(self, problems: ProblemArray) -> None:
        _check(self.lib.dlspm_mg_spmm_batched_f32_host(self.handle, len(problems), problems.array),
               "dlspm_mg_spmm_batched_f32_host")

    def spmm_rowshard_host(self, M, K, N, nnz, values, row_offsets, column_indices, B, Cout) -> None:
        _check(self.lib.dlspm_mg_spmm_rowshard_f32_host(
            self.handle, M, K, N, nnz, _host_ptr(values, np.float32, "values"),
            _host_ptr(row_offsets, np.int32, "row_offsets"), _host_ptr(column_indices, np.int32, "column_indices"),
            _host_ptr(B, np.float32, "B"), _host_ptr(Cout, np.float32, "C")), "dlspm_mg_spmm_rowshard_f32_host")

    def close(self) -> None:
        if self.handle:
            self.lib.dlspm_mg_destroy(self.handle)
            self.handle = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- host utilities (no GPU needed) ------------------------------------------------------------------

def read_smtx(path: str):
    """Returns (M, K, nnz, row_offsets, column_indices) as numpy int32 arrays."""
    lib = load_library()
    M, K, nnz = _I(), _I(), _I()
    ro, ci = C.POINTER(_I)(), C.POINTER(_I)()
    _check(lib.dlspm_read_smtx_host(path.encode(), C.byref(M), C.byref(K), C.byref(nnz), C.byref(ro), C.byref(ci)),
           f"dlspm_read_smtx_host({path})")
    try:
        row_offsets = np.ctypeslib.as_array(ro, shape=(M.value + 1,)).copy()
        cols = np.ctypeslib.as_array(ci, shape=(max(nnz.value, 1),))[: nnz.value].copy()
    finally:
        lib.dlspm_free_host(ro)
        lib.dlspm_free_host(ci)
    return M.value, K.value, nnz.value, row_offsets, cols


def write_smtx(path: str, M: int, K: int, row_offsets: np.ndarray, column_indices: np.ndarray) -> None:
    lib = load_library()
    nnz = int(column_indices.size)
    _check(lib.dlspm_write_smtx_host(path.encode(), M, K, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
                                     _host_ptr(column_indices, np.int32, "column_indices")), "dlspm_write_smtx_host")


def _read_with_values(fn_name: str, path: str):
    lib = load_library()
    M, K, nnz = _I(), _I(), _I()
    ro, ci, va = C.POINTER(_I)(), C.POINTER(_I)(), C.POINTER(C.c_float)()
    _check(getattr(lib, fn_name)(path.encode(), C.byref(M), C.byref(K), C.byref(nnz), C.byref(ro), C.byref(ci),
                                 C.byref(va)), f"{fn_name}({path})")
    try:
        row_offsets = np.ctypeslib.as_array(ro, shape=(M.value + 1,)).copy()
        cols = np.ctypeslib.as_array(ci, shape=(max(nnz.value, 1),))[: nnz.value].copy()
        values = np.ctypeslib.as_array(va, shape=(max(nnz.value, 1),))[: nnz.value].copy() if va else None
    finally:
        lib.dlspm_free_host(ro)
        lib.dlspm_free_host(ci)
        if va:
            lib.dlspm_free_host(va)
    return M.value, K.value, nnz.value, row_offsets, cols, values


def read_smtx_values(path: str):
    """Text format with the optional fourth block: (M, K, nnz, row_offsets, column_indices, values or None)."""
    return _read_with_values("dlspm_read_smtx_values_host", path)


def write_smtx_values(path: str, M: int, K: int, row_offsets, column_indices, values) -> None:
    lib = load_library()
    nnz = int(column_indices.size)
    _check(lib.dlspm_write_smtx_values_host(
        path.encode(), M, K, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
        _host_ptr(column_indices, np.int32, "column_indices"), _host_ptr(values, np.float32, "values")),
        "dlspm_write_smtx_values_host")


def read_csr_cache(path: str):
    """Binary cache: (M, K, nnz, row_offsets, column_indices, values or None)."""
    return _read_with_values("dlspm_read_csr_cache_host", path)


def write_csr_cache(path: str, M: int, K: int, row_offsets, column_indices, values=None) -> None:
    lib = load_library()
    nnz = int(column_indices.size)
    _check(lib.dlspm_write_csr_cache_host(
        path.encode(), M, K, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
        _host_ptr(column_indices, np.int32, "column_indices"),
        _host_ptr(values, np.float32, "values") if values is not None else None), "dlspm_write_csr_cache_host")


def sanity_check(M, K, N, nnz, row_offsets, column_indices):
    """Returns (status, reason)."""
    lib = load_library()
    why = C.create_string_buffer(128)
    st = lib.dlspm_sanity_check_csr_host(M, K, N, nnz, _host_ptr(row_offsets, np.int32, "row_offsets"),
                                         _host_ptr(column_indices, np.int32, "column_indices"), why, 128)
    return st, why.value.decode()


def rand_u64(seed: int, stream: int, index: int) -> int:
    return load_library().dlspm_rand_u64(seed, stream, index)


def gen_dense_host(n: int, seed: int, stream: int, first_index: int = 0, kind: int = KIND_UNIFORM_PM1) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    _check(load_library().dlspm_gen_dense_host(_host_ptr(out, np.float32, "out"), n, seed, stream, first_index, kind),
           "dlspm_gen_dense_host")
    return out


def gen_bernoulli_csr_host(M: int, K: int, density: float, seed: int):
    cap = int(M * K * min(1.0, density * 1.25 + 0.01)) + 1024
    cap = min(cap, M * K) if M * K > 0 else 1
    ro = np.zeros(M + 1, dtype=np.int32)
    ci = np.empty(max(cap, 1), dtype=np.int32)
    nnz = _I()
    _check(load_library().dlspm_gen_bernoulli_csr_host(M, K, density, seed, ro.ctypes.data, ci.ctypes.data, cap,
                                                       C.byref(nnz)), "dlspm_gen_bernoulli_csr_host")
    return ro, ci[: nnz.value].copy()


def gen_band_csr_host(M: int, K: int, half_band: int, extra_density: float, seed: int):
    cap = min(M * K, int(M * (2 * half_band + 1 + K * (extra_density * 1.25 + 0.01))) + 1024)
    ro = np.zeros(M + 1, dtype=np.int32)
    ci = np.empty(max(cap, 1), dtype=np.int32)
    nnz = _I()
    _check(load_library().dlspm_gen_band_csr_host(M, K, half_band, extra_density, seed, ro.ctypes.data,
                                                  ci.ctypes.data, cap, C.byref(nnz)), "dlspm_gen_band_csr_host")
    return ro, ci[: nnz.value].copy()


def gen_rowlen_normal_host(M: int, K: int, sparsity: float, cov: float, seed: int) -> np.ndarray:
    ro = np.zeros(M + 1, dtype=np.int32)
    _check(load_library().dlspm_gen_rowlen_normal_host(M, K, sparsity, cov, seed, ro.ctypes.data),
           "dlspm_gen_rowlen_normal_host")
    return ro


def gen_sample_columns_host(M: int, K: int, row_offsets: np.ndarray, seed: int) -> np.ndarray:
    ci = np.empty(max(int(row_offsets[M]), 1), dtype=np.int32)
    _check(load_library().dlspm_gen_sample_columns_host(M, K, _host_ptr(row_offsets, np.int32, "row_offsets"), seed,
                                                        ci.ctypes.data), "dlspm_gen_sample_columns_host")
    return ci[: int(row_offsets[M])].copy()


def partition_lpt(weights: np.ndarray, parts: int) -> np.ndarray:
    w = np.ascontiguousarray(weights, dtype=np.float64)
    owner = np.zeros(max(w.size, 1), dtype=np.int32)
    _check(load_library().dlspm_partition_lpt_host(int(w.size), w.ctypes.data if w.size else None, parts,
                                                   owner.ctypes.data), "dlspm_partition_lpt_host")
    return owner[: w.size]


def partition_rows_by_nnz(row_offsets: np.ndarray, parts: int) -> np.ndarray:
    M = int(row_offsets.size) - 1
    bounds = np.zeros(parts + 1, dtype=np.int32)
    _check(load_library().dlspm_partition_rows_by_nnz_host(M, _host_ptr(row_offsets, np.int32, "row_offsets"), parts,
                                                           bounds.ctypes.data), "dlspm_partition_rows_by_nnz_host")
    return bounds
