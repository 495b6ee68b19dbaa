"""Benchmark of the B200 sparse-kernel library on the reference's headline workload.

    python bench.py --gpus N --steps K --warmup W              # this library (CUDA kernels)
    python bench.py --impl reference --gpus N --steps K ...    # the reference's CPU loop, host cores
    torchrun --nproc-per-node N bench.py --gpus N ...          # one rank per GPU

Workload (`config.workload`): the batch of 8192 independent CSR SpMMs drawn from the shape /
sparsity / width grid of the sweep configuration (shapes 64x64 .. 1024x4096, sparsity 0.5 .. 0.98,
row lengths Normal with CoV 0.4, N in {256, 1024, 3136}), all matrices generated on the device from
a seed.  A step is one pass over the whole batch: one grouped launch per GPU.  With N GPUs the
problems are dealt out by nnz*N (longest-processing-time), so total work is fixed ("strong").
The metric is GFLOP/s = sum(2*nnz*N) / time.

One JSON line is printed by rank 0.  Besides the contract keys it carries `roofline` (algorithmic
bytes of rank 0's launch over its event-timed duration, against the measured HBM copy bandwidth),
`e2e` (the same metric through the host-buffer C-ABI call, copies included, on a stated sample of
the batch), `cpu_baseline` (the CPU oracle on the host cores, N=1 only) and `extras` (the other
configurations: single SpMM, SDDMM, fused, the 90 % sparsity sweep, the row-sharded large SpMM).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

SHAPES = [(64, 64), (256, 256), (512, 2048), (2048, 512), (1024, 4096)]
SPARSITIES = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]
WIDTHS = [256, 1024, 3136]
COV = 0.4
STREAM_PICK = 50
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per algorithmic byte of the two kernels of a step, from one ncu capture each on the
# first 256 problems of the batch (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic
# bytes of the problems the kernel served: 2.18 + 0.61 GB for 3.06 GB on the row-gather kernel, whose
# last results are still in L2 when it ends; 0.72 + 0.16 GB for 0.82 GB on the tiled kernel).  Traffic
# grows with the bytes of the problems processed, so the ratios are applied to the full launch.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {"spmm_batched_kernel": 0.913, "spmm_tile_kernel": 1.077}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def align(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


# ---- workload description ------------------------------------------------------------------------------

def batch_descriptors(pkg, count: int, seed: int):
    """(M, K, N, sparsity, problem_seed, row_offsets) for every problem of the batch."""
    out = []
    for k in range(count):
        h = pkg.rand_u64(seed, STREAM_PICK, k)
        M, K = SHAPES[h % 5]
        sp = SPARSITIES[(h >> 8) % 6]
        N = WIDTHS[(h >> 16) % 3]
        pseed = seed * (1 << 20) + k
        ro = pkg.gen_rowlen_normal_host(M, K, sp, COV, pseed)
        out.append((M, K, N, sp, pseed, ro))
    return out


def spmm_bytes(M, K, N, nnz):
    """Algorithmic bytes of one SpMM: A once, B once, C written once."""
    return 4 * (M + 1) + 8 * nnz + 4 * K * N + 4 * M * N


class DeviceBatch:
    """The problems of one rank, generated in two device pools (int32 and fp32)."""

    def __init__(self, pkg, ctx, dev, descs, mine):
        import torch

        self.pkg, self.ctx, self.dev = pkg, ctx, dev
        self.items = [descs[i] for i in mine]
        n_ro = n_int = n_flt = 0
        self.layout = []
        for (M, K, N, sp, pseed, ro) in self.items:
            nnz = int(ro[-1])
            o_ro = n_ro
            n_ro += align(M + 1)
            o_ci = n_int
            n_int += align(nnz)
            o_v = n_flt
            n_flt += align(nnz)
            o_B = n_flt
            n_flt += align(K * N)
            o_C = n_flt
            n_flt += align(M * N)
            self.layout.append((o_ro, o_ci, o_v, o_B, o_C, nnz))
        self.ipool = torch.empty(max(n_int, 1), dtype=torch.int32, device=dev)
        self.fpool = torch.empty(max(n_flt, 1), dtype=torch.float32, device=dev)
        self.bytes_device = 4 * (n_ro + n_int + n_flt)
        # row offsets: one host array in pool layout, one copy
        host_ro = np.zeros(max(n_ro, 1), dtype=np.int32)
        for (M, K, N, sp, pseed, ro), (o_ro, *_rest) in zip(self.items, self.layout):
            host_ro[o_ro:o_ro + M + 1] = ro
        self.rpool = torch.from_numpy(host_ro).to(dev)
        self.flops = 0.0
        self.alg_bytes = 0.0
        self.problems = pkg.ProblemArray(len(self.items))
        rb, ib, fb = self.rpool.data_ptr(), self.ipool.data_ptr(), self.fpool.data_ptr()
        for i, ((M, K, N, sp, pseed, ro), (o_ro, o_ci, o_v, o_B, o_C, nnz)) in enumerate(zip(self.items, self.layout)):
            ro_t = self.rpool[o_ro:o_ro + M + 1]
            ctx.gen_sample_columns(M, K, ro_t, pseed, self.ipool[o_ci:o_ci + max(nnz, 1)])
            if nnz:
                ctx.gen_dense(self.fpool[o_v:o_v + nnz], pseed, 2)
            ctx.gen_dense(self.fpool[o_B:o_B + K * N], pseed, 10)
            self.problems.set_raw(i, M, K, N, nnz, fb + 4 * o_v if nnz else None, rb + 4 * o_ro,
                                  ib + 4 * o_ci if nnz else None, fb + 4 * o_B, fb + 4 * o_C)
            self.flops += 2.0 * nnz * N
            self.alg_bytes += spmm_bytes(M, K, N, nnz)
        torch.cuda.synchronize()
        self.batch = ctx.batch_create(self.problems)

    def host_sample(self, max_bytes: int, max_problems: int):
        """Pinned host copies of the first problems of this rank: all inputs in ONE pinned arena in
        the order and spacing of the library's staging layout (per problem row_offsets,
        column_indices, values, B, each padded to 256 bytes), all outputs in a second one, so that
        dlspm_spmm_batched_f32_host can send every 128 MiB piece with one copy per direction."""
        import torch

        def pad(nbytes):
            return (nbytes + 255) // 256 * 256

        picked, total, in_bytes, out_bytes = [], 0, 0, 0
        for idx, ((M, K, N, sp, pseed, ro), lay) in enumerate(zip(self.items, self.layout)):
            nnz = lay[5]
            b = spmm_bytes(M, K, N, nnz)
            if picked and (total + b > max_bytes or len(picked) >= max_problems):
                break
            total += b
            offs = []
            for nb in (4 * (M + 1), 4 * nnz, 4 * nnz, 4 * K * N):
                offs.append(in_bytes)
                in_bytes += pad(nb)
            picked.append((idx, offs, out_bytes))
            out_bytes += pad(4 * M * N)
        arena_in = torch.empty(max(in_bytes, 256), dtype=torch.uint8).pin_memory()
        arena_out = torch.empty(max(out_bytes, 256), dtype=torch.uint8).pin_memory()
        in_i32, in_f32 = arena_in.view(torch.int32), arena_in.view(torch.float32)
        base_in, base_out = arena_in.data_ptr(), arena_out.data_ptr()
        arr = self.pkg.ProblemArray(len(picked))
        flops = h2d = d2h = 0.0
        for i, (idx, (a_ro, a_ci, a_v, a_B), a_C) in enumerate(picked):
            M, K, N, sp, pseed, ro = self.items[idx]
            o_ro, o_ci, o_v, o_B, o_C, nnz = self.layout[idx]
            in_i32[a_ro // 4:a_ro // 4 + M + 1].copy_(self.rpool[o_ro:o_ro + M + 1])
            if nnz:
                in_i32[a_ci // 4:a_ci // 4 + nnz].copy_(self.ipool[o_ci:o_ci + nnz])
                in_f32[a_v // 4:a_v // 4 + nnz].copy_(self.fpool[o_v:o_v + nnz])
            in_f32[a_B // 4:a_B // 4 + K * N].copy_(self.fpool[o_B:o_B + K * N])
            arr.set_raw(i, M, K, N, nnz, base_in + a_v if nnz else None, base_in + a_ro,
                        base_in + a_ci if nnz else None, base_in + a_B, base_out + a_C)
            flops += 2.0 * nnz * N
            h2d += 4 * (M + 1) + 8 * nnz + 4 * K * N
            d2h += 4 * M * N
        torch.cuda.synchronize()
        return arr, (arena_in, arena_out, picked), flops, h2d, d2h


# ---- parity of the timed launch (outside the timed region) -----------------------------------------------------

PARITY_TOL = 1e-4  # the tolerance of the parity tests: |out - ref| <= tol * max(|ref|, sum |products|)


def parity_sample(pkg, oracle, batch, max_problems=90):
    """Checks what the timed launch left in C against the CPU oracle, for one problem of every
    distinct (shape, sparsity, width) combination of this rank's share (the batch has 90): the
    inputs are regenerated on the host from the seeds (same bits as the device generators), the
    output is copied back from the pool the timed launch wrote."""
    threads = oracle.max_threads()
    seen, picks = set(), []
    for idx, (M, K, N, sp, pseed, ro) in enumerate(batch.items):
        if (M, K, N, sp) not in seen:
            seen.add((M, K, N, sp))
            picks.append(idx)
    if len(picks) > max_problems:
        picks = [picks[i * len(picks) // max_problems] for i in range(max_problems)]
    violations, worst, elements = 0, 0.0, 0
    for idx in picks:
        M, K, N, sp, pseed, ro = batch.items[idx]
        o_ro, o_ci, o_v, o_B, o_C, nnz = batch.layout[idx]
        ci = pkg.gen_sample_columns_host(M, K, ro, pseed)
        vals = pkg.gen_dense_host(int(ci.size), pseed, 2)
        B = pkg.gen_dense_host(K * N, pseed, 10).reshape(K, N)
        out = batch.fpool[o_C:o_C + M * N].cpu().numpy().reshape(M, N)
        ref = oracle.spmm(vals, ro, ci, B, M, N, threads=max(threads, 2))
        scale = oracle.spmm_scale(vals, ro, ci, B, M, N, threads=max(threads, 2))
        bad, w = oracle.violations(ref, out, scale, PARITY_TOL)
        violations += int(bad)
        worst = max(worst, min(float(w), 1e30))
        elements += M * N
    return {"checked": len(picks), "violations": violations, "elements": elements, "worst_ratio_of_tol": worst / PARITY_TOL if PARITY_TOL else None,
            "tol": PARITY_TOL, "against": "CPU oracle (the reference's host loop), inputs regenerated from the seeds",
            "what": "C of the timed grouped launch, one problem per distinct (shape, sparsity, N) of rank 0's share"}


# ---- clocks ------------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, dev_index: int):
        import torch

        self.proc = None
        self.path = f"/tmp/dlspm_clocks_{os.getpid()}.csv"
        try:
            uuid = str(torch.cuda.get_device_properties(dev_index).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception as e:  # nvidia-smi missing: report empty clocks
            log("clock sampler unavailable:", e)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def host_memory_available() -> float:
    """Bytes of host memory this process may still use: MemAvailable, capped by the cgroup limit."""
    avail = 64e9
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable:"):
                avail = float(line.split()[1]) * 1024.0
    except OSError:
        pass
    for path, used in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                       ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            lim = open(path).read().strip()
            if lim != "max":
                avail = min(avail, float(lim) - float(open(used).read().strip()))
        except (OSError, ValueError):
            pass
    return max(avail, 1e9)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- CPU baseline (the oracle: the reference's host loop, rows spread over the host threads) -----------------

def cpu_sample(pkg, descs, budget_flops: float):
    """Problems for the CPU arm, regenerated on the host (same bits as the device generators)."""
    order = sorted(range(len(descs)), key=lambda i: float(descs[i][5][-1]) * descs[i][2])
    # walk from the median-cost problem outwards so that the sample is neither all tiny nor all huge
    mid = len(order) // 2
    walk = [order[mid]]
    for step in range(1, len(order)):
        for pos in (mid - step, mid + step):
            if 0 <= pos < len(order):
                walk.append(order[pos])
    picked, flops = [], 0.0
    for i in walk:
        M, K, N, sp, pseed, ro = descs[i]
        f = 2.0 * float(ro[-1]) * N
        if picked and flops + f > budget_flops:
            break
        picked.append(i)
        flops += f
    data = []
    for i in picked:
        M, K, N, sp, pseed, ro = descs[i]
        ci = pkg.gen_sample_columns_host(M, K, ro, pseed)
        vals = pkg.gen_dense_host(int(ci.size), pseed, 2)
        B = pkg.gen_dense_host(K * N, pseed, 10).reshape(K, N)
        data.append((M, K, N, ro, ci, vals, B))
    return data, flops


def time_cpu(oracle, data, threads: int) -> float:
    t0 = time.perf_counter()
    for (M, K, N, ro, ci, vals, B) in data:
        oracle.spmm(vals, ro, ci, B, M, N, threads=max(threads, 2))
    return time.perf_counter() - t0


def cpu_rate_probe(pkg, oracle, threads):
    """GFLOP/s of the CPU loop on one mid-sized problem (sizes the bounded sample)."""
    M, K, N = 256, 256, 256
    ro = pkg.gen_rowlen_normal_host(M, K, 0.8, COV, 99)
    ci = pkg.gen_sample_columns_host(M, K, ro, 99)
    vals = pkg.gen_dense_host(int(ci.size), 99, 2)
    B = pkg.gen_dense_host(K * N, 99, 10).reshape(K, N)
    t = time_cpu(oracle, [(M, K, N, ro, ci, vals, B)], threads)
    return 2.0 * ci.size * N / t * 1e-9


def cpu_variants(oracle, data, flops, dt_all, threads):
    """The two other ways the reference's loop can be run on the host, on bounded sub-samples: one
    thread, exactly as the reference's drivers call it, and a speed build (-O3 -march=native,
    compiled on this machine) on all threads."""
    out = {}
    # one thread: a prefix of the sample worth about 3 s at 1/threads of the all-thread rate
    budget = flops / dt_all / max(threads, 1) * 3.0
    sub, f = [], 0.0
    for d in data:
        w = 2.0 * d[4].size * d[2]
        if sub and f + w > budget:
            break
        sub.append(d)
        f += w
    t0 = time.perf_counter()
    for (M, K, N, ro, ci, vals, B) in sub:
        oracle.spmm(vals, ro, ci, B, M, N, threads=1)
    out["single_thread"] = {"value": f / (time.perf_counter() - t0) * 1e-9, "unit": "GFLOP/s",
                            "sample": f"{len(sub)} problems ({f / 1e9:.2f} GFLOP)"}
    try:
        speed = oracle.SpeedBuild()
        t0 = time.perf_counter()
        for (M, K, N, ro, ci, vals, B) in data:
            speed.spmm(vals, ro, ci, B, M, N, max(threads, 2))
        out["o3_march_native"] = {"value": flops / (time.perf_counter() - t0) * 1e-9, "unit": "GFLOP/s", "cores": threads}
    except Exception as e:  # no compiler on the box: the figure is simply absent
        out["o3_march_native"] = {"value": None, "why": str(e)[:120]}
    # the same arithmetic with the loops interchanged (row of C innermost, unit stride): what a tuned
    # CPU library does at least; bit-identical results, since every element still sums in CSR order
    t0 = time.perf_counter()
    for (M, K, N, ro, ci, vals, B) in data:
        oracle.spmm(vals, ro, ci, B, M, N, threads=max(threads, 2), fast_order=True)
    out["loops_interchanged"] = {"value": flops / (time.perf_counter() - t0) * 1e-9, "unit": "GFLOP/s", "cores": threads}
    out["onemkl"] = time_onemkl(oracle, data, flops)
    return out


def time_onemkl(oracle, data, flops):
    """The reference's other CPU-side comparison is oneMKL's sparse BLAS (its MKL/ programs).  If
    the single dynamic library is installed on this machine, mkl_sparse_s_mm is timed on the same
    sample and checked against the oracle; otherwise the row says so."""
    import ctypes as C

    try:
        mkl = C.CDLL("libmkl_rt.so")
    except OSError:
        return {"value": None, "why": "unavailable on this box (no libmkl_rt.so)"}
    try:
        class Descr(C.Structure):
            _fields_ = [("type", C.c_int), ("mode", C.c_int), ("diag", C.c_int)]

        create = mkl.mkl_sparse_s_create_csr
        create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        mm = mkl.mkl_sparse_s_mm
        mm.argtypes = [C.c_int, C.c_float, C.c_void_p, Descr, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_float,
                       C.c_void_p, C.c_int]
        destroy = mkl.mkl_sparse_destroy
        destroy.argtypes = [C.c_void_p]
        descr = Descr(20, 40, 50)  # general matrix
        total, checked = 0.0, False
        for (M, K, N, ro, ci, vals, B) in data:
            ro32, ci32 = np.ascontiguousarray(ro, dtype=np.int32), np.ascontiguousarray(ci, dtype=np.int32)
            v32, b32 = np.ascontiguousarray(vals, dtype=np.float32), np.ascontiguousarray(B, dtype=np.float32)
            out = np.zeros((M, N), dtype=np.float32)
            h = C.c_void_p()
            if create(C.byref(h), 0, M, K, ro32.ctypes.data, ro32.ctypes.data + 4, ci32.ctypes.data, v32.ctypes.data):
                return {"value": None, "why": "mkl_sparse_s_create_csr failed"}
            t0 = time.perf_counter()
            st = mm(10, 1.0, h, descr, 101, b32.ctypes.data, N, N, 0.0, out.ctypes.data, N)
            total += time.perf_counter() - t0
            destroy(h)
            if st:
                return {"value": None, "why": f"mkl_sparse_s_mm status {st}"}
            if not checked:
                ref = oracle.spmm(vals, ro, ci, B, M, N, threads=2)
                if not np.allclose(out, ref, rtol=1e-4, atol=1e-4):
                    return {"value": None, "why": "mkl_sparse_s_mm result differs from the oracle"}
                checked = True
        return {"value": flops / total * 1e-9, "unit": "GFLOP/s", "threads": "library default"}
    except Exception as e:
        return {"value": None, "why": f"oneMKL call failed: {str(e)[:100]}"}


def run_reference_arm(args, rank, world):
    """Times the reference's own CPU implementation of the path (the pinned oracle) on host cores."""
    if rank != 0:
        return
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    threads = oracle.max_threads()
    descs = batch_descriptors(pkg, args.problems, args.seed)
    rate = cpu_rate_probe(pkg, oracle, threads)
    steps_total = max(1, args.steps + args.warmup)
    budget_s = min(20.0, 150.0 / steps_total)
    data, flops = cpu_sample(pkg, descs, rate * 1e9 * budget_s)
    for _ in range(args.warmup):
        time_cpu(oracle, data, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        time_cpu(oracle, data, threads)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    gflops = flops / dt * 1e-9
    sample = f"{len(data)} problems of the batch around the median cost ({flops / 1e9:.2f} GFLOP per step)"
    line = {
        "impl": "reference", "metric": "spmm_batch_gflops", "value": gflops, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, world),
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {"workload": f"batch of {args.problems} independent CSR SpMMs from the sweep grid "
                        "(5 shapes x 6 sparsities x N in {256,1024,3136}, row-length CoV 0.4), fp32",
            "problems": args.problems, "seed": args.seed, "partition": f"lpt by nnz*N over {world} gpu(s)",
            "l2": "inputs larger than L2 (no flush needed)"}


# ---- extras: the other configurations ---------------------------------------------------------------------------

def time_graph(fn, inner=20, reps=5):
    """Warm per-launch time in ms: `inner` back-to-back launches captured in one CUDA graph, so that
    host launch latency (about 10 us per call from Python) does not sit between the events."""
    import torch

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(inner):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / inner)
    return times


def time_kernel(fn, reps, flush=None):
    """Per-launch device times in ms (CUDA events on the current stream)."""
    import torch

    times = []
    for _ in range(reps):
        if flush is not None:
            flush.fill_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return times


def summarize(times_warm, times_cold, flops, nbytes, hbm_gbs, fp32_tflops):
    warm, cold = min(times_warm), statistics.median(times_cold)
    t_roof_ms = max(nbytes / (hbm_gbs * 1e9), flops / (fp32_tflops * 1e12)) * 1e3
    return {"us_warm_min": warm * 1e3, "us_cold_median": cold * 1e3,
            "gflops_warm": flops / warm * 1e-6, "gflops_cold": flops / cold * 1e-6,
            "hbm_gbs_cold": nbytes / cold * 1e-6, "hbm_frac_cold": nbytes / cold * 1e-6 / hbm_gbs,
            "roof_frac_cold": t_roof_ms / cold, "roof_frac_warm": t_roof_ms / warm,
            "binds": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (fp32_tflops * 1e12) else "fp32"}


def run_extras(pkg, ctx, dev, hbm_gbs, fp32_tflops, reps=20):
    import torch

    out = {}
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)  # 256 MiB > L2

    def up(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    # single SpMM 512 x 512, density 0.1, N = 128
    M, K, N = 512, 512, 128
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.1, 1)
    nnz = int(ci.size)
    d = [up(pkg.gen_dense_host(nnz, 1, 2)), up(ro), up(ci), up(pkg.gen_dense_host(K * N, 1, 10)), torch.empty(M * N, device=dev)]
    fn = lambda: ctx.spmm(M, K, N, nnz, *d)
    fn(); fn()
    out["spmm_512x512_d0.1_n128"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 2.0 * nnz * N,
                                               spmm_bytes(M, K, N, nnz), hbm_gbs, fp32_tflops)

    # SDDMM 2048 x 512 mask at density 0.2, inner dimension 128
    M, K, N = 2048, 512, 128
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.2, 2)
    nnz = int(ci.size)
    s = [up(ro), up(ci), up(pkg.gen_dense_host(M * N, 2, 11, kind=2)), up(pkg.gen_dense_host(K * N, 2, 12, kind=2)),
         torch.empty(nnz, device=dev)]
    fn = lambda: ctx.sddmm(M, K, N, nnz, *s)
    fn(); fn()
    out["sddmm_2048x512_d0.2_n128"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 2.0 * nnz * N,
                                                 4 * (M + 1) + 8 * nnz + 4 * M * N + 4 * K * N, hbm_gbs, fp32_tflops)

    # fused SDDMM -> SpMM, band(64) + 5 % mask 4096 x 4096, d = 64
    M = K = 4096
    N = 64
    ro, ci = pkg.gen_band_csr_host(M, K, 32, 0.05, 4)
    nnz = int(ci.size)
    f = [up(ro), up(ci), up(pkg.gen_dense_host(M * N, 4, 11, kind=2)), up(pkg.gen_dense_host(K * N, 4, 12, kind=2)),
         up(pkg.gen_dense_host(K * N, 4, 13, kind=2)), torch.empty(M * N, device=dev)]
    fn = lambda: ctx.fused(M, K, N, nnz, *f)
    fn(); fn()
    out["fused_band4096_d64"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 4.0 * nnz * N,
                                          4 * (M + 1) + 4 * nnz + 4 * N * (M + 2 * K) + 4 * M * N, hbm_gbs, fp32_tflops)

    # the same two kernels on patterns large enough to fill the device (the shapes of the ncu summaries)
    M, K, N = 8192, 2048, 128
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.2, 22)
    nnz = int(ci.size)
    s2 = [up(ro), up(ci), up(pkg.gen_dense_host(M * N, 22, 11, kind=2)), up(pkg.gen_dense_host(K * N, 22, 12, kind=2)),
          torch.empty(nnz, device=dev)]
    fn = lambda: ctx.sddmm(M, K, N, nnz, *s2)
    fn(); fn()
    out["sddmm_8192x2048_d0.2_n128"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 2.0 * nnz * N,
                                                  4 * (M + 1) + 8 * nnz + 4 * M * N + 4 * K * N, hbm_gbs, fp32_tflops)
    M, K, N = 16384, 4096, 64
    ro, ci = pkg.gen_bernoulli_csr_host(M, K, 0.066, 23)
    nnz = int(ci.size)
    f2 = [up(ro), up(ci), up(pkg.gen_dense_host(M * N, 23, 11, kind=2)), up(pkg.gen_dense_host(K * N, 23, 12, kind=2)),
          up(pkg.gen_dense_host(K * N, 23, 13, kind=2)), torch.empty(M * N, device=dev)]
    fn = lambda: ctx.fused(M, K, N, nnz, *f2)
    fn(); fn()
    out["fused_16384x4096_d0.066_n64"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 4.0 * nnz * N,
                                                   4 * (M + 1) + 4 * nnz + 4 * N * (M + 2 * K) + 4 * M * N, hbm_gbs, fp32_tflops)
    M = K = 4096
    N = 64
    nnz = int(f[1].numel())

    # the same chain as sparse attention: scale 1/sqrt(d) and a row softmax between the two products
    fn = lambda: ctx.attention(M, K, N, nnz, *f, scale=N ** -0.5, flags=pkg.ATTN_SOFTMAX)
    fn(); fn()
    out["attention_softmax_band4096_d64"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 4.0 * nnz * N,
                                                      4 * (M + 1) + 4 * nnz + 4 * N * (M + 2 * K) + 4 * M * N,
                                                      hbm_gbs, fp32_tflops)

    # the 90 % sparsity column of the sweep: 5 shapes x 3 widths
    sweep = {}
    for (M, K) in SHAPES:
        for N in WIDTHS:
            seed = 9000 + M + N
            ro = pkg.gen_rowlen_normal_host(M, K, 0.9, COV, seed)
            ci = pkg.gen_sample_columns_host(M, K, ro, seed)
            nnz = int(ci.size)
            Bm = torch.empty(K * N, device=dev)
            ctx.gen_dense(Bm, seed, 10)
            v = torch.empty(max(nnz, 1), device=dev)[:nnz]
            ctx.gen_dense(v, seed, 2)
            a = [v, up(ro), up(ci), Bm, torch.empty(M * N, device=dev)]
            fn = lambda: ctx.spmm(M, K, N, nnz, *a)
            fn(); fn()
            sweep[f"{M}x{K}_n{N}"] = summarize(time_graph(fn), time_kernel(fn, reps, flush), 2.0 * nnz * N,
                                                spmm_bytes(M, K, N, nnz), hbm_gbs, fp32_tflops)
    out["spmm_sweep_s0.9"] = sweep

    # the same 15 cases at batch granularity: 24 independent copies of each (distinct seeds) in one
    # prepared grouped launch, about 6 GB resident, so that launch latency and L2 residency drop out
    import statistics as st

    copies = 24
    arr = pkg.ProblemArray(15 * copies)
    keep, flops, nbytes, idx = [], 0.0, 0.0, 0
    for (M, K) in SHAPES:
        for N in WIDTHS:
            for c in range(copies):
                seed = 70000 + 100 * idx + c
                ro = pkg.gen_rowlen_normal_host(M, K, 0.9, COV, seed)
                nnz = int(ro[-1])
                d_ro = up(ro)
                d_ci = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)[:nnz]
                ctx.gen_sample_columns(M, K, d_ro, seed, d_ci)
                v = torch.empty(max(nnz, 1), device=dev)[:nnz]
                ctx.gen_dense(v, seed, 2)
                Bm = torch.empty(K * N, device=dev)
                ctx.gen_dense(Bm, seed, 10)
                Cm = torch.empty(M * N, device=dev)
                arr.set(idx * copies + c, M, K, N, nnz, v, d_ro, d_ci, Bm, Cm)
                flops += 2.0 * nnz * N
                nbytes += spmm_bytes(M, K, N, nnz)
            idx += 1
    batch = ctx.batch_create(arr)
    batch.launch()
    torch.cuda.synchronize()
    times = time_kernel(batch.launch, 5)
    ms = st.median(times)
    out["spmm_sweep_s0.9_batched"] = {
        "problems": 15 * copies, "ms_median": ms, "gflops": flops / ms * 1e-6, "hbm_gbs": nbytes / ms * 1e-6,
        "hbm_frac": nbytes / ms * 1e-6 / hbm_gbs,
        "roof_frac": max(nbytes / (hbm_gbs * 1e9), flops / (fp32_tflops * 1e12)) * 1e3 / ms,
        "binds": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (fp32_tflops * 1e12) else "fp32"}
    batch.close()

    # SDDMM and the fused chain on the same 90 % sparsity grid (mask shapes of the sweep, inner
    # dimension 32 / 128 / 256): lone launches, then 24 copies of every case in one grouped call
    inner = [32, 128, 256]

    def sddmm_bytes(M, K, N, nnz):
        return 4 * (M + 1) + 8 * nnz + 4 * M * N + 4 * K * N

    def fused_bytes(M, K, N, nnz):
        return 4 * (M + 1) + 4 * nnz + 4 * N * (M + 2 * K) + 4 * M * N

    for op in ("sddmm", "fused"):
        lone = {}
        copies = 24
        arr = pkg.RowProblemArray(op, 15 * copies)
        flops = nbytes = 0.0
        idx = 0
        for (M, K) in SHAPES:
            for N in inner:
                for c in range(copies):
                    seed = 80000 + 100 * idx + c
                    ro = pkg.gen_rowlen_normal_host(M, K, 0.9, COV, seed)
                    nnz = int(ro[-1])
                    d_ro = up(ro)
                    d_ci = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)[:nnz]
                    ctx.gen_sample_columns(M, K, d_ro, seed, d_ci)
                    a = torch.empty(M * N, device=dev)
                    ctx.gen_dense(a, seed, 11, kind=2)
                    b = torch.empty(K * N, device=dev)
                    ctx.gen_dense(b, seed, 12, kind=2)
                    if op == "sddmm":
                        o = torch.empty(max(nnz, 1), device=dev)[:nnz]
                        arr.set_sddmm(idx * copies + c, M, K, N, nnz, d_ro, d_ci, a, b, o)
                        fl, by = 2.0 * nnz * N, sddmm_bytes(M, K, N, nnz)
                        fn = (lambda M=M, K=K, N=N, nnz=nnz, t=(d_ro, d_ci, a, b, o): ctx.sddmm(M, K, N, nnz, *t))
                    else:
                        dv = torch.empty(K * N, device=dev)
                        ctx.gen_dense(dv, seed, 13, kind=2)
                        o = torch.empty(M * N, device=dev)
                        arr.set_fused(idx * copies + c, M, K, N, nnz, d_ro, d_ci, a, b, dv, o)
                        fl, by = 4.0 * nnz * N, fused_bytes(M, K, N, nnz)
                        fn = (lambda M=M, K=K, N=N, nnz=nnz, t=(d_ro, d_ci, a, b, dv, o): ctx.fused(M, K, N, nnz, *t))
                    flops += fl
                    nbytes += by
                    if c == 0:
                        fn(); fn()
                        lone[f"{M}x{K}_n{N}"] = summarize(time_graph(fn), time_kernel(fn, 10, flush), fl, by, hbm_gbs, fp32_tflops)
                idx += 1
        out[f"{op}_sweep_s0.9"] = lone
        call = (lambda: ctx.sddmm_batched(arr)) if op == "sddmm" else (lambda: ctx.fused_batched(arr))
        call()
        torch.cuda.synchronize()
        ms = st.median(time_kernel(call, 7))
        out[f"{op}_sweep_s0.9_batched"] = {
            "problems": 15 * copies, "ms_median": ms, "us_per_problem": ms * 1e3 / (15 * copies), "gflops": flops / ms * 1e-6,
            "hbm_gbs": nbytes / ms * 1e-6, "hbm_frac": nbytes / ms * 1e-6 / hbm_gbs,
            "roof_frac": max(nbytes / (hbm_gbs * 1e9), flops / (fp32_tflops * 1e12)) * 1e3 / ms,
            "binds": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (fp32_tflops * 1e12) else "fp32",
            "note": "one dlspm_%s_batched_f32 call: table build and copy included, three launches (one per inner dimension)" % op}
        del arr

    # shapes whose algorithmic intensity is below the fp32 ridge (HBM-bound on paper), many copies
    # of one shape in a grouped launch, about 1.5 GB resident each
    small = {}
    for (M, K, N, sp) in ((64, 64, 1024, 0.9), (64, 64, 1024, 0.98), (64, 64, 3136, 0.98), (256, 256, 3136, 0.98)):
        copies = int(min(3000, 1.5e9 / spmm_bytes(M, K, N, int(M * K * (1 - sp)))))
        arr = pkg.ProblemArray(copies)
        flops = nbytes = 0.0
        for c in range(copies):
            seed = 1000 * M + N + 7919 * c
            ro = pkg.gen_rowlen_normal_host(M, K, sp, COV, seed)
            nnz = int(ro[-1])
            d_ro = up(ro)
            d_ci = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)[:nnz]
            ctx.gen_sample_columns(M, K, d_ro, seed, d_ci)
            v = torch.empty(max(nnz, 1), device=dev)[:nnz]
            ctx.gen_dense(v, seed, 2)
            Bm = torch.empty(K * N, device=dev)
            ctx.gen_dense(Bm, seed, 10)
            arr.set(c, M, K, N, nnz, v, d_ro, d_ci, Bm, torch.empty(M * N, device=dev))
            flops += 2.0 * nnz * N
            nbytes += spmm_bytes(M, K, N, nnz)
        batch = ctx.batch_create(arr)
        batch.launch()
        torch.cuda.synchronize()
        ms = st.median(time_kernel(batch.launch, 5))
        batch.close()
        small[f"{M}x{K}_n{N}_s{sp}"] = {"copies": copies, "us_per_problem": ms * 1e3 / copies,
                                        "gflops": flops / ms * 1e-6, "hbm_gbs": nbytes / ms * 1e-6,
                                        "hbm_frac": nbytes / ms * 1e-6 / hbm_gbs}
        del arr
    out["spmm_hbm_bound_shapes_batched"] = small
    del flush
    return out


_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def _mix64_np(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def bernoulli_row_host(pkg, K, row, density, seed):
    """Columns of one row of the Bernoulli pattern of `seed`, computed on the host with the
    library's counter-based generator restated in numpy (checked against dlspm_rand_u64)."""
    key = _mix64((seed + 0x9E3779B97F4A7C15) & _M64) ^ _mix64((1 * 0xD1342543DE82EF95 + 0x2545F4914F6CDD1D) & _M64)
    with np.errstate(over="ignore"):
        idx = np.uint64(row) * np.uint64(K) + np.arange(K, dtype=np.uint64)
        h = _mix64_np(np.uint64(key) + (idx + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15))
    assert int(h[0]) == pkg.rand_u64(seed, 1, row * K) and int(h[-1]) == pkg.rand_u64(seed, 1, row * K + K - 1)
    thr = 0 if density <= 0 else (1 << 24) if density >= 1 else int(density * 16777216.0)
    return np.nonzero((h >> np.uint64(40)) < np.uint64(thr))[0].astype(np.int32)


def rowshard_reference_rows(pkg, oracle, K, N, density, seed, ro_all, rows):
    """Oracle result (and tolerance magnitudes) of the sampled global rows of the row-sharded SpMM,
    from inputs regenerated on the host: pattern rows, their values by CSR position, and all of B."""
    cols, vals, lens = [], [], []
    for r in rows:
        c = bernoulli_row_host(pkg, K, int(r), density, seed)
        assert c.size == int(ro_all[r + 1] - ro_all[r]), "row length differs from the device generator's"
        cols.append(c)
        vals.append(pkg.gen_dense_host(int(c.size), seed, 2, first_index=int(ro_all[r])))
        lens.append(c.size)
    ro = np.zeros(len(rows) + 1, dtype=np.int32)
    ro[1:] = np.cumsum(lens)
    ci = np.concatenate(cols) if cols else np.zeros(0, np.int32)
    v = np.concatenate(vals) if vals else np.zeros(0, np.float32)
    Bh = pkg.gen_dense_host(K * N, seed, 10).reshape(K, N)
    ref = oracle.spmm(v, ro, ci, Bh, len(rows), N)
    scale = oracle.spmm_scale(v, ro, ci, Bh, len(rows), N)
    return ref, scale


def run_rowshard(pkg, ctx, dev, rank, world, hbm_gbs, fp32_tflops, reps=5):
    """One 65536 x 65536 SpMM at 1 % density, N = 512, rows sharded by nonzeros, C blocks gathered."""
    import torch
    import torch.distributed as dist

    sharding = __import__("importlib").import_module(entry.PKG_NAME + ".sharding")
    M = K = 65536
    N = 512
    density, seed = 0.01, 5
    counts = torch.zeros(M, dtype=torch.int32, device=dev)
    ctx.gen_bernoulli_count(M, K, density, seed, counts)
    ro_all = np.zeros(M + 1, dtype=np.int32)
    ro_all[1:] = np.cumsum(counts.cpu().numpy().astype(np.int64)).astype(np.int32)
    r0, r1, bounds = sharding.row_block(pkg, ro_all, rank, world)
    rows = r1 - r0
    ro = torch.from_numpy(sharding.rebase_offsets(ro_all, r0, r1)).to(dev)
    nnz = int(ro_all[r1] - ro_all[r0])
    ci = torch.empty(max(nnz, 1), dtype=torch.int32, device=dev)[:nnz]
    ctx.gen_bernoulli_fill(rows, K, density, seed, ro, ci, first_row=r0)
    vals = torch.empty(max(nnz, 1), device=dev)[:nnz]
    ctx.gen_dense(vals, seed, 2, first_index=int(ro_all[r0]))
    B = torch.empty(K * N, device=dev)  # replicated on every rank
    ctx.gen_dense(B, seed, 10)
    Cl = torch.empty(rows, N, device=dev)
    torch.cuda.synchronize()

    def step():
        ctx.spmm(rows, K, N, nnz, vals, ro, ci, B, Cl)
        if world > 1:
            return sharding.gather_row_blocks(Cl, bounds, N)
        return Cl

    step(); step()
    torch.cuda.synchronize()
    times, ktimes = [], []
    for _ in range(reps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        ctx.spmm(rows, K, N, nnz, vals, ro, ci, B, Cl)
        e1.record()
        if world > 1:
            sharding.gather_row_blocks(Cl, bounds, N)
        e2.record()
        e2.synchronize()
        t = torch.tensor([e0.elapsed_time(e2), e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t[0]))
        ktimes.append(float(t[1]))
    total_nnz = int(ro_all[-1])
    flops = 2.0 * total_nnz * N
    nbytes = spmm_bytes(M, K, N, total_nnz)
    ms = statistics.median(times)
    out = {"workload": "65536x65536 density 0.01 N=512, rows sharded by nnz, B replicated, C blocks gathered on every GPU",
           "nccl_gather": {"ms_total_median": ms, "ms_kernel_median": statistics.median(ktimes),
                           "gflops": flops / ms * 1e-6},
           "nnz": total_nnz, "n_gpus": world}
    best_ms = ms
    # oracle check of sampled rows (spread over every rank's block), inputs regenerated on the host
    oracle = entry.load_oracle()
    sample_rows = np.unique(np.linspace(0, M - 1, 96).astype(np.int64))
    ref_rows, scale_rows = rowshard_reference_rows(pkg, oracle, K, N, density, seed, ro_all, sample_rows)
    rows_t = torch.from_numpy(sample_rows).to(dev)

    def violations_of(full_c):
        got = full_c.index_select(0, rows_t).cpu().numpy()
        bad, _w = oracle.violations(ref_rows, got, scale_rows, PARITY_TOL)
        v = torch.tensor([int(bad)], device=dev, dtype=torch.int64)
        if world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.SUM)
        return int(v[0])

    full_nccl = step()
    torch.cuda.synchronize()
    out["nccl_gather"]["oracle_rows_checked_per_rank"] = int(sample_rows.size)
    out["nccl_gather"]["oracle_violations_all_ranks"] = violations_of(full_nccl.view(M, N))
    if world > 1:
        # fused form: the SpMM epilogue stores every row into the full C of all ranks over NVLink
        # (peer mappings through CUDA IPC), so no collective follows the kernel
        full_ptr, handle = ctx.peer_alloc(M * N * 4)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        opened = {r: ctx.peer_open(h) for r, h in enumerate(handles) if r != rank}
        peers = list(opened.values())
        # destinations in ring order starting with this rank: at every step of the kernel's round of
        # destinations the ranks then store to different GPUs
        dsts = [full_ptr if (rank + j) % world == rank else opened[(rank + j) % world] for j in range(world)]
        gathered = full_nccl

        def time_scatter(dst_list):
            for _ in range(2):
                ctx.spmm_scatter(rows, K, N, nnz, vals, ro, ci, B, dst_list, r0)
            torch.cuda.synchronize()
            dist.barrier()
            ts = []
            for _ in range(reps):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ctx.spmm_scatter(rows, K, N, nnz, vals, ro, ci, B, dst_list, r0)
                e1.record()
                e1.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts.append(float(t[0]))
            dist.barrier()
            return statistics.median(ts)

        local_only_ms = time_scatter([full_ptr])  # same kernel, own C only: what the remote stores add
        fms = time_scatter(dsts)
        mine = pkg.DeviceArray(full_ptr, (M, N)).tensor(dev)
        same = torch.tensor([1 if torch.equal(mine, gathered.view(M, N)) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        out["fused_peer_stores"] = {"ms_total_median": fms, "gflops": flops / fms * 1e-6,
                                    "ms_one_destination": local_only_ms,
                                    "equals_nccl_result_on_every_rank": bool(int(same[0])),
                                    "oracle_rows_checked_per_rank": int(sample_rows.size),
                                    "oracle_violations_all_ranks": violations_of(mine)}
        best_ms = min(best_ms, fms)
        del mine, gathered
        torch.cuda.synchronize()
        dist.barrier()
        for p in peers:
            ctx.peer_close(p)
        dist.barrier()
        ctx.peer_free(full_ptr)
    # roofs of `world` GPUs together (B is read by every GPU: algorithmic bytes count it once)
    out.update({"ms_total_median": best_ms, "gflops": flops / best_ms * 1e-6,
                "hbm_frac": nbytes / best_ms * 1e-6 / (hbm_gbs * world),
                "roof_frac": max(nbytes / (hbm_gbs * 1e9), flops / (fp32_tflops * 1e12)) * 1e3 / best_ms / world})
    return out


def rowshard_summary(r):
    """The figures of the row-sharded large SpMM in a few numbers (kept near the front of the line)."""
    if not r:
        return None
    f = r.get("fused_peer_stores") or {}
    g = r.get("nccl_gather") or {}
    return {"n_gpus": r.get("n_gpus"), "ms": r.get("ms_total_median"), "ms_nccl_form": g.get("ms_total_median"),
            "ms_kernel_only": g.get("ms_kernel_median"), "ms_fused_form": f.get("ms_total_median"),
            "ms_fused_one_destination": f.get("ms_one_destination"),
            "oracle_violations": (g.get("oracle_violations_all_ranks", 0) or 0) + (f.get("oracle_violations_all_ranks", 0) or 0),
            "oracle_rows_per_rank": g.get("oracle_rows_checked_per_rank")}


# ---- main arm ------------------------------------------------------------------------------------------------------

def bind_to_gpu_cpus(local_rank):
    """With several ranks on one host the pinned staging buffers of a rank should live on the NUMA
    node of its GPU (first touch places them where the rank runs), or eight ranks pull their copies
    through one socket.  This restricts the rank's own CPU affinity to the CPUs NVML names for the
    GPU, when the process is allowed to run on any of them; nothing about the GPU is changed."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        ideal = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        both = ideal & allowed
        note = f"[rank {local_rank}] cpus allowed {len(allowed)}, near the GPU {len(ideal)}, both {len(both)}"
        if both and both != allowed:
            os.sched_setaffinity(0, both)
            note += " -> bound"
        print(note, file=sys.stderr, flush=True)
    except Exception as e:  # no NVML, or the query is not supported: run unbound
        print(f"[rank {local_rank}] cpu binding skipped: {str(e)[:80]}", file=sys.stderr, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--problems", type=int, default=8192)
    ap.add_argument("--seed", type=int, default=2024)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed launch")
    ap.add_argument("--tile-density", type=int, default=None, help="DLSPM_OPT_TILE_MIN_DENSITY in thousandths")
    ap.add_argument("--spmm-kernel", type=int, default=0, help="0 auto, 1 row-gather only, 2 tiled where possible, 3 tiled with zeros")
    ap.add_argument("--e2e-bytes", type=float, default=None,
                    help="host bytes of the e2e sample per rank (default: 16e9 on one GPU, 4e9 per rank on several)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        bind_to_gpu_cpus(local_rank)
        dist.init_process_group("nccl", device_id=dev)

    pkg = entry.load_package()
    ctx = pkg.Context(local_rank)
    if args.tile_density is not None:
        ctx.set_option(pkg.OPT_TILE_MIN_DENSITY, args.tile_density)
    ctx.set_option(pkg.OPT_SPMM_KERNEL, args.spmm_kernel)
    hbm_gbs, peak_kind = measured_peaks()
    fp32_tflops = ctx.measure_fp32_peak()

    t_setup = time.perf_counter()
    descs = batch_descriptors(pkg, args.problems, args.seed)
    weights = np.array([float(d[5][-1]) * d[2] for d in descs])
    sharding = __import__("importlib").import_module(entry.PKG_NAME + ".sharding")
    mine = sharding.my_problems(pkg, weights, rank, world)
    # the batch must fit the memory that is free on this GPU (113 GiB for all 8192 problems on one
    # GPU); if it does not, every rank drops the same tail of the batch and the line says so
    need = sum(4.0 * (descs[i][0] + 1 + 2 * float(descs[i][5][-1]) + descs[i][1] * descs[i][2] + descs[i][0] * descs[i][2])
               for i in mine)
    free_bytes, _total = torch.cuda.mem_get_info(dev)
    fit = torch.tensor([min(1.0, 0.85 * free_bytes / max(need, 1.0))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(fit, op=dist.ReduceOp.MIN)
    if float(fit[0]) < 1.0:
        args.problems = max(world, int(args.problems * float(fit[0])))
        log(f"[rank {rank}] batch cut to {args.problems} problems to fit device memory")
        descs = descs[:args.problems]
        weights = weights[:args.problems]
        mine = sharding.my_problems(pkg, weights, rank, world)
    batch = DeviceBatch(pkg, ctx, dev, descs, mine)
    n_gather, n_tiled, _ = batch.batch.info()
    part_stats = list(batch.batch.stats)
    launches_per_step = (1 if n_gather else 0) + (1 if n_tiled else 0)
    log(f"[rank {rank}] {len(mine)} problems ({n_tiled} tiled, {n_gather} row-gather), "
        f"{batch.bytes_device / 2**30:.1f} GiB on device, "
        f"{batch.flops / 1e12:.2f} TFLOP per step, set-up {time.perf_counter() - t_setup:.1f} s")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        batch.batch.launch()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for s in range(args.steps):
        batch.batch.launch()
        ev[s + 1].record()
    barrier()
    clocks = sampler.stop() if sampler else None
    my_ms = ev[0].elapsed_time(ev[-1])
    launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    t = torch.tensor([my_ms], device=dev, dtype=torch.float64)
    tot = torch.tensor([batch.flops, batch.alg_bytes], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    total_ms = float(t[0])
    ms_per_step = total_ms / args.steps
    value = float(tot[0]) / (ms_per_step * 1e-3) * 1e-9

    # each kernel of the step on its own (rank 0's share), for the roofline of the dominant one
    parts = {}
    for part, name, nprob, fl, by in ((1, "spmm_batched_kernel", n_gather, part_stats[0], part_stats[1]),
                                      (2, "spmm_tile_kernel", n_tiled, part_stats[2], part_stats[3])):
        if not nprob:
            continue
        batch.batch.launch_part(part)
        torch.cuda.synchronize()
        pe = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        pe[0].record()
        for i in range(3):
            batch.batch.launch_part(part)
            pe[i + 1].record()
        torch.cuda.synchronize()
        ms = statistics.mean(pe[i].elapsed_time(pe[i + 1]) for i in range(3))
        parts[name] = {"problems": nprob, "launch_ms": ms, "gflops": fl / ms * 1e-6,
                       "algorithmic_bytes_per_launch": by, "achieved_gbs": by / ms * 1e-6,
                       "fp32_frac": fl / (ms * 1e-3) * 1e-12 / fp32_tflops}
    barrier()

    # what the timed launches computed, against the CPU oracle (rank 0's share; after the timed
    # region, so the check costs the measurement nothing)
    parity = None
    if rank == 0 and not args.no_parity:
        parity = parity_sample(pkg, entry.load_oracle(), batch)
        log(f"[rank 0] parity: {parity['checked']} problems, {parity['violations']} violations, "
            f"worst {parity['worst_ratio_of_tol']:.3f} of tolerance")
    barrier()

    # end to end through the host-buffer entry point (copies inside the timed region)
    # the sample is bounded by the host memory the ranks of this machine can pin together
    # (several ranks pin and copy their samples at once through the same host: 4 GB per rank there)
    want_bytes = float(args.e2e_bytes) if args.e2e_bytes is not None else (16e9 if world == 1 else 4e9)
    e_bytes = min(want_bytes, 0.35 * host_memory_available() / max(world, 1))
    arr, keep, e_flops, e_h2d, e_d2h = batch.host_sample(int(e_bytes), 1 << 20)
    n_sample = len(keep[2])
    e_steps = max(3, min(args.steps, 5))
    ctx.spmm_batched_host(arr)
    barrier()
    copies0 = ctx.host_copy_count()
    t0 = time.perf_counter()
    for _ in range(e_steps):
        ctx.spmm_batched_host(arr)
    torch.cuda.synchronize()
    e_dt = (time.perf_counter() - t0) / e_steps
    copies_per_step = (ctx.host_copy_count() - copies0) / e_steps
    # what came back to the host is what the device-resident launch computed (same kernel, same bits)
    out_f32 = keep[1].view(torch.float32)
    e_same = True
    for (idx, _offs, a_C) in keep[2][:: max(1, n_sample // 16)]:
        M, K, N = batch.items[idx][:3]
        o_C = batch.layout[idx][4]
        e_same = e_same and bool(torch.equal(out_f32[a_C // 4:a_C // 4 + M * N], batch.fpool[o_C:o_C + M * N].cpu()))
    et = torch.tensor([e_dt], device=dev, dtype=torch.float64)
    ef = torch.tensor([e_flops, e_h2d, e_d2h, 1.0 if e_same else 0.0], device=dev, dtype=torch.float64)
    emin = ef[3:4].clone()
    if world > 1:
        dist.all_reduce(et, op=dist.ReduceOp.MAX)
        dist.all_reduce(ef, op=dist.ReduceOp.SUM)
        dist.all_reduce(emin, op=dist.ReduceOp.MIN)
    e2e = {"value": float(ef[0]) / float(et[0]) * 1e-9, "unit": "GFLOP/s",
           "h2d_bytes_per_step": float(ef[1]), "d2h_bytes_per_step": float(ef[2]),
           "sample": f"first {n_sample} problems of every rank's share (rank 0's count), inputs in one pinned arena and "
                     "outputs in another, dlspm_spmm_batched_f32_host (H2D + grouped launch + D2H per step)",
           "ms_per_step": float(et[0]) * 1e3,
           "h2d_gbs_per_rank": float(ef[1]) / world / float(et[0]) * 1e-9,
           "d2h_gbs_per_rank": float(ef[2]) / world / float(et[0]) * 1e-9,
           "memcpy_calls_per_step_rank0": copies_per_step,
           "results_equal_device_resident_launch": bool(float(emin[0]) > 0.5)}
    del arr, keep, out_f32

    extras = {}
    if not args.no_extras:
        try:
            extras["rowshard_65536"] = run_rowshard(pkg, ctx, dev, rank, world, hbm_gbs, fp32_tflops)
            if rank == 0 and world == 1:
                extras.update(run_extras(pkg, ctx, dev, hbm_gbs, fp32_tflops))
        except Exception as e:  # extras never invalidate the headline line
            extras["error"] = repr(e)
    barrier()

    if rank == 0:
        step_avg_ms = statistics.mean(launch_ms)
        dominant = max(parts, key=lambda k: parts[k]["launch_ms"])
        dom = parts[dominant]
        launch_avg_ms = dom["launch_ms"]
        achieved = dom["achieved_gbs"]
        dom_flops = dom["gflops"] * 1e6 * dom["launch_ms"]
        t_roof_ms = max(dom["algorithmic_bytes_per_launch"] / (hbm_gbs * 1e9), dom_flops / (fp32_tflops * 1e12)) * 1e3
        line = {
            "metric": "spmm_batch_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "rowshard_65536_summary": rowshard_summary(extras.get("rowshard_65536")),
            "data": "synthetic", "config": workload_config(args, world),
            "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps * launches_per_step, "parity": parity,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": achieved / hbm_gbs,
                         "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE[dominant] * dom["algorithmic_bytes_per_launch"]
                                     if dominant in NCU_TRAFFIC_PER_ALGORITHMIC_BYTE else None),
                         "peak_source": f"of {peak_kind}",
                         "kernel": dominant, "launch_ms": launch_avg_ms,
                         "algorithmic_bytes_per_launch": dom["algorithmic_bytes_per_launch"],
                         "fp32_peak_tflops_measured": fp32_tflops,
                         "fp32_frac": dom["fp32_frac"],
                         "binding_roof": "hbm" if dom["algorithmic_bytes_per_launch"] / (hbm_gbs * 1e9) >= dom_flops / (fp32_tflops * 1e12) else "fp32",
                         "roof_frac": t_roof_ms / launch_avg_ms,
                         "step_ms_rank0": step_avg_ms, "kernels": parts},
            "extras": extras,
        }
        if world == 1 and not args.no_cpu:
            oracle = entry.load_oracle()
            threads = oracle.max_threads()
            rate = cpu_rate_probe(pkg, oracle, threads)
            data, flops = cpu_sample(pkg, descs, rate * 1e9 * 15.0)
            dt = time_cpu(oracle, data, threads)
            line["cpu_baseline"] = {"value": flops / dt * 1e-9, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{len(data)} problems of the batch around the median cost "
                                              f"({flops / 1e9:.2f} GFLOP, {dt:.1f} s)",
                                    "build": "-O2 -ffp-contract=off (the build the parity tests pin)"}
            line["cpu_baseline"].update(cpu_variants(oracle, data, flops, dt, threads))
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    ctx.close()
    if parity is not None and parity["violations"]:
        raise SystemExit(f"parity check failed: {parity['violations']} elements beyond tolerance")


if __name__ == "__main__":
    main()
