// Shared pieces of the command-line drivers.  The drivers mirror the reference's self-checking
// programs: build inputs, run a naive host loop, run the GPU kernel several times, print the minimum
// kernel time, GFLOP/s and the largest difference, and optionally append a CSV row
// (SPMM/spmm-esimd-fromfile.cpp:86-320, SDDMM/sddmm-esimd-fromfile_v4.cpp:38-259,
// FUSED/fused-esimd_cb.cpp:223-386).
//
// The host loops below exist only to print that difference, as the reference's mains do; they are
// never used to produce a result and are skipped with --no-check.  The library itself has no CPU
// path.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <string>
#include <vector>

#include "../../include/dlspm.h"

namespace drv {

struct Options {
    std::vector<std::string> positional;
    int reps = 20;
    uint64_t seed = 1;
    bool check = true;
    bool signed_values = false;  // default: values in [0,1) like the reference's rand()/RAND_MAX
    bool planned = false;
    bool cold = false;           // also time with L2 flushed between repetitions
    int device = 0;
    std::string csv;
    bool graph = false;          // also time 100 launches captured in one CUDA graph (automatic below 10 us)
    bool cache = false;          // from-file drivers: keep a binary copy "<file>.csrbin" beside the text
    bool attention = false;      // fused driver: scale (and softmax) between the two products
    bool softmax = false;
    float scale = 1.f;
    int check_rows = 0;          // > 0: the host loop checks about this many evenly spaced rows only
    std::string list;            // from-file drivers: a file of "<pattern file> <batchsize>" lines, all run by one process
};

// Distance between checked rows: 1 = every row.
inline int check_stride(const Options &o, int M)
{
    if (o.check_rows <= 0 || o.check_rows >= M) return 1;
    return (M + o.check_rows - 1) / o.check_rows;
}

inline Options parse(int argc, char **argv)
{
    Options o;
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto next = [&]() -> const char * { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "--reps") o.reps = std::max(1, atoi(next()));
        else if (a == "--seed") o.seed = strtoull(next(), nullptr, 10);
        else if (a == "--csv") o.csv = next();
        else if (a == "--device") o.device = atoi(next());
        else if (a == "--no-check") o.check = false;
        else if (a == "--signed") o.signed_values = true;
        else if (a == "--planned") o.planned = true;
        else if (a == "--cold") o.cold = true;
        else if (a == "--cache") o.cache = true;
        else if (a == "--graph") o.graph = true;
        else if (a == "--softmax") o.attention = o.softmax = true;
        else if (a == "--scale") { o.attention = true; o.scale = (float)atof(next()); }
        else if (a == "--check-rows") o.check_rows = atoi(next());
        else if (a == "--list") o.list = next();
        else o.positional.push_back(a);
    }
    return o;
}

#define DRV_TRY(call)                                                                  \
    do {                                                                               \
        int rc__ = (call);                                                             \
        if (rc__ != DLSPM_OK) {                                                        \
            printf("%s failed: %s\n", #call, dlspm_strerror(rc__));                    \
            return rc__;                                                               \
        }                                                                              \
    } while (0)

#define DRV_CUDA(call)                                                                 \
    do {                                                                               \
        cudaError_t e__ = (call);                                                      \
        if (e__ != cudaSuccess) {                                                      \
            printf("%s failed: %s\n", #call, cudaGetErrorString(e__));                 \
            return 2;                                                                  \
        }                                                                              \
    } while (0)

template <typename T>
T *to_device(const std::vector<T> &h)
{
    T *d = nullptr;
    if (cudaMalloc(&d, std::max<size_t>(h.size(), 1) * sizeof(T)) != cudaSuccess) return nullptr;
    if (!h.empty()) cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

// Minimum and median device time in ms of `reps` launches, each bracketed by events; the reference
// reports the minimum (SPMM/spmm-esimd-fromfile.cpp:231-238).  With flush != nullptr a buffer
// larger than L2 is rewritten before every launch.
// Stream the timed launches go to: the default stream, except while a graph is being captured.
inline void *&launch_stream()
{
    static void *s = nullptr;
    return s;
}

// Per-launch time with `count` back-to-back launches captured in one CUDA graph, so that the gap
// between a lone launch and its events (a few microseconds) does not count: the figure for
// kernels that run less than about 10 us.
template <class F>
int time_graph(F &&launch, int count, double *ms_per_launch)
{
    cudaStream_t st;
    DRV_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    launch_stream() = st;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = DLSPM_OK;
    cudaError_t err = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    for (int i = 0; err == cudaSuccess && rc == DLSPM_OK && i < count; i++) rc = launch();
    cudaError_t end_err = cudaStreamEndCapture(st, &graph);
    launch_stream() = nullptr;
    if (err == cudaSuccess) err = end_err;
    if (err == cudaSuccess && rc == DLSPM_OK) err = cudaGraphInstantiate(&exec, graph, 0);
    if (err != cudaSuccess || rc != DLSPM_OK) {
        printf("graph timing skipped: %s\n", err != cudaSuccess ? cudaGetErrorString(err) : dlspm_strerror(rc));
        if (graph) cudaGraphDestroy(graph);
        cudaStreamDestroy(st);
        cudaGetLastError();
        return DLSPM_OK;
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float best = 1e30f;
    for (int r = 0; r < 6; r++) {  // the first replay warms up
        cudaEventRecord(e0, st);
        cudaGraphLaunch(exec, st);
        cudaEventRecord(e1, st);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r > 0 && ms < best) best = ms;
    }
    *ms_per_launch = (double)best / count;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    cudaStreamDestroy(st);
    return DLSPM_OK;
}

template <typename F>
int time_launches(F &&launch, int reps, float *flush, size_t flush_elems, double *min_ms, double *median_ms)
{
    cudaEvent_t e0, e1;
    DRV_CUDA(cudaEventCreate(&e0));
    DRV_CUDA(cudaEventCreate(&e1));
    std::vector<float> t;
    for (int r = 0; r < reps + 2; r++) {
        if (flush) cudaMemsetAsync(flush, r & 0xff, flush_elems * sizeof(float), 0);
        cudaEventRecord(e0, 0);
        int rc = launch();
        cudaEventRecord(e1, 0);
        if (rc != DLSPM_OK) {
            printf("kernel launch failed: %s\n", dlspm_strerror(rc));
            return rc;
        }
        DRV_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (r >= 2) t.push_back(ms);  // two warm-up launches
    }
    std::sort(t.begin(), t.end());
    *min_ms = t.front();
    *median_ms = t[t.size() / 2];
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return DLSPM_OK;
}

// ---- verification loops (print-only) -----------------------------------------------------------

// fp32 accumulation in CSR order, the reference's Spmm (SPMM/spmm-esimd-fromfile.cpp:63-83).
// (stride > 1: only rows 0, stride, 2*stride, ... are computed; the others are left as they are)
inline void check_spmm(const float *a, const int *ro, const int *ci, const float *b, float *c, int M, int N, int stride = 1)
{
    for (int i = 0; i < M; i += stride)
        for (int j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int l = ro[i]; l < ro[i + 1]; l++) acc += a[l] * b[(size_t)ci[l] * N + j];
            c[(size_t)i * N + j] = acc;
        }
}

// double accumulation, the reference's Sddmm (SDDMM/sddmm-esimd-fromfile_v4.cpp:18-36).
inline void check_sddmm(const int *ro, const int *ci, const float *lhs, const float *rhs, float *out, int M, int N, int stride = 1)
{
    for (int i = 0; i < M; i += stride)
        for (int j = ro[i]; j < ro[i + 1]; ++j) {
            double acc = 0.0;
            for (int l = 0; l < N; ++l) acc += (double)lhs[(size_t)i * N + l] * (double)rhs[(size_t)ci[j] * N + l];
            out[j] = (float)acc;
        }
}

// double accumulation, the Spmm of the fused reference (FUSED/fused.cpp:67-89).
inline void check_spmm_f64(const float *a, const int *ro, const int *ci, const float *d, float *e, int M, int N, int stride = 1)
{
    for (int i = 0; i < M; i += stride)
        for (int j = 0; j < N; ++j) {
            double acc = 0.0;
            for (int l = ro[i]; l < ro[i + 1]; ++l) acc += (double)a[l] * (double)d[(size_t)ci[l] * N + j];
            e[(size_t)i * N + j] = (float)acc;
        }
}

struct Diff {
    double max_diff = 0.0, max_rel_diff = 0.0;
    size_t maxi = 0;
};

inline Diff compare(const float *cpu, const float *gpu, size_t n)
{
    Diff d;
    for (size_t i = 0; i < n; i++) {
        const double diff = fabs((double)cpu[i] - (double)gpu[i]);
        const double den = std::max(fabs((double)cpu[i]), fabs((double)gpu[i]));
        if (den > 0.0) d.max_rel_diff = std::max(d.max_rel_diff, diff / den);
        if (diff > d.max_diff) {
            d.max_diff = diff;
            d.maxi = i;
        }
    }
    return d;
}

// The same over the checked rows only: row i covers elements [begin(i), end(i)).
template <class Begin, class End>
Diff compare_rows(const float *cpu, const float *gpu, int M, int stride, Begin begin, End end)
{
    Diff d;
    for (int i = 0; i < M; i += stride) {
        const size_t b = begin(i), e = end(i);
        if (e <= b) continue;
        const Diff r = compare(cpu + b, gpu + b, e - b);
        d.max_rel_diff = std::max(d.max_rel_diff, r.max_rel_diff);
        if (r.max_diff > d.max_diff) {
            d.max_diff = r.max_diff;
            d.maxi = b + r.maxi;
        }
    }
    return d;
}

inline double mean_square(const float *x, size_t n)
{
    double s = 0.0;
    for (size_t i = 0; i < n; i++) s += (double)x[i] * x[i];
    return n ? s / (double)n : 0.0;
}

inline void print_device(dlspm_ctx *ctx)
{
    char name[256];
    int sms = 0;
    size_t mem = 0;
    dlspm_device_info(ctx, name, sizeof(name), &sms, &mem);
    printf("Running on %s (%d SMs, %.0f GiB)\n", name, sms, (double)mem / (1024.0 * 1024.0 * 1024.0));
}

// ---- one SpMM case: inputs, optional host check, timed launches, report ------------------------
// Report lines and CSV columns follow SPMM/spmm-esimd-fromfile.cpp:241-291
// (CSV: M,N,K,density,gflops,max_diff,opcount).
// file_values: the values block of the input file if it carried one; generated values otherwise
inline int run_spmm_case(dlspm_ctx *ctx, const Options &o, int M, int K, int N, const std::vector<int> &ro,
                         const std::vector<int> &ci, const std::vector<float> *file_values = nullptr)
{
    const int nnz = (int)ci.size();
    std::vector<float> vals((size_t)nnz), B((size_t)K * N), C((size_t)M * N, 0.f), Ccpu;
    const int kind = o.signed_values ? 0 : 1;
    if (file_values && file_values->size() == vals.size()) vals = *file_values;
    else dlspm_gen_dense_host(vals.data(), vals.size(), o.seed, 2, 0, kind);
    dlspm_gen_dense_host(B.data(), B.size(), o.seed, 10, 0, kind);
    printf("rhs_matrix allocated\n");
    if (o.check) {
        Ccpu.assign((size_t)M * N, 0.f);
        check_spmm(vals.data(), ro.data(), ci.data(), B.data(), Ccpu.data(), M, N, check_stride(o, M));
        if (check_stride(o, M) > 1) printf("host check on every %d-th row\n", check_stride(o, M));
        printf("checksum_cpu = %.7g\n", mean_square(Ccpu.data(), Ccpu.size()));
    }
    int *d_ro = to_device(ro), *d_ci = to_device(ci);
    float *d_v = to_device(vals), *d_B = to_device(B), *d_C = to_device(C);
    if (!d_ro || !d_ci || !d_v || !d_B || !d_C) {
        printf("device allocation failed\n");
        return DLSPM_ERR_NOMEM;
    }
    printf("copy to device completed\n");
    dlspm_plan *plan = nullptr;
    if (o.planned) {
        // set-up time is reported on its own line, never inside the kernel time
        cudaDeviceSynchronize();
        const auto t0 = std::chrono::steady_clock::now();
        DRV_TRY(dlspm_plan_create(ctx, M, K, nnz, d_ro, d_ci, nullptr, &plan));
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        printf("plan (rows binned by length) created in %f ms\n", ms);
    }
    printf("Start kernel execution\n");
    auto launch = [&]() {
        return plan ? dlspm_spmm_csr_f32_planned(ctx, plan, N, d_v, d_ro, d_ci, d_B, d_C, launch_stream())
                    : dlspm_spmm_csr_f32(ctx, M, K, N, nnz, d_v, d_ro, d_ci, d_B, d_C, launch_stream());
    };
    double min_ms = 0, med_ms = 0;
    DRV_TRY(time_launches(launch, o.reps, nullptr, 0, &min_ms, &med_ms));
    const double density = (double)nnz / ((double)M * K);
    printf("MSZ = %d KSZ = %d NSZ = %d SP = %f\n", M, K, N, density);
    printf("Total kernel time was %f ms.\n", min_ms);
    // the reference's operation count: (2*nnz - M) * N
    const float opcount = (2 * (float)nnz - M) * N;
    const float gflops = opcount / (min_ms * 1.0E+6);
    printf("GFLOPS:  %8.2f\n", gflops);
    const double flops2 = 2.0 * nnz * (double)N;
    const double bytes = 4.0 * (M + 1) + 8.0 * nnz + 4.0 * (double)K * N + 4.0 * (double)M * N;
    printf("GFLOPS (2*nnz*N): %8.2f  algorithmic GB/s: %8.2f  median ms: %f\n", flops2 / (min_ms * 1e6),
           bytes / (min_ms * 1e6), med_ms);
    if (o.graph || min_ms < 0.010) {
        double g_ms = 0;
        DRV_TRY(time_graph(launch, 100, &g_ms));
        if (g_ms > 0) printf("graph of 100 launches: %f ms per launch  GFLOPS (2*nnz*N): %8.2f\n", g_ms, flops2 / (g_ms * 1e6));
    }
    if (o.cold) {
        float *flush = nullptr;
        const size_t fe = (size_t)64 << 20;
        DRV_CUDA(cudaMalloc(&flush, fe * sizeof(float)));
        double cmin = 0, cmed = 0;
        DRV_TRY(time_launches(launch, o.reps, flush, fe, &cmin, &cmed));
        printf("cold-L2 median ms: %f  GFLOPS (2*nnz*N): %8.2f  algorithmic GB/s: %8.2f\n", cmed,
               flops2 / (cmed * 1e6), bytes / (cmed * 1e6));
        cudaFree(flush);
    }
    DRV_CUDA(cudaMemcpy(C.data(), d_C, C.size() * sizeof(float), cudaMemcpyDeviceToHost));
    printf("checksum_gpu = %.7g\n", mean_square(C.data(), C.size()));
    Diff d;
    if (o.check) {
        d = compare_rows(Ccpu.data(), C.data(), M, check_stride(o, M), [&](int i) { return (size_t)i * N; },
                         [&](int i) { return (size_t)(i + 1) * N; });
        printf("maxi = %zu max_diff = %g max_rel_diff = %g\n", d.maxi, d.max_diff, d.max_rel_diff);
        if (!C.empty()) {
            printf("output_cpu[%zu] = %.7g\n", d.maxi, Ccpu[d.maxi]);
            printf("output_gpu[%zu] = %.7g\n\n", d.maxi, C[d.maxi]);
        }
    }
    if (!o.csv.empty()) {
        FILE *f = fopen(o.csv.c_str(), "a");
        if (f) {
            fprintf(f, "%d,%d,%d,%g,%g,%g,%g\n", M, N, K, density, gflops, d.max_diff, opcount);
            fclose(f);
        }
    }
    if (plan) dlspm_plan_destroy(plan);
    cudaFree(d_ro); cudaFree(d_ci); cudaFree(d_v); cudaFree(d_B); cudaFree(d_C);
    return DLSPM_OK;
}

// ---- one SDDMM case (SDDMM/sddmm-esimd-fromfile_v4.cpp:91-242; CSV: M,K,N,density,gflops,flops,max_diff)
inline int run_sddmm_case(dlspm_ctx *ctx, const Options &o, int M, int K, int N, const std::vector<int> &ro,
                          const std::vector<int> &ci)
{
    const int nnz = (int)ci.size();
    std::vector<float> lhs((size_t)M * N), rhs((size_t)K * N), out((size_t)nnz, 0.f), out_cpu;
    const int kind = o.signed_values ? 0 : 1;
    dlspm_gen_dense_host(lhs.data(), lhs.size(), o.seed, 11, 0, kind);
    dlspm_gen_dense_host(rhs.data(), rhs.size(), o.seed, 12, 0, kind);
    if (o.check) {
        out_cpu.assign((size_t)nnz, 0.f);
        check_sddmm(ro.data(), ci.data(), lhs.data(), rhs.data(), out_cpu.data(), M, N, check_stride(o, M));
        if (check_stride(o, M) > 1) printf("host check on every %d-th row\n", check_stride(o, M));
    }
    int *d_ro = to_device(ro), *d_ci = to_device(ci);
    float *d_l = to_device(lhs), *d_r = to_device(rhs), *d_o = to_device(out);
    if (!d_ro || !d_ci || !d_l || !d_r || !d_o) {
        printf("device allocation failed\n");
        return DLSPM_ERR_NOMEM;
    }
    auto launch = [&]() { return dlspm_sddmm_csr_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_l, d_r, d_o, launch_stream()); };
    double min_ms = 0, med_ms = 0;
    DRV_TRY(time_launches(launch, o.reps, nullptr, 0, &min_ms, &med_ms));
    printf("MSZ = %d,  NSZ = %d  KSZ = %d\n", M, N, K);
    printf("Total kernel time was %f ms.\n", min_ms);
    const double flops = (double)nnz * (2.0 * N - 1.0);  // the reference's count
    const double gflops1 = flops / (min_ms * 1.0E+6);
    printf("GFLOPS :  %8.2f\n", gflops1);
    const double bytes = 4.0 * (M + 1) + 8.0 * nnz + 4.0 * (double)M * N + 4.0 * (double)K * N;
    printf("GFLOPS (2*nnz*N): %8.2f  algorithmic GB/s: %8.2f  median ms: %f\n", 2.0 * nnz * N / (min_ms * 1e6),
           bytes / (min_ms * 1e6), med_ms);
    if (o.graph || min_ms < 0.010) {
        double g_ms = 0;
        DRV_TRY(time_graph(launch, 100, &g_ms));
        if (g_ms > 0) printf("graph of 100 launches: %f ms per launch  GFLOPS (2*nnz*N): %8.2f\n", g_ms, 2.0 * nnz * N / (g_ms * 1e6));
    }
    if (o.cold) {
        float *flush = nullptr;
        const size_t fe = (size_t)64 << 20;
        DRV_CUDA(cudaMalloc(&flush, fe * sizeof(float)));
        double cmin = 0, cmed = 0;
        DRV_TRY(time_launches(launch, o.reps, flush, fe, &cmin, &cmed));
        printf("cold-L2 median ms: %f  GFLOPS (2*nnz*N): %8.2f  algorithmic GB/s: %8.2f\n", cmed,
               2.0 * nnz * N / (cmed * 1e6), bytes / (cmed * 1e6));
        cudaFree(flush);
    }
    DRV_CUDA(cudaMemcpy(out.data(), d_o, out.size() * sizeof(float), cudaMemcpyDeviceToHost));
    Diff d;
    if (o.check) {
        printf("checksum_cpu = %.7g\n", mean_square(out_cpu.data(), out_cpu.size()));
        printf("checksum_gpu = %.7g\n", mean_square(out.data(), out.size()));
        d = compare_rows(out_cpu.data(), out.data(), M, check_stride(o, M), [&](int i) { return (size_t)ro[(size_t)i]; },
                         [&](int i) { return (size_t)ro[(size_t)i + 1]; });
        printf("maxi = %zu max_diff = %g\n", d.maxi, d.max_diff);
        if (nnz) {
            printf("output_cpu[%zu] = %.7g\n", d.maxi, out_cpu[d.maxi]);
            printf("output_gpu[%zu] = %.7g\n", d.maxi, out[d.maxi]);
        }
    } else {
        printf("checksum_gpu = %.7g\n", mean_square(out.data(), out.size()));
    }
    if (!o.csv.empty()) {
        FILE *f = fopen(o.csv.c_str(), "a");
        if (f) {
            fprintf(f, "%d,%d,%d,%g,%g,%g,%g\n", M, K, N, (double)nnz / ((double)M * K), gflops1, flops, d.max_diff);
            fclose(f);
        }
    }
    cudaFree(d_ro); cudaFree(d_ci); cudaFree(d_l); cudaFree(d_r); cudaFree(d_o);
    return DLSPM_OK;
}

// ---- one fused case (FUSED/fused-esimd_cb.cpp:261-366): inputs scaled by 0.01 as there ------------
inline int run_fused_case(dlspm_ctx *ctx, const Options &o, int M, int K, int N, const std::vector<int> &ro,
                          const std::vector<int> &ci)
{
    const int nnz = (int)ci.size();
    std::vector<float> c((size_t)M * N), b((size_t)K * N), dd((size_t)K * N), e((size_t)M * N, 0.f), e_gold, a_values;
    const int kind = o.signed_values ? 0 : 1;
    dlspm_gen_dense_host(c.data(), c.size(), o.seed, 11, 0, kind);
    dlspm_gen_dense_host(b.data(), b.size(), o.seed, 12, 0, kind);
    dlspm_gen_dense_host(dd.data(), dd.size(), o.seed, 13, 0, kind);
    for (auto &x : c) x *= 0.01f;
    for (auto &x : b) x *= 0.01f;
    for (auto &x : dd) x *= 0.01f;
    if (o.check) {
        a_values.resize((size_t)nnz);
        e_gold.resize((size_t)M * N);
        const int stride = check_stride(o, M);
        if (stride > 1) printf("host check on every %d-th row\n", stride);
        std::fill(a_values.begin(), a_values.end(), 0.f);
        std::fill(e_gold.begin(), e_gold.end(), 0.f);
        check_sddmm(ro.data(), ci.data(), c.data(), b.data(), a_values.data(), M, N, stride);
        printf("checksum_a_values = %f\n", sqrt(mean_square(a_values.data(), a_values.size())));
        if (o.attention) {  // weights from the sampled products: scale, then softmax over each row
            for (int i = 0; i < M; i++) {
                double top = -INFINITY, sum = 0.0;
                for (int p = ro[(size_t)i]; p < ro[(size_t)i + 1]; p++) top = std::max(top, (double)a_values[(size_t)p] * o.scale);
                for (int p = ro[(size_t)i]; p < ro[(size_t)i + 1]; p++) {
                    const double s = (double)a_values[(size_t)p] * o.scale;
                    a_values[(size_t)p] = (float)(o.softmax ? exp(s - top) : s);
                    sum += a_values[(size_t)p];
                }
                if (o.softmax)
                    for (int p = ro[(size_t)i]; p < ro[(size_t)i + 1]; p++) a_values[(size_t)p] = (float)(a_values[(size_t)p] / sum);
            }
        }
        check_spmm_f64(a_values.data(), ro.data(), ci.data(), dd.data(), e_gold.data(), M, N, stride);
        printf("checksum_e = %f\n", sqrt(mean_square(e_gold.data(), e_gold.size())));
    }
    int *d_ro = to_device(ro), *d_ci = to_device(ci);
    float *d_c = to_device(c), *d_b = to_device(b), *d_d = to_device(dd), *d_e = to_device(e);
    if (!d_ro || !d_ci || !d_c || !d_b || !d_d || !d_e) {
        printf("device allocation failed\n");
        return DLSPM_ERR_NOMEM;
    }
    printf("copy to device completed\n");
    printf("Start kernel execution\n");
    auto launch = [&]() {
        if (o.attention)
            return dlspm_fused_attention_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_c, d_b, d_d, d_e, o.scale,
                                             o.softmax ? DLSPM_ATTN_SOFTMAX : 0u, launch_stream());
        return dlspm_fused_sddmm_spmm_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_c, d_b, d_d, d_e, launch_stream());
    };
    double min_ms = 0, med_ms = 0;
    DRV_TRY(time_launches(launch, o.reps, nullptr, 0, &min_ms, &med_ms));
    printf("MSZ = %d,  NSZ = %d  KSZ = %d  SP = %f\n", M, N, K, (double)nnz / ((double)M * K));
    printf("Total kernel time was %f ms.\n", min_ms);
    const float opcount1 = (2 * (float)nnz - M) * N;
    const float opcount2 = (float)((double)nnz * (2.0 * N - 1.0));
    const double gflops1 = (opcount1 + opcount2) / (min_ms * 1.0E+6);
    printf("GFLOPS/s :  %8.2f\n", gflops1);
    const double bytes = 4.0 * (M + 1) + 4.0 * nnz + 4.0 * N * ((double)M + 2.0 * K) + 4.0 * (double)M * N;
    printf("GFLOPS (4*nnz*N): %8.2f  algorithmic GB/s: %8.2f  median ms: %f\n", 4.0 * nnz * N / (min_ms * 1e6),
           bytes / (min_ms * 1e6), med_ms);
    if (o.graph || min_ms < 0.010) {
        double g_ms = 0;
        DRV_TRY(time_graph(launch, 100, &g_ms));
        if (g_ms > 0) printf("graph of 100 launches: %f ms per launch  GFLOPS (4*nnz*N): %8.2f\n", g_ms, 4.0 * nnz * N / (g_ms * 1e6));
    }
    DRV_CUDA(cudaMemcpy(e.data(), d_e, e.size() * sizeof(float), cudaMemcpyDeviceToHost));
    printf("checksum_e using gpu = %f\n", sqrt(mean_square(e.data(), e.size())));
    Diff d;
    if (o.check) {
        d = compare_rows(e_gold.data(), e.data(), M, check_stride(o, M), [&](int i) { return (size_t)i * N; },
                         [&](int i) { return (size_t)(i + 1) * N; });
        printf("maxi = %zu max_diff = %g\n", d.maxi, d.max_diff);
        if (!e.empty()) {
            printf("gold output[%zu] = %.7g\n", d.maxi, e_gold[d.maxi]);
            printf("computed[%zu] = %.7g\n", d.maxi, e[d.maxi]);
        }
    }
    if (!o.csv.empty()) {
        FILE *f = fopen(o.csv.c_str(), "a");
        if (f) {
            fprintf(f, "%d,%d,%d,%g,%g,%g\n", M, K, N, (double)nnz / ((double)M * K), gflops1, d.max_diff);
            fclose(f);
        }
    }
    cudaFree(d_ro); cudaFree(d_ci); cudaFree(d_c); cudaFree(d_b); cudaFree(d_d); cudaFree(d_e);
    return DLSPM_OK;
}

// Bernoulli pattern with the reference's capacity rule (1.01*M*K*SP + 100 entries,
// SPMM/spmm-esimd-allbenchs2.cpp:59).
inline int make_bernoulli(int M, int K, double density, uint64_t seed, std::vector<int> &ro, std::vector<int> &ci)
{
    const size_t cap = (size_t)(1.05 * M * (double)K * density) + 4096;
    ro.assign((size_t)M + 1, 0);
    ci.assign(cap, 0);
    int nnz = 0;
    int rc = dlspm_gen_bernoulli_csr_host(M, K, density, seed, ro.data(), ci.data(), cap, &nnz);
    if (rc != DLSPM_OK) return rc;
    ci.resize((size_t)nnz);
    printf("nnz = %d mnnz = %zu\n", nnz, cap);
    return DLSPM_OK;
}

// Reads a pattern file and validates it, printing what the reference prints on failure.  With
// `cache`, a binary copy "<path>.csrbin" is read instead when it exists and is intact, and written
// after a successful text parse otherwise.  `values` (optional) receives the file's values block,
// or stays empty if the file has none.
inline int load_smtx(const std::string &path, int N, int *M, int *K, std::vector<int> &ro, std::vector<int> &ci,
                     bool cache = false, std::vector<float> *values = nullptr)
{
    int nnz = 0, *pro = nullptr, *pci = nullptr;
    float *pva = nullptr;
    const std::string bin = path + ".csrbin";
    int rc = DLSPM_ERR_IO;
    bool from_cache = false;
    if (cache) {
        rc = dlspm_read_csr_cache_host(bin.c_str(), M, K, &nnz, &pro, &pci, &pva);
        from_cache = rc == DLSPM_OK;
        if (from_cache) printf("read %s\n", bin.c_str());
    }
    if (!from_cache) rc = dlspm_read_smtx_values_host(path.c_str(), M, K, &nnz, &pro, &pci, &pva);
    if (rc == DLSPM_ERR_IO) {
        printf("Error opening file!\n");
        return rc;
    }
    if (rc != DLSPM_OK) {
        printf("Something went wrong reading %s: %s\n", path.c_str(), dlspm_strerror(rc));
        return rc;
    }
    printf("MSZ: %d, KSZ: %d, NSZ: %d, nnz: %d\n", *M, *K, N, nnz);
    ro.assign(pro, pro + *M + 1);
    ci.assign(pci, pci + nnz);
    if (values) {
        values->clear();
        if (pva) values->assign(pva, pva + nnz);
    }
    dlspm_free_host(pro);
    dlspm_free_host(pci);
    dlspm_free_host(pva);
    char why[128];
    rc = dlspm_sanity_check_csr_host(*M, *K, N, nnz, ro.data(), ci.data(), why, sizeof(why));
    if (rc != DLSPM_OK) {
        printf("%s\n", why);
        return rc;
    }
    if (cache && !from_cache) {
        const bool has_values = values && !values->empty();
        if (dlspm_write_csr_cache_host(bin.c_str(), *M, *K, nnz, ro.data(), ci.data(), has_values ? values->data() : nullptr) == DLSPM_OK)
            printf("wrote %s\n", bin.c_str());
    }
    return rc;
}

// Lines "<pattern file> <batchsize>" of a list file (for --list: one process, one context, many files).
inline bool read_list(const std::string &path, std::vector<std::pair<std::string, int>> &items)
{
    FILE *f = fopen(path.c_str(), "r");
    if (!f) {
        printf("Error opening file!\n");
        return false;
    }
    char name[4096];
    int n = 0;
    while (fscanf(f, "%4095s %d", name, &n) == 2) items.emplace_back(name, n);
    fclose(f);
    return true;
}

}  // namespace drv
