// Internal declarations shared by the .cu files of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/dlspm.h"

// staging slots of the pipelined host-buffer calls (copy in, launch, copy out overlap across slots)
constexpr int kPipeSlots = 4;
constexpr int kSideStreams = 11;

struct dlspm_ctx {
    int device;
    int sm_count;
    size_t global_mem;
    char name[256];
    char last_error[512];
    int strict_fp32;  // DLSPM_OPT_STRICT_FP32
    int spmm_kernel;  // DLSPM_OPT_SPMM_KERNEL
    int tile_min_density_permille;  // DLSPM_OPT_TILE_MIN_DENSITY
    int tile_min_density_set;       // the caller has set it (a forced kernel choice honours only an explicit threshold)
    int check_input;                // DLSPM_OPT_CHECK_INPUT
    // Device scratch owned by the context, grown on demand (grouped-launch tables, staging for
    // the host-buffer entry points).  Freed in dlspm_destroy.
    void *scratch;
    size_t scratch_bytes;
    void *stage;  // staging for *_host entry points
    size_t stage_bytes;
    cudaStream_t stream;  // private stream of the *_host entry points (compute)
    // copy streams and events of the pipelined host-buffer batch (created on first use)
    cudaStream_t h2d_stream, d2h_stream;
    cudaEvent_t ev_h2d[kPipeSlots], ev_kernel[kPipeSlots], ev_d2h[kPipeSlots];
    int pipeline_ready;
    void *pinned;  // pinned host memory for the launch tables of the pipelined batch
    size_t pinned_bytes;
    // side streams on which the launches of one grouped SDDMM / fused call run side by side (created
    // on first use); events to fork them from the caller's stream and to join them again
    cudaStream_t side_stream[kSideStreams];
    cudaEvent_t side_fork, side_join[kSideStreams];
    int side_ready;
    long long host_copies;  // cudaMemcpyAsync calls issued by the pipelined host-buffer batch so far
};

struct dlspm_plan {
    dlspm_ctx *ctx;
    int M, K, nnz;
    int *row_order;  // device: rows in decreasing length bins
    int sorted_rows; // 1 if every row's columns are ascending
    int max_row_len;
};

// Records a CUDA failure in the context and returns DLSPM_ERR_CUDA.
int dlspm_cuda_fail(dlspm_ctx *ctx, cudaError_t err, const char *what);

#define DLSPM_CUDA_TRY(ctx, call)                                   \
    do {                                                            \
        cudaError_t err__ = (call);                                 \
        if (err__ != cudaSuccess) return dlspm_cuda_fail((ctx), err__, #call); \
    } while (0)

// Makes the context's device current for the calling thread.
static inline int dlspm_use(dlspm_ctx *ctx)
{
    if (!ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    cudaError_t err = cudaSetDevice(ctx->device);
    if (err != cudaSuccess) return dlspm_cuda_fail(ctx, err, "cudaSetDevice");
    return DLSPM_OK;
}

// DLSPM_OPT_CHECK_INPUT: validates a CSR pattern in device (host) memory when the option is set;
// DLSPM_ERR_CSR with the reason in ctx->last_error, DLSPM_OK when the option is off (context.cu).
int dlspm_check_input(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets, const int *column_indices,
                      cudaStream_t st);
int dlspm_check_input_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                           const int *column_indices);

// Grows ctx->scratch to at least `bytes` (contents are not preserved).
int dlspm_scratch_reserve(dlspm_ctx *ctx, size_t bytes);
int dlspm_stage_reserve(dlspm_ctx *ctx, size_t bytes);

// One-shot grouped launch with caller-provided table memory (spmm.cu).
size_t dlspm_batched_table_bytes(int count);
// `pinned` (optional, host memory of the same size): the tables are built there and copied
// asynchronously; the caller must not reuse it before the launch has finished.
int dlspm_spmm_batched_at(dlspm_ctx *ctx, int count, const dlspm_problem *problems, void *tables, cudaStream_t st,
                          void *pinned = nullptr);

// Grouped SDDMM / fused launches with caller-provided table memory (sddmm_batch.cu).
size_t dlspm_rows_batched_table_bytes(int count);
int dlspm_sddmm_batched_at(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems, void *tables, void *pinned,
                           cudaStream_t st);
int dlspm_fused_batched_at(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems, void *tables, void *pinned,
                           cudaStream_t st);

static inline int dlspm_ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long dlspm_ceil_div64(long long a, long long b) { return (a + b - 1) / b; }

// Widest vector (in floats) usable for rows of `N` floats starting at these base pointers.
static inline int dlspm_vec_width(int N, const void *p0, const void *p1, const void *p2 = nullptr,
                                  const void *p3 = nullptr)
{
    uintptr_t bits = (uintptr_t)p0 | (uintptr_t)p1 | (uintptr_t)p2 | (uintptr_t)p3;
    if ((N % 4 == 0) && (bits % 16 == 0)) return 4;
    if ((N % 2 == 0) && (bits % 8 == 0)) return 2;
    return 1;
}

// Argument check shared by the SpMM entry points.
static inline int check_spmm_args(int M, int K, int N, int nnz, const float *values, const int *row_offsets,
                    const int *cols, const float *B, float *C)
{
    if (M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (M > 0 && !row_offsets) return DLSPM_ERR_INVALID_ARGUMENT;
    if (nnz > 0 && (!values || !cols || !B)) return DLSPM_ERR_INVALID_ARGUMENT;
    if (M > 0 && N > 0 && !C) return DLSPM_ERR_INVALID_ARGUMENT;
    return DLSPM_OK;
}
