// Entry points that take HOST buffers: copy in, run the device entry point, copy out.  These are the
// calls a program that keeps its matrices in host memory binds to, as the reference drivers do
// around their kernels (explicit memcpy before and after, SPMM/spmm-esimd-fromfile.cpp:172-180,255).
// Device staging memory belongs to the context and is reused between calls.  Pinned host memory
// makes the copies asynchronous DMA; pageable memory works too.
#include <vector>

#include "common.cuh"

namespace {

struct Carver {
    char *base;
    size_t off;
    explicit Carver(void *b) : base((char *)b), off(0) {}
    template <typename T>
    T *take(size_t n)
    {
        T *p = (T *)(base + off);
        off += (n * sizeof(T) + 255) & ~(size_t)255;
        return p;
    }
};

inline size_t padded(size_t bytes) { return (bytes + 255) & ~(size_t)255; }

}  // namespace

extern "C" int dlspm_spmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                                       const int *row_offsets, const int *column_indices, const float *B,
                                       float *C)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && (!values || !column_indices)) || ((size_t)K * N > 0 && !B) ||
        ((size_t)M * N > 0 && !C))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nB = (size_t)K * N, nC = (size_t)M * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + 2 * padded(4 * (size_t)nnz) + padded(4 * nB) +
                                      padded(4 * nC) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_v = cv.take<float>((size_t)nnz);
    float *d_B = cv.take<float>(nB);
    float *d_C = cv.take<float>(nC);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) {
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_v, values, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    }
    if (nB) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, B, 4 * nB, cudaMemcpyHostToDevice, st));
    rc = dlspm_spmm_csr_f32(ctx, M, K, N, nnz, d_v, d_ro, d_ci, d_B, d_C, st);
    if (rc) return rc;
    if (nC) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(C, d_C, 4 * nC, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

extern "C" int dlspm_sddmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                                        const int *column_indices, const float *lhs, const float *rhs,
                                        float *out_values)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && (!column_indices || !out_values)) || ((size_t)M * N > 0 && !lhs) ||
        ((size_t)K * N > 0 && !rhs))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nL = (size_t)M * N, nR = (size_t)K * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + 2 * padded(4 * (size_t)nnz) + padded(4 * nL) +
                                      padded(4 * nR) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_out = cv.take<float>((size_t)nnz);
    float *d_L = cv.take<float>(nL);
    float *d_R = cv.take<float>(nR);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    if (nL) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_L, lhs, 4 * nL, cudaMemcpyHostToDevice, st));
    if (nR) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_R, rhs, 4 * nR, cudaMemcpyHostToDevice, st));
    rc = dlspm_sddmm_csr_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_L, d_R, d_out, st);
    if (rc) return rc;
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(out_values, d_out, 4 * (size_t)nnz, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

extern "C" int dlspm_fused_sddmm_spmm_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                               const int *row_offsets, const int *column_indices,
                                               const float *C, const float *B, const float *D, float *E)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && !column_indices) || ((size_t)M * N > 0 && (!C || !E)) ||
        ((size_t)K * N > 0 && (!B || !D)))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nM = (size_t)M * N, nK = (size_t)K * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + padded(4 * (size_t)nnz) + 2 * padded(4 * nM) +
                                      2 * padded(4 * nK) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_C = cv.take<float>(nM);
    float *d_E = cv.take<float>(nM);
    float *d_B = cv.take<float>(nK);
    float *d_D = cv.take<float>(nK);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    if (nM) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_C, C, 4 * nM, cudaMemcpyHostToDevice, st));
    if (nK) {
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, B, 4 * nK, cudaMemcpyHostToDevice, st));
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_D, D, 4 * nK, cudaMemcpyHostToDevice, st));
    }
    rc = dlspm_fused_sddmm_spmm_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_C, d_B, d_D, d_E, st);
    if (rc) return rc;
    if (nM) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(E, d_E, 4 * nM, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

// Batched SpMM with host pointers.  The batch is cut into pieces whose device copies fit a staging
// budget; each piece is copied in, run as one grouped launch, and its C blocks copied out.
extern "C" int dlspm_spmm_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_problem *problems)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t budget = (size_t)4 << 30;
    auto need = [](const dlspm_problem &q) {
        return padded(4 * ((size_t)q.M + 1)) + 2 * padded(4 * (size_t)q.nnz) + padded(4 * (size_t)q.K * q.N) +
               padded(4 * (size_t)q.M * q.N);
    };
    for (int i = 0; i < count; i++) {
        const dlspm_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || q.nnz < 0 || !q.row_offsets ||
            (q.nnz > 0 && (!q.values || !q.column_indices)) || ((size_t)q.K * q.N > 0 && !q.B) ||
            ((size_t)q.M * q.N > 0 && !q.C))
            return DLSPM_ERR_INVALID_ARGUMENT;
    }
    cudaStream_t st = ctx->stream;
    std::vector<dlspm_problem> dev;
    int first = 0;
    while (first < count) {
        size_t bytes = 0;
        int last = first;
        while (last < count && (last == first || bytes + need(problems[last]) <= budget)) {
            bytes += need(problems[last]);
            last++;
        }
        rc = dlspm_stage_reserve(ctx, bytes + 256);
        if (rc) return rc;
        Carver cv(ctx->stage);
        dev.clear();
        for (int i = first; i < last; i++) {
            const dlspm_problem &q = problems[i];
            dlspm_problem d = q;
            int *d_ro = cv.take<int>((size_t)q.M + 1);
            int *d_ci = cv.take<int>((size_t)q.nnz);
            float *d_v = cv.take<float>((size_t)q.nnz);
            float *d_B = cv.take<float>((size_t)q.K * q.N);
            float *d_C = cv.take<float>((size_t)q.M * q.N);
            DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, q.row_offsets, 4 * ((size_t)q.M + 1), cudaMemcpyHostToDevice, st));
            if (q.nnz) {
                DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, q.column_indices, 4 * (size_t)q.nnz, cudaMemcpyHostToDevice, st));
                DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_v, q.values, 4 * (size_t)q.nnz, cudaMemcpyHostToDevice, st));
            }
            if ((size_t)q.K * q.N > 0) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, q.B, 4 * (size_t)q.K * q.N, cudaMemcpyHostToDevice, st));
            d.row_offsets = d_ro;
            d.column_indices = d_ci;
            d.values = d_v;
            d.B = d_B;
            d.C = d_C;
            dev.push_back(d);
        }
        rc = dlspm_spmm_batched_f32(ctx, (int)dev.size(), dev.data(), st);
        if (rc) return rc;
        for (int i = first; i < last; i++) {
            const dlspm_problem &q = problems[i];
            const size_t nC = (size_t)q.M * q.N;
            if (nC) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(q.C, dev[(size_t)(i - first)].C, 4 * nC, cudaMemcpyDeviceToHost, st));
        }
        DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
        first = last;
    }
    return DLSPM_OK;
}
