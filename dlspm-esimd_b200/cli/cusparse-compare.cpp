// cuSPARSE beside this library on the same inputs: ./cusparse-compare spmm|sddmm <M> <K> <N> <density>
// or, for the 72 cases of the reference's comparison grid in one process: ./cusparse-compare spmm|sddmm grid
// Comparison only, as in the reference (CUSPARSE/spmm.cu, CUSPARSE/sddmm.cu): cusparseSpMM and
// cusparseSDDMM with ALG_DEFAULT on row-major fp32 operands, minimum of 20 event-timed runs, next
// to dlspm_spmm_csr_f32 / dlspm_sddmm_csr_f32 timed the same way, plus the largest difference
// between the two results.  libdlspm.so itself never links or calls cuSPARSE.
#include <cusparse.h>

#include "driver_common.hpp"

#define CUSP(call)                                                               \
    do {                                                                         \
        cusparseStatus_t s__ = (call);                                           \
        if (s__ != CUSPARSE_STATUS_SUCCESS) {                                    \
            printf("%s failed: %s\n", #call, cusparseGetErrorString(s__));       \
            return 3;                                                            \
        }                                                                        \
    } while (0)

// One comparison: the same CSR pattern and dense operands through cuSPARSE and through this library.
static int compare_case(dlspm_ctx *ctx, const drv::Options &o, bool spmm, int M, int K, int N, double density)
{
    std::vector<int> ro, ci;
    DRV_TRY(drv::make_bernoulli(M, K, density, o.seed, ro, ci));
    const int nnz = (int)ci.size();
    const int kind = o.signed_values ? 0 : 1;
    std::vector<float> vals((size_t)nnz), dense_k((size_t)K * N), dense_m((size_t)M * N);
    dlspm_gen_dense_host(vals.data(), vals.size(), o.seed, 2, 0, kind);
    dlspm_gen_dense_host(dense_k.data(), dense_k.size(), o.seed, spmm ? 10 : 12, 0, kind);
    dlspm_gen_dense_host(dense_m.data(), dense_m.size(), o.seed, 11, 0, kind);
    int *d_ro = drv::to_device(ro), *d_ci = drv::to_device(ci);
    float *d_vals = drv::to_device(vals), *d_k = drv::to_device(dense_k), *d_m = drv::to_device(dense_m);
    std::vector<float> zeros_out(spmm ? (size_t)M * N : (size_t)nnz, 0.f);
    float *d_ours = drv::to_device(zeros_out), *d_theirs = drv::to_device(zeros_out);
    if (!d_ro || !d_ci || !d_vals || !d_k || !d_m || !d_ours || !d_theirs) {
        printf("device allocation failed\n");
        return DLSPM_ERR_NOMEM;
    }

    cusparseHandle_t handle = nullptr;
    CUSP(cusparseCreate(&handle));
    const float alpha = 1.0f, beta = 0.0f;
    cusparseSpMatDescr_t matA;
    cusparseDnMatDescr_t matK, matM;
    // sparse operand: values for SpMM, the output for SDDMM
    CUSP(cusparseCreateCsr(&matA, M, K, nnz, d_ro, d_ci, spmm ? d_vals : d_theirs, CUSPARSE_INDEX_32I,
                           CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
    CUSP(cusparseCreateDnMat(&matK, K, N, N, d_k, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    CUSP(cusparseCreateDnMat(&matM, M, N, N, spmm ? d_theirs : d_m, CUDA_R_32F, CUSPARSE_ORDER_ROW));
    size_t buffer_size = 0;
    void *d_buffer = nullptr;
    if (spmm) {
        CUSP(cusparseSpMM_bufferSize(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                                     matA, matK, &beta, matM, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, &buffer_size));
    } else {
        CUSP(cusparseSDDMM_bufferSize(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_TRANSPOSE, &alpha,
                                      matM, matK, &beta, matA, CUDA_R_32F, CUSPARSE_SDDMM_ALG_DEFAULT, &buffer_size));
    }
    DRV_CUDA(cudaMalloc(&d_buffer, buffer_size ? buffer_size : 16));
    cusparseStatus_t last = CUSPARSE_STATUS_SUCCESS;
    auto theirs = [&]() {
        last = spmm ? cusparseSpMM(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                                   matA, matK, &beta, matM, CUDA_R_32F, CUSPARSE_SPMM_ALG_DEFAULT, d_buffer)
                    : cusparseSDDMM(handle, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_TRANSPOSE, &alpha,
                                    matM, matK, &beta, matA, CUDA_R_32F, CUSPARSE_SDDMM_ALG_DEFAULT, d_buffer);
        return last == CUSPARSE_STATUS_SUCCESS ? DLSPM_OK : DLSPM_ERR_CUDA;
    };
    auto ours = [&]() {
        return spmm ? dlspm_spmm_csr_f32(ctx, M, K, N, nnz, d_vals, d_ro, d_ci, d_k, d_ours, nullptr)
                    : dlspm_sddmm_csr_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_m, d_k, d_ours, nullptr);
    };
    double t_min = 0, t_med = 0, o_min = 0, o_med = 0;
    DRV_TRY(drv::time_launches(theirs, o.reps, nullptr, 0, &t_min, &t_med));
    DRV_TRY(drv::time_launches(ours, o.reps, nullptr, 0, &o_min, &o_med));
    const double flops = 2.0 * nnz * (double)N;
    printf("%s MSZ = %d KSZ = %d NSZ = %d SP = %f nnz = %d\n", spmm ? "spmm" : "sddmm", M, K, N, density, nnz);
    printf("cuSPARSE  kernel time in ms: %f  GFLOPS (2*nnz*N): %8.2f  (buffer %zu bytes)\n", t_min, flops / (t_min * 1e6), buffer_size);
    printf("dlspm     kernel time in ms: %f  GFLOPS (2*nnz*N): %8.2f\n", o_min, flops / (o_min * 1e6));
    printf("speedup over cuSPARSE: %.2f\n", t_min / o_min);
    std::vector<float> a(zeros_out.size()), b(zeros_out.size());
    DRV_CUDA(cudaMemcpy(a.data(), d_ours, a.size() * sizeof(float), cudaMemcpyDeviceToHost));
    DRV_CUDA(cudaMemcpy(b.data(), d_theirs, b.size() * sizeof(float), cudaMemcpyDeviceToHost));
    drv::Diff d = drv::compare(b.data(), a.data(), a.size());
    printf("maxi = %zu max_diff = %g max_rel_diff = %g\n", d.maxi, d.max_diff, d.max_rel_diff);
    if (!o.csv.empty()) {
        FILE *f = fopen(o.csv.c_str(), "a");
        if (f) {
            fprintf(f, "%s,%d,%d,%d,%g,%g,%g,%g\n", spmm ? "spmm" : "sddmm", M, K, N, (double)nnz / ((double)M * K),
                    flops / (t_min * 1e6), flops / (o_min * 1e6), d.max_diff);
            fclose(f);
        }
    }
    cusparseDestroySpMat(matA);
    cusparseDestroyDnMat(matK);
    cusparseDestroyDnMat(matM);
    cusparseDestroy(handle);
    cudaFree(d_buffer);
    cudaFree(d_ro); cudaFree(d_ci); cudaFree(d_vals); cudaFree(d_k); cudaFree(d_m); cudaFree(d_ours); cudaFree(d_theirs);
    return 0;
}

int main(int argc, char **argv)
{
    drv::Options o = drv::parse(argc, argv);
    const bool grid = o.positional.size() == 2 && o.positional[1] == "grid";
    if ((o.positional.size() != 5 && !grid) || (o.positional[0] != "spmm" && o.positional[0] != "sddmm")) {
        printf("Usage: ./cusparse-compare spmm|sddmm <M> <K> <N> <density>\n       ./cusparse-compare spmm|sddmm grid\n");
        return 0;
    }
    const bool spmm = o.positional[0] == "spmm";
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    drv::print_device(ctx);
    int rc = 0;
    if (grid) {
        // the reference's comparison grid (CUSPARSE/batch-spmm:8-24, the shapes of
        // SPMM/spmm-esimd-allbenchs2.cpp:259-262): 12 (M, K) pairs x density {0.3, 0.2, 0.1} x N {32, 128}
        const int MSZ_arr[12] = {1024, 3072, 4096, 2048, 6144, 8192, 4096, 12288, 16384, 8192, 24576, 32768};
        const int KSZ_arr[12] = {1024, 1024, 1024, 2048, 2048, 2048, 4096, 4096, 4096, 8192, 8192, 8192};
        const int NSZ_arr[2] = {32, 128};
        const double SP_arr[3] = {0.3, 0.2, 0.1};
        for (int N : NSZ_arr)
            for (int c = 0; c < 12 && rc == 0; c++)
                for (double sp : SP_arr)
                    if ((rc = compare_case(ctx, o, spmm, MSZ_arr[c], KSZ_arr[c], N, sp)) != 0) break;
    } else {
        rc = compare_case(ctx, o, spmm, atoi(o.positional[1].c_str()), atoi(o.positional[2].c_str()),
                          atoi(o.positional[3].c_str()), atof(o.positional[4].c_str()));
    }
    dlspm_destroy(ctx);
    return rc;
}
