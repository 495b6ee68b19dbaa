// Synthetic SpMM sweep: ./spmm-allbenchs [options]
// Without arguments runs the reference's grid (SPMM/spmm-esimd-allbenchs2.cpp:259-273): 12 (M, K)
// pairs x density {0.3, 0.2, 0.1} x N {32, 128}.  --sweep dlmc runs the pruned-weight grid instead:
// 5 shapes x sparsity {0.5 .. 0.98} x N {256, 1024, 3136} with Normal row lengths (CoV 0.4).
// One case only: ./spmm-allbenchs <M> <K> <N> <density>
#include "driver_common.hpp"

static int one_case(dlspm_ctx *ctx, const drv::Options &o, int M, int K, int N, double density)
{
    std::vector<int> ro, ci;
    int rc = drv::make_bernoulli(M, K, density, o.seed, ro, ci);
    if (rc != DLSPM_OK) return rc;
    return drv::run_spmm_case(ctx, o, M, K, N, ro, ci);
}

static int one_case_rowlen(dlspm_ctx *ctx, const drv::Options &o, int M, int K, int N, double sparsity)
{
    std::vector<int> ro((size_t)M + 1);
    int rc = dlspm_gen_rowlen_normal_host(M, K, sparsity, 0.4, o.seed, ro.data());
    if (rc != DLSPM_OK) return rc;
    std::vector<int> ci((size_t)ro[(size_t)M]);
    rc = dlspm_gen_sample_columns_host(M, K, ro.data(), o.seed, ci.data());
    if (rc != DLSPM_OK) return rc;
    printf("nnz = %d sparsity = %g\n", ro[(size_t)M], sparsity);
    return drv::run_spmm_case(ctx, o, M, K, N, ro, ci);
}

int main(int argc, char **argv)
{
    bool dlmc = false;
    std::vector<char *> rest;
    for (int i = 0; i < argc; i++) {
        if (std::string(argv[i]) == "--sweep" && i + 1 < argc) dlmc = std::string(argv[++i]) == "dlmc";
        else rest.push_back(argv[i]);
    }
    drv::Options o = drv::parse((int)rest.size(), rest.data());
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    drv::print_device(ctx);
    int rc = DLSPM_OK;
    if (o.positional.size() == 4) {
        rc = one_case(ctx, o, atoi(o.positional[0].c_str()), atoi(o.positional[1].c_str()),
                      atoi(o.positional[2].c_str()), atof(o.positional[3].c_str()));
    } else if (dlmc) {
        const int shapes[5][2] = {{64, 64}, {256, 256}, {512, 2048}, {2048, 512}, {1024, 4096}};
        const double sparsities[6] = {0.5, 0.7, 0.8, 0.9, 0.95, 0.98};
        const int widths[3] = {256, 1024, 3136};
        for (int N : widths)
            for (auto &s : shapes)
                for (double sp : sparsities)
                    if ((rc = one_case_rowlen(ctx, o, s[0], s[1], N, sp)) != DLSPM_OK) break;
    } else {
        const int MSZ_arr[12] = {1024, 3072, 4096, 2048, 6144, 8192, 4096, 12288, 16384, 8192, 24576, 32768};
        const int KSZ_arr[12] = {1024, 1024, 1024, 2048, 2048, 2048, 4096, 4096, 4096, 8192, 8192, 8192};
        const int NSZ_arr[2] = {32, 128};
        const double SP_arr[3] = {0.3, 0.2, 0.1};
        for (int N : NSZ_arr)
            for (int c = 0; c < 12; c++)
                for (double sp : SP_arr)
                    if ((rc = one_case(ctx, o, MSZ_arr[c], KSZ_arr[c], N, sp)) != DLSPM_OK) break;
    }
    dlspm_destroy(ctx);
    return rc;
}
