// Fused SDDMM -> SpMM on a synthetic pattern: ./fused <MSZ> <KSZ> <NSZ> <SP> [options]
// The reference fixes these four at compile time (-DMSZ -DKSZ -DNSZ -DSP,
// FUSED/batch-run-fused:29); here they are run-time arguments with the same meaning (SP is the
// fraction of nonzeros).  --band h adds a band of half-width h around the diagonal; --scale x and
// --softmax run the sparse-attention form (scaled products, row softmax) instead of the plain chain.
#include "driver_common.hpp"

int main(int argc, char **argv)
{
    int half_band = -1;
    std::vector<char *> rest;
    for (int i = 0; i < argc; i++) {
        if (std::string(argv[i]) == "--band" && i + 1 < argc) half_band = atoi(argv[++i]);
        else rest.push_back(argv[i]);
    }
    drv::Options o = drv::parse((int)rest.size(), rest.data());
    if (o.positional.size() != 4) {
        printf("Usage: ./fused <MSZ> <KSZ> <NSZ> <SP> [--band h] [--scale x] [--softmax]\n");
        return 0;
    }
    const int M = atoi(o.positional[0].c_str()), K = atoi(o.positional[1].c_str()), N = atoi(o.positional[2].c_str());
    const double SP = atof(o.positional[3].c_str());
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    drv::print_device(ctx);
    std::vector<int> ro, ci;
    int rc;
    if (half_band >= 0) {
        const size_t cap = (size_t)((double)M * (2 * half_band + 1 + 1.05 * K * SP)) + 4096;
        ro.assign((size_t)M + 1, 0);
        ci.assign(cap, 0);
        int nnz = 0;
        rc = dlspm_gen_band_csr_host(M, K, half_band, SP, o.seed, ro.data(), ci.data(), cap, &nnz);
        ci.resize((size_t)nnz);
    } else {
        rc = drv::make_bernoulli(M, K, SP, o.seed, ro, ci);
    }
    printf("MSZ = %d KSZ = %d NSZ = %d SP = %f\n", M, K, N, SP);
    if (rc == DLSPM_OK) rc = drv::run_fused_case(ctx, o, M, K, N, ro, ci);
    dlspm_destroy(ctx);
    return rc;
}
