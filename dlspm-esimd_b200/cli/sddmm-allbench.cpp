// Synthetic SDDMM sweep: ./sddmm-allbench [options]
// Without arguments runs the reference's grid (SDDMM/sddmm-esimd-allbench_v4.cpp:241-255): 12 (M, K)
// pairs x density {0.3, 0.2, 0.1} x inner dimension {32, 128}.
// One case only: ./sddmm-allbench <M> <K> <N> <density>
#include "driver_common.hpp"

static int one_case(dlspm_ctx *ctx, const drv::Options &o, int M, int K, int N, double density)
{
    std::vector<int> ro, ci;
    int rc = drv::make_bernoulli(M, K, density, o.seed, ro, ci);
    if (rc != DLSPM_OK) return rc;
    return drv::run_sddmm_case(ctx, o, M, K, N, ro, ci);
}

int main(int argc, char **argv)
{
    drv::Options o = drv::parse(argc, argv);
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    drv::print_device(ctx);
    int rc = DLSPM_OK;
    if (o.positional.size() == 4) {
        rc = one_case(ctx, o, atoi(o.positional[0].c_str()), atoi(o.positional[1].c_str()),
                      atoi(o.positional[2].c_str()), atof(o.positional[3].c_str()));
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
