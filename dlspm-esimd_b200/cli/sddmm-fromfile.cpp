// SDDMM from a pattern file: ./sddmm-fromfile <filename>.smtx <batchsize> [options]
// Same command line and report as the reference driver (SDDMM/sddmm-esimd-fromfile_v4.cpp:38-46);
// <batchsize> is the inner (dot-product) dimension.
#include "driver_common.hpp"

int main(int argc, char **argv)
{
    drv::Options o = drv::parse(argc, argv);
    if (o.positional.size() != 2) {
        printf("Usage: ./app <filename>.smtx <batchsize>\n");
        return 0;
    }
    const std::string filename = o.positional[0];
    const int N = atoi(o.positional[1].c_str());
    printf("Filename = %s, batchsize (=NSZ) = %d\n", filename.c_str(), N);
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    drv::print_device(ctx);
    int M = 0, K = 0;
    std::vector<int> ro, ci;
    int rc = drv::load_smtx(filename, N, &M, &K, ro, ci, o.cache);
    if (rc == DLSPM_OK) rc = drv::run_sddmm_case(ctx, o, M, K, N, ro, ci);
    dlspm_destroy(ctx);
    return rc;
}
