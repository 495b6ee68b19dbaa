// SDDMM from a pattern file: ./sddmm-fromfile <filename>.smtx <batchsize> [options]
// Same command line and report as the reference driver (SDDMM/sddmm-esimd-fromfile_v4.cpp:38-46);
// <batchsize> is the inner (dot-product) dimension.  --check-rows k: the host loop checks about k
// evenly spaced rows; --list file: run every "<filename> <batchsize>" line in this one process.
#include "driver_common.hpp"

int main(int argc, char **argv)
{
    drv::Options o = drv::parse(argc, argv);
    std::vector<std::pair<std::string, int>> items;
    if (!o.list.empty()) {
        if (!drv::read_list(o.list, items)) return 0;
    } else if (o.positional.size() == 2) {
        items.emplace_back(o.positional[0], atoi(o.positional[1].c_str()));
    } else {
        printf("Usage: ./app <filename>.smtx <batchsize>\n");
        return 0;
    }
    dlspm_ctx *ctx = nullptr;
    DRV_TRY(dlspm_create(&ctx, o.device));
    int rc = DLSPM_OK;
    for (const auto &item : items) {  // one file, or every line of --list in this one process
        const std::string &filename = item.first;
        const int N = item.second;
        printf("Filename = %s, batchsize (=NSZ) = %d\n", filename.c_str(), N);
        drv::print_device(ctx);
        int M = 0, K = 0;
        std::vector<int> ro, ci;
        rc = drv::load_smtx(filename, N, &M, &K, ro, ci, o.cache);
        if (rc == DLSPM_OK) rc = drv::run_sddmm_case(ctx, o, M, K, N, ro, ci);
        fflush(stdout);
    }
    dlspm_destroy(ctx);
    return rc;
}
