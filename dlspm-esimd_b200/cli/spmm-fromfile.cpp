// SpMM from a pattern file: ./spmm-fromfile <filename>.smtx <batchsize> [options]
// Same command line and report as the reference driver (SPMM/spmm-esimd-fromfile2.cpp:86-95).
// Options: --reps n, --seed s, --csv file, --no-check, --signed, --planned, --cold, --device d,
// --graph (also time 100 launches in one CUDA graph; automatic below 10 us), --cache (binary copy
// of the parsed file beside it).  A file with a values block (fourth block of
// nnz floats) is multiplied with those values instead of generated ones.
// --check-rows k: the host loop checks about k evenly spaced rows; --list file: run every
// "<filename> <batchsize>" line of the file in this one process (what the batch script uses).
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
        std::vector<float> values;  // taken from the file when it carries a values block
        rc = drv::load_smtx(filename, N, &M, &K, ro, ci, o.cache, &values);
        if (rc == DLSPM_OK) rc = drv::run_spmm_case(ctx, o, M, K, N, ro, ci, values.empty() ? nullptr : &values);
        fflush(stdout);
    }
    dlspm_destroy(ctx);
    return rc;
}
