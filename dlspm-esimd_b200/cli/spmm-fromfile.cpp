// SpMM from a pattern file: ./spmm-fromfile <filename>.smtx <batchsize> [options]
// Same command line and report as the reference driver (SPMM/spmm-esimd-fromfile2.cpp:86-95).
// Options: --reps n, --seed s, --csv file, --no-check, --signed, --planned, --cold, --device d,
// --graph (also time 100 launches in one CUDA graph; automatic below 10 us), --cache (binary copy
// of the parsed file beside it).  A file with a values block (fourth block of
// nnz floats) is multiplied with those values instead of generated ones.
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
    std::vector<float> values;  // taken from the file when it carries a values block
    int rc = drv::load_smtx(filename, N, &M, &K, ro, ci, o.cache, &values);
    if (rc == DLSPM_OK) rc = drv::run_spmm_case(ctx, o, M, K, N, ro, ci, values.empty() ? nullptr : &values);
    dlspm_destroy(ctx);
    return rc;
}
