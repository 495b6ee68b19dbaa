// One host process driving several devices.  The reference runs on a single device
// (SPMM/batch-run-spmm_fromfile:45 pins one tile); this layer adds the two ways its workloads
// spread over the GPUs of one box: independent matrices of a batch are dealt out by work, and one
// large SpMM is cut into row blocks.  No data moves between devices: every device reads its inputs
// from host memory and writes its part of the result back to host memory.
#include <new>
#include <thread>
#include <vector>

#include "common.cuh"

struct dlspm_mg {
    std::vector<dlspm_ctx *> ctxs;
};

extern "C" int dlspm_mg_create(dlspm_mg **out, int ndev, const int *devices)
{
    if (!out || ndev < 1) return DLSPM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    dlspm_mg *mg = new (std::nothrow) dlspm_mg();
    if (!mg) return DLSPM_ERR_NOMEM;
    for (int i = 0; i < ndev; i++) {
        dlspm_ctx *c = nullptr;
        int rc = dlspm_create(&c, devices ? devices[i] : i);
        if (rc) {
            dlspm_mg_destroy(mg);
            return rc;
        }
        mg->ctxs.push_back(c);
    }
    *out = mg;
    return DLSPM_OK;
}

extern "C" int dlspm_mg_destroy(dlspm_mg *mg)
{
    if (!mg) return DLSPM_OK;
    for (dlspm_ctx *c : mg->ctxs) dlspm_destroy(c);
    delete mg;
    return DLSPM_OK;
}

extern "C" int dlspm_mg_device_count(const dlspm_mg *mg) { return mg ? (int)mg->ctxs.size() : 0; }

extern "C" int dlspm_mg_spmm_batched_f32_host(dlspm_mg *mg, int count, const dlspm_problem *problems)
{
    if (!mg || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    const int parts = (int)mg->ctxs.size();
    std::vector<double> w((size_t)count);
    for (int i = 0; i < count; i++) w[(size_t)i] = (double)problems[i].nnz * (double)problems[i].N;
    std::vector<int> owner((size_t)count);
    int rc = dlspm_partition_lpt_host(count, w.data(), parts, owner.data());
    if (rc) return rc;
    std::vector<std::vector<dlspm_problem>> mine((size_t)parts);
    for (int i = 0; i < count; i++) mine[(size_t)owner[(size_t)i]].push_back(problems[i]);
    std::vector<int> status((size_t)parts, DLSPM_OK);
    std::vector<std::thread> th;
    for (int p = 0; p < parts; p++) {
        th.emplace_back([&, p]() {
            status[(size_t)p] = dlspm_spmm_batched_f32_host(mg->ctxs[(size_t)p], (int)mine[(size_t)p].size(),
                                                            mine[(size_t)p].data());
        });
    }
    for (auto &t : th) t.join();
    for (int p = 0; p < parts; p++)
        if (status[(size_t)p]) return status[(size_t)p];
    return DLSPM_OK;
}

extern "C" int dlspm_mg_spmm_rowshard_f32_host(dlspm_mg *mg, int M, int K, int N, int nnz, const float *values,
                                               const int *row_offsets, const int *column_indices,
                                               const float *B, float *C)
{
    if (!mg || M < 0 || K < 0 || N < 0 || nnz < 0 || !row_offsets) return DLSPM_ERR_INVALID_ARGUMENT;
    const int parts = (int)mg->ctxs.size();
    std::vector<int> bounds((size_t)parts + 1);
    int rc = dlspm_partition_rows_by_nnz_host(M, row_offsets, parts, bounds.data());
    if (rc) return rc;
    std::vector<int> status((size_t)parts, DLSPM_OK);
    std::vector<std::thread> th;
    for (int p = 0; p < parts; p++) {
        th.emplace_back([&, p]() {
            const int r0 = bounds[(size_t)p], r1 = bounds[(size_t)p + 1];
            const int rows = r1 - r0;
            if (rows <= 0) return;
            const int off = row_offsets[r0];
            // offsets of the block, rebased to its first nonzero; column indices are untouched
            std::vector<int> ro((size_t)rows + 1);
            for (int i = 0; i <= rows; i++) ro[(size_t)i] = row_offsets[r0 + i] - off;
            status[(size_t)p] = dlspm_spmm_csr_f32_host(mg->ctxs[(size_t)p], rows, K, N, ro[(size_t)rows],
                                                        values ? values + off : nullptr, ro.data(),
                                                        column_indices ? column_indices + off : nullptr, B,
                                                        C ? C + (size_t)r0 * (size_t)N : nullptr);
        });
    }
    for (auto &t : th) t.join();
    for (int p = 0; p < parts; p++)
        if (status[(size_t)p]) return status[(size_t)p];
    return DLSPM_OK;
}
