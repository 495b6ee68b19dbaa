// Seeded synthetic inputs (host side) and the partitioners used to spread work over several GPUs.
//
// These generators stand in for the reference's rand()-based ones: Bernoulli-per-entry patterns
// (SPMM/spmm-esimd-allbenchs2.cpp:58-77), exact-count row samples (SDDMM/sddmm-esimd-v1.cpp:70-88)
// and rand()/RAND_MAX dense values (SPMM/spmm-esimd-fromfile.cpp:142-148).  Unlike those they are
// pure functions of (seed, stream, index), see rng.h.
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <queue>
#include <vector>

#include "../../include/dlspm.h"
#include "rng.h"

extern "C" uint64_t dlspm_rand_u64(uint64_t seed, uint64_t stream, uint64_t index)
{
    return dlspm_rng_at(dlspm_rng_key(seed, stream), index);
}

namespace {
const double kTwoPi = 6.283185307179586476925286766559;

// Standard normal from the uniforms at 2*index and 2*index+1.
double normal_at(uint64_t key, uint64_t index)
{
    const uint64_t h1 = dlspm_rng_at(key, 2 * index), h2 = dlspm_rng_at(key, 2 * index + 1);
    const double u1 = (double)((h1 >> 11) + 1) * (1.0 / 9007199254740992.0);  // (0, 1]
    const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);        // [0, 1)
    return sqrt(-2.0 * log(u1)) * cos(kTwoPi * u2);
}
}  // namespace

extern "C" int dlspm_gen_dense_host(float *out, size_t n, uint64_t seed, uint64_t stream,
                                    uint64_t first_index, int kind)
{
    if ((n > 0 && !out) || kind < 0 || kind > 2) return DLSPM_ERR_INVALID_ARGUMENT;
    const uint64_t key = dlspm_rng_key(seed, stream);
    for (size_t i = 0; i < n; i++) {
        const uint64_t idx = first_index + i;
        if (kind == 0) out[i] = dlspm_u24_to_pm1(dlspm_u24(dlspm_rng_at(key, idx)));
        else if (kind == 1) out[i] = dlspm_u24_to_01(dlspm_u24(dlspm_rng_at(key, idx)));
        else out[i] = (float)normal_at(key, idx);
    }
    return DLSPM_OK;
}

extern "C" int dlspm_gen_bernoulli_csr_host(int M, int K, double density, uint64_t seed, int *row_offsets,
                                            int *column_indices, size_t capacity, int *nnz)
{
    if (M < 0 || K < 0 || !row_offsets || !nnz || (capacity > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    const uint64_t key = dlspm_rng_key(seed, DLSPM_STREAM_PATTERN);
    const uint32_t thr = dlspm_density_threshold(density);
    size_t n = 0;
    row_offsets[0] = 0;
    for (int i = 0; i < M; i++) {
        for (int j = 0; j < K; j++) {
            if (dlspm_u24(dlspm_rng_at(key, (uint64_t)i * (uint64_t)K + (uint64_t)j)) < thr) {
                if (n >= capacity || n >= 0x7fffffffu) return DLSPM_ERR_NOMEM;
                column_indices[n++] = j;
            }
        }
        row_offsets[i + 1] = (int)n;
    }
    *nnz = (int)n;
    return DLSPM_OK;
}

extern "C" int dlspm_gen_band_csr_host(int M, int K, int half_band, double extra_density, uint64_t seed,
                                       int *row_offsets, int *column_indices, size_t capacity, int *nnz)
{
    if (M < 0 || K < 0 || half_band < 0 || !row_offsets || !nnz || (capacity > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    const uint64_t key = dlspm_rng_key(seed, DLSPM_STREAM_PATTERN);
    const uint32_t thr = dlspm_density_threshold(extra_density);
    size_t n = 0;
    row_offsets[0] = 0;
    for (int i = 0; i < M; i++) {
        for (int j = 0; j < K; j++) {
            const bool band = (j >= i - half_band) && (j <= i + half_band);
            if (band || dlspm_u24(dlspm_rng_at(key, (uint64_t)i * (uint64_t)K + (uint64_t)j)) < thr) {
                if (n >= capacity || n >= 0x7fffffffu) return DLSPM_ERR_NOMEM;
                column_indices[n++] = j;
            }
        }
        row_offsets[i + 1] = (int)n;
    }
    *nnz = (int)n;
    return DLSPM_OK;
}

extern "C" int dlspm_gen_rowlen_normal_host(int M, int K, double sparsity, double cov, uint64_t seed,
                                            int *row_offsets)
{
    if (M < 0 || K < 0 || !row_offsets || sparsity < 0.0 || sparsity > 1.0 || cov < 0.0)
        return DLSPM_ERR_INVALID_ARGUMENT;
    const uint64_t key = dlspm_rng_key(seed, DLSPM_STREAM_ROWLEN);
    const double mu = (double)K * (1.0 - sparsity), sigma = cov * mu;
    long long run = 0;
    row_offsets[0] = 0;
    for (int i = 0; i < M; i++) {
        long long c = llround(mu + sigma * normal_at(key, (uint64_t)i));
        c = std::max<long long>(0, std::min<long long>(K, c));
        run += c;
        if (run > 0x7fffffffLL) return DLSPM_ERR_UNSUPPORTED;
        row_offsets[i + 1] = (int)run;
    }
    return DLSPM_OK;
}

// Row i keeps the `count` columns with the smallest keys, where the key of column j is the top 32
// bits of the pattern hash of (i, j) with j itself as the tie-breaker; the kept columns are written
// in ascending order.  Every subset of that size is equally likely.
extern "C" int dlspm_gen_sample_columns_host(int M, int K, const int *row_offsets, uint64_t seed,
                                             int *column_indices)
{
    if (M < 0 || K < 0 || !row_offsets) return DLSPM_ERR_INVALID_ARGUMENT;
    const uint64_t key = dlspm_rng_key(seed, DLSPM_STREAM_PATTERN);
    std::vector<uint64_t> keys((size_t)K);
    for (int i = 0; i < M; i++) {
        const int count = row_offsets[i + 1] - row_offsets[i];
        if (count < 0 || count > K) return DLSPM_ERR_CSR;
        if (count == 0) continue;
        if (!column_indices) return DLSPM_ERR_INVALID_ARGUMENT;
        for (int j = 0; j < K; j++) {
            const uint64_t h = dlspm_rng_at(key, (uint64_t)i * (uint64_t)K + (uint64_t)j);
            keys[(size_t)j] = (h & 0xffffffff00000000ull) | (uint64_t)(uint32_t)j;
        }
        if (count < K) std::nth_element(keys.begin(), keys.begin() + (count - 1), keys.end());
        int *dst = column_indices + row_offsets[i];
        for (int c = 0; c < count; c++) dst[c] = (int)(uint32_t)(keys[(size_t)c] & 0xffffffffull);
        std::sort(dst, dst + count);
    }
    return DLSPM_OK;
}

// ---- partitioning ----------------------------------------------------------------------------

extern "C" int dlspm_partition_lpt_host(int count, const double *weights, int parts, int *owner)
{
    if (count < 0 || parts < 1 || (count > 0 && (!weights || !owner))) return DLSPM_ERR_INVALID_ARGUMENT;
    std::vector<int> order((size_t)count);
    for (int i = 0; i < count; i++) order[(size_t)i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return weights[a] > weights[b]; });
    // min-heap on (load, part): the least-loaded part, lowest index on ties
    typedef std::pair<double, int> LoadPart;
    std::priority_queue<LoadPart, std::vector<LoadPart>, std::greater<LoadPart>> heap;
    for (int p = 0; p < parts; p++) heap.push(LoadPart(0.0, p));
    for (int i : order) {
        LoadPart lp = heap.top();
        heap.pop();
        owner[i] = lp.second;
        lp.first += weights[i];
        heap.push(lp);
    }
    return DLSPM_OK;
}

extern "C" int dlspm_partition_rows_by_nnz_host(int M, const int *row_offsets, int parts, int *bounds)
{
    if (M < 0 || parts < 1 || !row_offsets || !bounds) return DLSPM_ERR_INVALID_ARGUMENT;
    const long long nnz = row_offsets[M];
    bounds[0] = 0;
    for (int p = 1; p < parts; p++) {
        // first row whose starting offset reaches p/parts of the nonzeros
        const long long target = (nnz * p + parts / 2) / parts;
        const int *it = std::lower_bound(row_offsets, row_offsets + M + 1, (int)target);
        int r = (int)(it - row_offsets);
        if (nnz == 0) r = (int)(((long long)M * p) / parts);  // no nonzeros: split rows evenly
        r = std::min(std::max(r, bounds[p - 1]), M);
        bounds[p] = r;
    }
    bounds[parts] = M;
    return DLSPM_OK;
}
