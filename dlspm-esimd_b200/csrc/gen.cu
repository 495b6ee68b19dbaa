// Device-side generators: the same bits as the host generators in host_gen.cpp, produced in HBM so
// that large benchmark inputs never cross PCIe.
#include "common.cuh"
#include "rng.h"

namespace {

constexpr int kGenThreads = 128;

__global__ void gen_dense_kernel(float *__restrict__ out, size_t n, uint64_t key, uint64_t first, int kind)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t idx = first + i;
        float v;
        if (kind == 0) v = dlspm_u24_to_pm1(dlspm_u24(dlspm_rng_at(key, idx)));
        else if (kind == 1) v = dlspm_u24_to_01(dlspm_u24(dlspm_rng_at(key, idx)));
        else {
            const uint64_t h1 = dlspm_rng_at(key, 2 * idx), h2 = dlspm_rng_at(key, 2 * idx + 1);
            const double u1 = (double)((h1 >> 11) + 1) * (1.0 / 9007199254740992.0);
            const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
            v = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2));
        }
        out[i] = v;
    }
}

// Exclusive prefix sum of one 64-bit value per thread over the block; *total gets the block sum.
__device__ __forceinline__ unsigned long long block_exclusive_scan(unsigned long long v,
                                                                   unsigned long long *warp_sums,
                                                                   unsigned long long *total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long incl = v;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const unsigned long long o = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    unsigned long long before = 0, all = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
        const unsigned long long s = warp_sums[w];
        if (w < warp) before += s;
        all += s;
    }
    __syncthreads();
    *total = all;
    return before + incl - v;
}

__device__ __forceinline__ int block_sum(int v, int *warp_sums)
{
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
    __syncthreads();
    int all = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) all += warp_sums[w];
    __syncthreads();
    return all;
}

__device__ __forceinline__ uint32_t key32_of(uint64_t key, uint64_t row_base, int j)
{
    return (uint32_t)(dlspm_rng_at(key, row_base + (uint64_t)j) >> 32);
}

// One thread block per row: keeps the `count` columns with the smallest (key32, column) pairs and
// writes them in ascending column order.  The threshold key is found by bisection on its 32 bits
// with a block-wide count per step; keys are cached in shared memory when the row fits.
constexpr int kKeyCache = 8192;

__global__ void __launch_bounds__(kGenThreads)
gen_sample_columns_kernel(int M, int K, const int *__restrict__ row_offsets, uint64_t key,
                          int *__restrict__ cols)
{
    __shared__ uint32_t cache[kKeyCache];
    __shared__ unsigned long long warp_sums64[kGenThreads / 32];
    __shared__ int warp_sums[kGenThreads / 32];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const int start = row_offsets[row];
        const int count = row_offsets[row + 1] - start;
        if (count <= 0) continue;  // uniform over the block
        const uint64_t row_base = (uint64_t)row * (uint64_t)K;
        const bool cached = K <= kKeyCache;
        if (cached) {
            for (int j = threadIdx.x; j < K; j += blockDim.x) cache[j] = key32_of(key, row_base, j);
        }
        __syncthreads();
        // smallest T with #(key32 <= T) >= count
        uint32_t lo = 0u, hi = 0xffffffffu;
        if (count < K) {
            while (lo < hi) {
                const uint32_t mid = lo + ((hi - lo) >> 1);
                int c = 0;
                for (int j = threadIdx.x; j < K; j += blockDim.x) {
                    const uint32_t k32 = cached ? cache[j] : key32_of(key, row_base, j);
                    c += (k32 <= mid) ? 1 : 0;
                }
                c = block_sum(c, warp_sums);
                if (c >= count) hi = mid;
                else lo = mid + 1;
            }
        } else {
            lo = 0xffffffffu;
        }
        const uint32_t T = lo;
        int less = 0;
        for (int j = threadIdx.x; j < K; j += blockDim.x) {
            const uint32_t k32 = cached ? cache[j] : key32_of(key, row_base, j);
            less += (k32 < T) ? 1 : 0;
        }
        less = block_sum(less, warp_sums);
        const int need_eq = count - less;  // ties at T are taken in column order
        // ordered compaction: low 32 bits count kept columns, high 32 bits count ties seen
        unsigned long long run = 0;
        for (int j0 = 0; j0 < K; j0 += blockDim.x) {
            const int j = j0 + threadIdx.x;
            uint32_t k32 = 0xffffffffu;
            bool lt = false, eq = false;
            if (j < K) {
                k32 = cached ? cache[j] : key32_of(key, row_base, j);
                lt = k32 < T;
                eq = k32 == T;
            }
            // a tie is kept while fewer than need_eq ties precede it; provisional flag first
            unsigned long long v = (lt ? 1ull : 0ull) | (eq ? (1ull << 32) : 0ull);
            unsigned long long total;
            const unsigned long long ex = block_exclusive_scan(v, warp_sums64, &total) + run;
            const int eq_before = (int)(ex >> 32);
            const int lt_before = (int)(ex & 0xffffffffull);
            if (lt) cols[start + lt_before + min(eq_before, need_eq)] = j;
            else if (eq && eq_before < need_eq) cols[start + lt_before + eq_before] = j;
            run += total;
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kGenThreads)
gen_bernoulli_count_kernel(int M, int K, int first_row, uint32_t thr, uint64_t key, int *__restrict__ counts)
{
    __shared__ int warp_sums[kGenThreads / 32];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const uint64_t row_base = (uint64_t)(first_row + row) * (uint64_t)K;
        int c = 0;
        for (int j = threadIdx.x; j < K; j += blockDim.x)
            c += dlspm_u24(dlspm_rng_at(key, row_base + (uint64_t)j)) < thr ? 1 : 0;
        c = block_sum(c, warp_sums);
        if (threadIdx.x == 0) counts[row] = c;
    }
}

__global__ void __launch_bounds__(kGenThreads)
gen_bernoulli_fill_kernel(int M, int K, int first_row, uint32_t thr, uint64_t key,
                          const int *__restrict__ row_offsets, int *__restrict__ cols)
{
    __shared__ unsigned long long warp_sums64[kGenThreads / 32];
    for (int row = blockIdx.x; row < M; row += gridDim.x) {
        const uint64_t row_base = (uint64_t)(first_row + row) * (uint64_t)K;
        const int start = row_offsets[row];
        unsigned long long run = 0;
        for (int j0 = 0; j0 < K; j0 += blockDim.x) {
            const int j = j0 + threadIdx.x;
            const bool on = j < K && dlspm_u24(dlspm_rng_at(key, row_base + (uint64_t)j)) < thr;
            unsigned long long total;
            const unsigned long long ex = block_exclusive_scan(on ? 1ull : 0ull, warp_sums64, &total) + run;
            if (on) cols[start + (int)ex] = j;
            run += total;
        }
    }
}

int grid_for_rows(const dlspm_ctx *ctx, int M) { return M < ctx->sm_count * 32 ? (M > 0 ? M : 1) : ctx->sm_count * 32; }

}  // namespace

extern "C" int dlspm_gen_dense(dlspm_ctx *ctx, float *out, size_t n, uint64_t seed, uint64_t stream,
                               uint64_t first_index, int kind, void *stream_)
{
    if (!ctx || (n > 0 && !out) || kind < 0 || kind > 2) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (n == 0) return DLSPM_OK;
    const size_t want = (n + 255) / 256;
    const int blocks = (int)(want < (size_t)ctx->sm_count * 16 ? want : (size_t)ctx->sm_count * 16);
    gen_dense_kernel<<<blocks, 256, 0, (cudaStream_t)stream_>>>(out, n, dlspm_rng_key(seed, stream), first_index, kind);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

extern "C" int dlspm_gen_sample_columns(dlspm_ctx *ctx, int M, int K, const int *row_offsets, uint64_t seed,
                                        int *column_indices, void *stream)
{
    if (!ctx || M < 0 || K < 0 || (M > 0 && !row_offsets)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (M == 0 || K == 0 || !column_indices) return DLSPM_OK;
    gen_sample_columns_kernel<<<grid_for_rows(ctx, M), kGenThreads, 0, (cudaStream_t)stream>>>(
        M, K, row_offsets, dlspm_rng_key(seed, DLSPM_STREAM_PATTERN), column_indices);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

extern "C" int dlspm_gen_bernoulli_count(dlspm_ctx *ctx, int M, int K, int first_row, double density,
                                         uint64_t seed, int *row_counts, void *stream)
{
    if (!ctx || M < 0 || K < 0 || first_row < 0 || (M > 0 && !row_counts)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (M == 0) return DLSPM_OK;
    gen_bernoulli_count_kernel<<<grid_for_rows(ctx, M), kGenThreads, 0, (cudaStream_t)stream>>>(
        M, K, first_row, dlspm_density_threshold(density), dlspm_rng_key(seed, DLSPM_STREAM_PATTERN), row_counts);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

extern "C" int dlspm_gen_bernoulli_fill(dlspm_ctx *ctx, int M, int K, int first_row, double density,
                                        uint64_t seed, const int *row_offsets, int *column_indices,
                                        void *stream)
{
    if (!ctx || M < 0 || K < 0 || first_row < 0 || (M > 0 && !row_offsets)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (M == 0 || !column_indices) return DLSPM_OK;
    gen_bernoulli_fill_kernel<<<grid_for_rows(ctx, M), kGenThreads, 0, (cudaStream_t)stream>>>(
        M, K, first_row, dlspm_density_threshold(density), dlspm_rng_key(seed, DLSPM_STREAM_PATTERN),
        row_offsets, column_indices);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}
