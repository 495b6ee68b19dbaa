// CSR SpMM for sm_100a: single-matrix launch, planned launch (rows binned by length) and the launch
// whose epilogue scatters rows to several destinations.  The grouped launch is in spmm_batch.cu.
//
// Thread-block tile: 8 warps = 8 rows of C times one slab of 32*VEC*U columns.  Tiles are
// numbered slab-major, so thread blocks that run at the same time work on the same columns of B
// and share them through L2/L1.
#include <algorithm>
#include <new>
#include <vector>

#include "common.cuh"
#include "spmm_device.cuh"

using namespace dlspm;

namespace {

struct SpmmArgs {
    const float *values;
    const int *row_offsets;
    const int *cols;
    const float *B;
    float *C;
    const int *row_order;  // nullptr = natural order
    int M, N;
    int row_groups;  // ceil(M / 8)
    int chunks;      // column chunks per slab (<= compiled U)
    int sm_count;
};

template <int VEC, int U, bool STRICT, int J>
__global__ void __launch_bounds__(kWarpsPerCta * 32) spmm_rows_kernel(const SpmmArgs a)
{
    __shared__ int2 stage[kWarpsPerCta][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long tile = blockIdx.x;
    const int slab = (int)(tile / a.row_groups);
    const int rg = (int)(tile - (long long)slab * a.row_groups);
    const int slot = rg * kWarpsPerCta + warp;
    if (slot >= a.M) return;
    const int row = a.row_order ? a.row_order[slot] : slot;
    const int start = __ldg(a.row_offsets + row), end = __ldg(a.row_offsets + row + 1);
    spmm_warp_row_slab<VEC, U, STRICT, J>(a.values, a.cols, start, end, a.B,
                                       a.C + (size_t)row * (size_t)a.N, a.N, slab * 32 * VEC * U, lane,
                                       stage[warp]);
}

// Few long rows: the S warps of a group share one row, each taking every S-th run of 32 nonzeros;
// the partial slabs are added in a fixed order through shared memory, so the result is deterministic
// (but not in CSR order: this path is not used in strict mode).  8/S rows per thread block.
template <int VEC, int U, int S>
__global__ void __launch_bounds__(kWarpsPerCta * 32) spmm_rows_split_kernel(const SpmmArgs a)
{
    __shared__ int2 stage[kWarpsPerCta][32];
    __shared__ float part[kWarpsPerCta][U][32 * VEC];
    constexpr int kRows = kWarpsPerCta / S;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = warp % S, local = warp / S;
    const long long tile = blockIdx.x;
    const int slab = (int)(tile / a.row_groups);
    const int rg = (int)(tile - (long long)slab * a.row_groups);
    const int slot = rg * kRows + local;
    const bool active = slot < a.M;
    const int row = active ? (a.row_order ? a.row_order[slot] : slot) : 0;
    const int n0 = slab * 32 * VEC * U;
    float acc[U][VEC];
    int cidx[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
        cidx[u] = n0 + (u * 32 + lane) * VEC;
#pragma unroll
        for (int v = 0; v < VEC; v++) acc[u][v] = 0.0f;
    }
    if (active) {
        const int start = __ldg(a.row_offsets + row), end = __ldg(a.row_offsets + row + 1);
        for (int base = start + 32 * split; base < end; base += 32 * S) {
            const int p = base + lane;
            int2 cv = make_int2(0, 0);
            if (p < end) cv = make_int2(__ldg(a.cols + p), __float_as_int(__ldg(a.values + p)));
            stage[warp][lane] = cv;
            __syncwarp();
            spmm_accumulate_staged<VEC, U, false, kLoneBatch<U>>(stage[warp], min(32, end - base), a.B, a.N, cidx, acc);
            __syncwarp();
        }
    }
    if (split != 0) {
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int v = 0; v < VEC; v++) part[warp][u][lane * VEC + v] = acc[u][v];
    }
    __syncthreads();
    if (split == 0 && active) {
#pragma unroll
        for (int sidx = 1; sidx < S; sidx++)
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int v = 0; v < VEC; v++) acc[u][v] += part[warp + sidx][u][lane * VEC + v];
        float *crow = a.C + (size_t)row * (size_t)a.N;
#pragma unroll
        for (int u = 0; u < U; u++)
            if (cidx[u] < a.N) store_vec<VEC>(crow + cidx[u], acc[u]);
    }
}

template <int VEC, int U, int S>
void launch_rows_split(SpmmArgs a, int slabs, cudaStream_t st)
{
    a.row_groups = dlspm_ceil_div(a.M, kWarpsPerCta / S);
    spmm_rows_split_kernel<VEC, U, S><<<(unsigned)((long long)a.row_groups * slabs), kWarpsPerCta * 32, 0, st>>>(a);
}

// Narrow dense operand (N <= 64 floats, 16-byte aligned rows): a full warp per row would leave most
// lanes idle, so a warp is cut into 32/LANES groups of LANES lanes and every group owns a row.  Lane t
// of a group holds columns 4t..4t+3; the group's (column, value) pairs are fetched LANES at a time
// (one per lane) and handed round with width-LANES shuffles; every B row segment is one 16-byte load
// per lane, LANES*16 contiguous bytes per group.  Each output element still accumulates in CSR order.
template <int LANES, bool STRICT>
__global__ void __launch_bounds__(kWarpsPerCta * 32) spmm_subwarp_kernel(const SpmmArgs a)
{
    constexpr int kRowsPerWarp = 32 / LANES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane / LANES, t = lane % LANES;
    const int slot = (blockIdx.x * kWarpsPerCta + warp) * kRowsPerWarp + g;
    const bool has_row = slot < a.M;
    const int row = has_row ? (a.row_order ? a.row_order[slot] : slot) : 0;
    int start = 0, len = 0;
    if (has_row) {
        start = __ldg(a.row_offsets + row);
        len = __ldg(a.row_offsets + row + 1) - start;
    }
    const bool active = has_row && t * 4 < a.N;
    const int longest = __reduce_max_sync(0xffffffffu, len);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float *bcol = a.B + t * 4;
    for (int base = 0; base < longest; base += LANES) {
        int c = 0;
        float v = 0.f;
        if (base + t < len) {
            c = __ldg(a.cols + start + base + t);
            v = __ldg(a.values + start + base + t);
        }
#pragma unroll
        for (int j = 0; j < LANES; j++) {
            const int cj = __shfl_sync(0xffffffffu, c, j, LANES);
            const float vj = __shfl_sync(0xffffffffu, v, j, LANES);
            if (active && base + j < len) {
                const float4 b = __ldg(reinterpret_cast<const float4 *>(bcol + (size_t)cj * (size_t)a.N));
                acc[0] = mad<STRICT>(vj, b.x, acc[0]);
                acc[1] = mad<STRICT>(vj, b.y, acc[1]);
                acc[2] = mad<STRICT>(vj, b.z, acc[2]);
                acc[3] = mad<STRICT>(vj, b.w, acc[3]);
            }
        }
    }
    if (active)
        *reinterpret_cast<float4 *>(a.C + (size_t)row * (size_t)a.N + t * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// The same narrow operand with too few rows for a row per lane group: the 32/LANES groups of a warp
// share ONE row.  The warp fetches 32 (column, value) pairs per step and deals them to the groups in
// turn (pair i to group i mod 32/LANES), every group gathers the B rows of its pairs with all its
// lanes busy, and the groups' partial rows are added with shuffles at the end (fixed order, but not
// CSR order: not used in strict mode).  A full warp per row with one 128-column chunk would leave
// 24 of 32 lanes idle at N = 32.
template <int LANES>
__global__ void __launch_bounds__(kWarpsPerCta * 32) spmm_subwarp_shared_kernel(const SpmmArgs a)
{
    constexpr int kGroups = 32 / LANES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane / LANES, t = lane % LANES;
    const int slot = blockIdx.x * kWarpsPerCta + warp;
    if (slot >= a.M) return;
    const int row = a.row_order ? a.row_order[slot] : slot;
    const int start = __ldg(a.row_offsets + row), len = __ldg(a.row_offsets + row + 1) - start;
    const bool active = t * 4 < a.N;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const float *bcol = a.B + t * 4;
    for (int base = 0; base < len; base += 32) {
        int c = 0;
        float v = 0.f;
        if (base + lane < len) {
            c = __ldg(a.cols + start + base + lane);
            v = __ldg(a.values + start + base + lane);
        }
#pragma unroll
        for (int j = 0; j < LANES; j++) {
            if (base + j * kGroups >= len) break;  // uniform over the warp
            const int src = j * kGroups + g;       // this group's j-th pair of the step
            const int cj = __shfl_sync(0xffffffffu, c, src);
            const float vj = __shfl_sync(0xffffffffu, v, src);
            if (active && base + src < len) {
                const float4 b = __ldg(reinterpret_cast<const float4 *>(bcol + (size_t)cj * (size_t)a.N));
                acc[0] = fmaf(vj, b.x, acc[0]);
                acc[1] = fmaf(vj, b.y, acc[1]);
                acc[2] = fmaf(vj, b.z, acc[2]);
                acc[3] = fmaf(vj, b.w, acc[3]);
            }
        }
    }
#pragma unroll
    for (int s = LANES; s < 32; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], s);
    }
    if (active && g == 0)
        *reinterpret_cast<float4 *>(a.C + (size_t)row * (size_t)a.N + t * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

template <int LANES>
void launch_subwarp_shared(const SpmmArgs &a, cudaStream_t st)
{
    spmm_subwarp_shared_kernel<LANES><<<(unsigned)dlspm_ceil_div(a.M, kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(a);
}

template <int LANES>
void launch_subwarp(const SpmmArgs &a, bool strict, cudaStream_t st)
{
    const int rows_per_block = kWarpsPerCta * (32 / LANES);
    const unsigned blocks = (unsigned)dlspm_ceil_div(a.M, rows_per_block);
    if (strict) spmm_subwarp_kernel<LANES, true><<<blocks, kWarpsPerCta * 32, 0, st>>>(a);
    else spmm_subwarp_kernel<LANES, false><<<blocks, kWarpsPerCta * 32, 0, st>>>(a);
}

template <int VEC, int U>
void launch_rows(const SpmmArgs &a, int slabs, bool strict, cudaStream_t st)
{
    const long long tiles = (long long)a.row_groups * slabs;
    dim3 grid((unsigned)tiles), block(kWarpsPerCta * 32);
    // The narrow slabs exist in two builds: with the batched loads (74 to 76 registers, three
    // resident blocks) for launches of a few waves, where the latency chain of a warp counts, and
    // with the plain loop (32 and 44 registers) for long launches, where occupancy hides it.
    // Measured: one-chunk slabs, 32768 x 8192 (9 waves) 0.71 -> 0.61 ms with the plain loop but
    // 8192 x 8192 (2.3 waves) 0.19 -> 0.20 ms; two-chunk slabs, 32768 x 2048 413 -> 338 us.
    const int waves = U == 1 ? 6 : 2;
    const bool lone = kLoneBatch<U> > 0 && tiles <= (long long)waves * 3 * a.sm_count;
    if (lone) {
        if (strict) spmm_rows_kernel<VEC, U, true, kLoneBatch<U>><<<grid, block, 0, st>>>(a);
        else spmm_rows_kernel<VEC, U, false, kLoneBatch<U>><<<grid, block, 0, st>>>(a);
    } else {
        if (strict) spmm_rows_kernel<VEC, U, true, 0><<<grid, block, 0, st>>>(a);
        else spmm_rows_kernel<VEC, U, false, 0><<<grid, block, 0, st>>>(a);
    }
}

template <int VEC, int U>
void launch_rows_maybe_split(const SpmmArgs &a, int slabs, int split, bool strict, cudaStream_t st)
{
    if (split == 8) launch_rows_split<VEC, U, 8>(a, slabs, st);
    else if (split == 4) launch_rows_split<VEC, U, 4>(a, slabs, st);
    else if (split == 2) launch_rows_split<VEC, U, 2>(a, slabs, st);
    else launch_rows<VEC, U>(a, slabs, strict, st);
}

// `split`: warps per row (1, 2, 4 or 8), see spmm_row_split.
template <int VEC>
void launch_rows_vec(SpmmArgs a, int split, bool strict, cudaStream_t st)
{
    a.chunks = spmm_slab_chunks(a.N, VEC);
    const int slabs = dlspm_ceil_div(a.N, 32 * VEC * a.chunks);
    const int U = a.chunks;
    if (U == 4) launch_rows_maybe_split<VEC, 4>(a, slabs, split, strict, st);
    else if (U == 2) launch_rows_maybe_split<VEC, 2>(a, slabs, split, strict, st);
    else launch_rows_maybe_split<VEC, 1>(a, slabs, split, strict, st);
}

// Warps per row for a lone matrix: with few rows one warp per (row, slab) leaves most of the device
// idle and every warp walks its whole row as one latency chain, so rows are shared by 2, 4 or 8
// warps until about 32 warps per SM exist or a warp would get fewer than 8 nonzeros.  Measured with
// the bound at 64 / 16 / 8 nonzeros per warp (lone launches, warm L2): 512 x 512 at 10 %, N = 128:
// 17.3 / 13.1 / 7.6 us; 1024 x 1024 at 10 %, N = 128: 35.6 / - / 8.5 us; 512 x 2048 at 10 %,
// N = 256: 47.8 / 12.8 / 12.8 us; nothing measured got slower by more than 10 %.
int spmm_row_split(const dlspm_ctx *ctx, int M, int N, int nnz, int vec, bool strict)
{
    if (strict || M <= 0) return 1;
    const int chunks = spmm_slab_chunks(N, vec);
    const long long warps = (long long)M * dlspm_ceil_div(N, 32 * vec * chunks);
    const long long want = (long long)ctx->sm_count * 32;
    const double avg = (double)nnz / (double)M;
    int s = 1;
    while (s < 8 && warps * s < want && avg / (2 * s) >= 8.0) s *= 2;
    return s;
}


// max_row_len: longest row if known (from a plan), else 0.
int spmm_launch(dlspm_ctx *ctx, int M, int N, int nnz, const float *values, const int *row_offsets,
                const int *cols, const float *B, float *C, const int *row_order, int max_row_len, cudaStream_t st)
{
    if (M == 0 || N == 0) return DLSPM_OK;
    SpmmArgs a{values, row_offsets, cols, B, C, row_order, M, N, dlspm_ceil_div(M, kWarpsPerCta), 1, ctx->sm_count};
    const int vec = dlspm_vec_width(N, B, C);
    const bool strict = ctx->strict_fp32 != 0;
    int split = spmm_row_split(ctx, M, N, nnz, vec, strict);
    // Long rows of uneven length (known only with a plan): eight warps per row make every thread
    // block finish its row together, which the binning by powers of two does not.  Measured on
    // planned launches with a 40 % row-length spread and narrow slabs: mean length 1229: 178 -> 138 us,
    // 2458: 614 -> 553 us, 819: 387 -> 357 us; at mean length 614 it went either way (2048 rows
    // 48.7 -> 39.8 us, 8192 rows 131 -> 146 us), at 205 it lost 10 to 45 %, and with uniform rows it
    // loses at every length, hence both conditions.
    const double mean_len = (double)nnz / (double)M;
    if (!strict && max_row_len > 0 && mean_len >= 800.0 && (double)max_row_len >= 1.3 * mean_len &&
        spmm_slab_chunks(N, vec) <= 2)
        split = 8;
    // narrow N: several rows per warp, but never so many that the matrix yields too few warps
    int lanes = 32;
    if (vec == 4 && N <= 64 && !strict) {
        // Too few rows for a row per lane group (fewer than 16 warps per SM that way), enough for a
        // row per warp: the groups share the row.  Measured at N = 32 and 30 % nonzeros, GFLOP/s:
        // 4096 x 1024 2019 -> 3687, 8192 x 2048 3856 -> 6312, 4096 x 4096 2668 -> 4971, 8192 x 8192
        // 3610 -> 5651; with fewer rows than 16 per SM the launch gets too few warps either way and
        // the warps-per-row split below does better (1024 x 1024 1016 -> 844: left alone).
        const int narrow = N <= 16 ? 4 : N <= 32 ? 8 : 16;
        if ((long long)M * narrow / 32 < (long long)ctx->sm_count * 16 && (long long)M >= (long long)ctx->sm_count * 16 &&
            mean_len >= 16.0) {
            if (narrow == 4) launch_subwarp_shared<4>(a, st);
            else if (narrow == 8) launch_subwarp_shared<8>(a, st);
            else launch_subwarp_shared<16>(a, st);
            DLSPM_CUDA_TRY(ctx, cudaGetLastError());
            return DLSPM_OK;
        }
    }
    if (vec == 4 && N <= 64 && split == 1) {
        lanes = N <= 16 ? 4 : N <= 32 ? 8 : 16;
        while (lanes < 32 && (long long)M * lanes / 32 < (long long)ctx->sm_count * 16) lanes *= 2;
    }
    if (lanes == 4) launch_subwarp<4>(a, strict, st);
    else if (lanes == 8) launch_subwarp<8>(a, strict, st);
    else if (lanes == 16) launch_subwarp<16>(a, strict, st);
    else if (vec == 4) launch_rows_vec<4>(a, split, strict, st);
    else if (vec == 2) launch_rows_vec<2>(a, split, strict, st);
    else launch_rows_vec<1>(a, split, strict, st);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

}  // namespace

extern "C" int dlspm_spmm_csr_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                                  const int *row_offsets, const int *column_indices, const float *B,
                                  float *C, void *stream)
{
    if (!ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = check_spmm_args(M, K, N, nnz, values, row_offsets, column_indices, B, C);
    if (rc) return rc;
    rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = dlspm_check_input(ctx, M, K, nnz, row_offsets, column_indices, (cudaStream_t)stream);
    if (rc) return rc;
    return spmm_launch(ctx, M, N, nnz, values, row_offsets, column_indices, B, C, nullptr, 0,
                       (cudaStream_t)stream);
}

extern "C" int dlspm_spmm_csr_f32_planned(dlspm_ctx *ctx, const dlspm_plan *plan, int N,
                                          const float *values, const int *row_offsets,
                                          const int *column_indices, const float *B, float *C,
                                          void *stream)
{
    if (!ctx || !plan || plan->ctx != ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = check_spmm_args(plan->M, plan->K, N, plan->nnz, values, row_offsets, column_indices, B, C);
    if (rc) return rc;
    rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = dlspm_check_input(ctx, plan->M, plan->K, plan->nnz, row_offsets, column_indices, (cudaStream_t)stream);
    if (rc) return rc;
    return spmm_launch(ctx, plan->M, N, plan->nnz, values, row_offsets, column_indices, B, C, plan->row_order,
                       plan->max_row_len, (cudaStream_t)stream);
}

// ---- SpMM whose result rows go to several destinations (fused compute + gather) -----------------
// A row-sharded SpMM needs its row block in the full C of every GPU afterwards.  Instead of running
// the product and then a collective, the epilogue stores each finished row segment into every
// destination buffer: the local C and the peers' C, reached through peer mappings (NVLink).  The
// remote stores are fire-and-forget and overlap with the gathers of the rows still being computed.
namespace {

constexpr int kMaxDst = 8;

struct ScatterArgs {
    SpmmArgs a;
    float *dst[kMaxDst];  // full-size C buffers (local and peers)
    long long first_row;  // global row of local row 0
    int ndst;
};

// (Three resident blocks as the bound: with the default the compiler stops at 58 registers and keeps
// fewer gathers in flight than the plain kernel's 66-register build; 8192 rows of a 65536-column
// pattern at 1 %, N = 512, one destination: 657 -> 574 us, the plain kernel 563 us.)
template <int VEC, int U, bool STRICT>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 3) spmm_rows_scatter_kernel(const __grid_constant__ ScatterArgs s)
{
    // (__grid_constant__: the destination list is indexed with a run-time index below; without it
    // every thread would first copy the argument block to local memory)
    __shared__ int2 stage[kWarpsPerCta][32];
    const SpmmArgs &a = s.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long tile = blockIdx.x;
    const int slab = (int)(tile / a.row_groups);
    const int rg = (int)(tile - (long long)slab * a.row_groups);
    const int slot = rg * kWarpsPerCta + warp;
    if (slot >= a.M) return;
    const int row = a.row_order ? a.row_order[slot] : slot;
    const int start = __ldg(a.row_offsets + row), end = __ldg(a.row_offsets + row + 1);
    const int n0 = slab * 32 * VEC * U;
    // the sums of spmm_warp_row_slab (same code), then the slab is stored to every destination
    float acc[U][VEC];
    int cidx[U];
    spmm_warp_row_sums<VEC, U, STRICT, 0, false>(a.values, a.cols, start, end, a.B, a.N, n0, lane, stage[warp],
                                                 make_int2(0, 0), cidx, acc);
    const size_t off = (size_t)(s.first_row + row) * (size_t)a.N;
    // Every warp starts its round of destinations at another one, so that the warps of a GPU (and,
    // when every GPU lists its destinations starting with itself in ring order, the GPUs among
    // themselves) do not all store to the same peer at the same moment.
    int dd = (int)((tile + warp) % s.ndst);
    for (int d = 0; d < s.ndst; d++) {
        float *crow = s.dst[dd] + off;
        if (++dd == s.ndst) dd = 0;
#pragma unroll
        for (int u = 0; u < U; u++)
            if (cidx[u] < a.N) store_vec<VEC>(crow + cidx[u], acc[u]);
    }
}

template <int VEC, int U>
void launch_scatter(const ScatterArgs &s, bool strict, cudaStream_t st)
{
    const int slabs = dlspm_ceil_div(s.a.N, 32 * VEC * U);
    const unsigned blocks = (unsigned)((long long)s.a.row_groups * slabs);
    if (strict) spmm_rows_scatter_kernel<VEC, U, true><<<blocks, kWarpsPerCta * 32, 0, st>>>(s);
    else spmm_rows_scatter_kernel<VEC, U, false><<<blocks, kWarpsPerCta * 32, 0, st>>>(s);
}

}  // namespace

extern "C" int dlspm_spmm_csr_f32_scatter(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                                          const int *row_offsets, const int *column_indices, const float *B,
                                          int ndst, float *const *C_dsts, long long first_row, void *stream)
{
    if (!ctx || ndst < 1 || ndst > kMaxDst || !C_dsts || first_row < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = check_spmm_args(M, K, N, nnz, values, row_offsets, column_indices, B, C_dsts[0]);
    if (rc) return rc;
    rc = dlspm_use(ctx);
    if (rc) return rc;
    if (M == 0 || N == 0) return DLSPM_OK;
    ScatterArgs s;
    s.a = SpmmArgs{values, row_offsets, column_indices, B, nullptr, nullptr, M, N, dlspm_ceil_div(M, kWarpsPerCta), 1, ctx->sm_count};
    s.first_row = first_row;
    s.ndst = ndst;
    const void *align_probe = B;
    for (int d = 0; d < kMaxDst; d++) {
        s.dst[d] = d < ndst ? C_dsts[d] : nullptr;
        if (d < ndst) {
            if (!C_dsts[d]) return DLSPM_ERR_INVALID_ARGUMENT;
            if (((uintptr_t)C_dsts[d] % 16) != 0) align_probe = C_dsts[d];  // forces the narrow path
        }
    }
    const int vec = dlspm_vec_width(N, B, align_probe);
    const int U = spmm_slab_chunks(N, vec);
    cudaStream_t st = (cudaStream_t)stream;
    const bool strict = ctx->strict_fp32 != 0;
    if (vec == 4) {
        if (U == 4) launch_scatter<4, 4>(s, strict, st);
        else if (U == 2) launch_scatter<4, 2>(s, strict, st);
        else launch_scatter<4, 1>(s, strict, st);
    } else if (vec == 2) {
        if (U == 4) launch_scatter<2, 4>(s, strict, st);
        else if (U == 2) launch_scatter<2, 2>(s, strict, st);
        else launch_scatter<2, 1>(s, strict, st);
    } else {
        if (U == 4) launch_scatter<1, 4>(s, strict, st);
        else if (U == 2) launch_scatter<1, 2>(s, strict, st);
        else launch_scatter<1, 1>(s, strict, st);
    }
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

// ---- plan: rows binned by length --------------------------------------------------------------
namespace {

constexpr int kBins = 33;  // bin b holds rows with 2^(b-1) <= length < 2^b; bin 0 = empty rows

__device__ __forceinline__ int length_bin(int len) { return len <= 0 ? 0 : 32 - __clz(len); }

// Rows are placed in a fixed order: bins from the longest rows to the shortest, inside a bin by
// ascending row number.  Every thread block owns a contiguous range of `span` rows; it counts its
// rows per bin (plan_hist_kernel), a scan over (bin, block) gives the first slot of every block in
// every bin (plan_scan_kernel), and the block then places its rows chunk by chunk, its warps one
// after the other, each row at its rank among the rows of the same bin before it
// (plan_scatter_kernel).  No slot is handed out by a global atomic, so the order, and with it the
// timing of the kernels that walk it, is the same in every run.
//
// info[0..32] = rows per bin, info[33] = 1 while every row is sorted, info[34] = longest row;
// block_hist[block * kBins + bin] = rows of the block in the bin.
__global__ void __launch_bounds__(256) plan_hist_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                                                        int M, int span, int *info, int *__restrict__ block_hist)
{
    __shared__ int hist[kBins];
    __shared__ int s_sorted, s_max;
    if (threadIdx.x < kBins) hist[threadIdx.x] = 0;
    if (threadIdx.x == 0) { s_sorted = 1; s_max = 0; }
    __syncthreads();
    const int first = blockIdx.x * span, last = min(first + span, M);
    for (int r = first + threadIdx.x; r < last; r += blockDim.x) {
        const int s = row_offsets[r], e = row_offsets[r + 1];
        atomicAdd(&hist[length_bin(e - s)], 1);
        atomicMax(&s_max, e - s);
        bool sorted = true;
        for (int p = s + 1; p < e; p++) sorted &= cols[p - 1] < cols[p];
        if (!sorted) s_sorted = 0;
    }
    __syncthreads();
    if (threadIdx.x < kBins) block_hist[blockIdx.x * kBins + threadIdx.x] = hist[threadIdx.x];
    if (threadIdx.x == 0) {
        if (!s_sorted) atomicAnd(&info[kBins], 0);
        atomicMax(&info[kBins + 1], s_max);
    }
}

// cursor[block * kBins + bin] = first slot of the block's rows of the bin, bins laid out from the
// longest to the shortest and blocks in order inside a bin; info[bin] = rows of the bin.  One thread
// block of 64 threads: thread t sums bin t over the blocks, then the bins are scanned.
__global__ void plan_scan_kernel(const int *__restrict__ block_hist, int blocks, int *info, int *__restrict__ cursor)
{
    __shared__ int total[kBins], first[kBins];
    const int bin = threadIdx.x;
    if (bin < kBins) {
        int run = 0;
        for (int b = 0; b < blocks; b++) run += block_hist[b * kBins + bin];
        total[bin] = run;
        info[bin] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int b = kBins - 1; b >= 0; b--) {
            first[b] = run;
            run += total[b];
        }
    }
    __syncthreads();
    if (bin < kBins) {
        int run = first[bin];
        for (int b = 0; b < blocks; b++) {
            cursor[b * kBins + bin] = run;
            run += block_hist[b * kBins + bin];
        }
    }
}

__global__ void __launch_bounds__(256) plan_scatter_kernel(const int *__restrict__ row_offsets, int M, int span,
                                                           const int *__restrict__ cursor, int *__restrict__ row_order)
{
    __shared__ int next[kBins];  // next free slot of every bin for this block
    if (threadIdx.x < kBins) next[threadIdx.x] = cursor[blockIdx.x * kBins + threadIdx.x];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = blockIdx.x * span, last = min(first + span, M);
    for (int base = first; base < last; base += blockDim.x) {  // same trip count for the whole block
        const int r = base + threadIdx.x;
        const bool have = r < last;
        const int bin = have ? length_bin(row_offsets[r + 1] - row_offsets[r]) : 0;
        const unsigned active = __ballot_sync(0xffffffffu, have);
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
            if (warp == w && have) {
                const unsigned peers = __match_any_sync(active, bin);  // lanes of this warp with a row of the same bin
                const int leader = __ffs(peers) - 1;
                int slot = 0;
                if (lane == leader) {
                    slot = next[bin];
                    next[bin] = slot + __popc(peers);
                }
                slot = __shfl_sync(peers, slot, leader);
                row_order[slot + __popc(peers & ((1u << lane) - 1u))] = r;
            }
            __syncthreads();
        }
    }
}

}  // namespace

extern "C" int dlspm_plan_create(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets,
                                 const int *column_indices, void *stream, dlspm_plan **out)
{
    if (!ctx || !out || M < 0 || K < 0 || nnz < 0 || (M > 0 && !row_offsets) ||
        (nnz > 0 && !column_indices))
        return DLSPM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    dlspm_plan *plan = new (std::nothrow) dlspm_plan();
    if (!plan) return DLSPM_ERR_NOMEM;
    plan->ctx = ctx;
    plan->M = M;
    plan->K = K;
    plan->nnz = nnz;
    plan->row_order = nullptr;
    plan->sorted_rows = 1;
    plan->max_row_len = 0;
    if (M == 0) {
        *out = plan;
        return DLSPM_OK;
    }
    // every thread block owns `span` consecutive rows (a multiple of its 256 threads)
    const int blocks_max = std::max(1, std::min(dlspm_ceil_div(M, 256), ctx->sm_count * 8));
    const int span = dlspm_ceil_div(dlspm_ceil_div(M, blocks_max), 256) * 256;
    const int blocks = dlspm_ceil_div(M, span);
    int *work = nullptr;  // [0..34] info, from 40: rows per (block, bin), then first slots per (block, bin)
    const size_t work_ints = 40 + 2 * (size_t)blocks * kBins;
    cudaError_t err = cudaMalloc(&plan->row_order, sizeof(int) * (size_t)M);
    if (err == cudaSuccess) err = cudaMalloc(&work, sizeof(int) * work_ints);
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "cudaMalloc(plan)");
        if (plan->row_order) cudaFree(plan->row_order);
        delete plan;
        return DLSPM_ERR_NOMEM;
    }
    int init[40];
    memset(init, 0, sizeof(init));
    init[kBins] = 1;
    int info[kBins + 2];
    int *block_hist = work + 40, *cursor = work + 40 + (size_t)blocks * kBins;
    err = cudaMemcpyAsync(work, init, sizeof(init), cudaMemcpyHostToDevice, st);
    if (err == cudaSuccess) {
        plan_hist_kernel<<<blocks, 256, 0, st>>>(row_offsets, column_indices, M, span, work, block_hist);
        plan_scan_kernel<<<1, 64, 0, st>>>(block_hist, blocks, work, cursor);
        plan_scatter_kernel<<<blocks, 256, 0, st>>>(row_offsets, M, span, cursor, plan->row_order);
        err = cudaMemcpyAsync(info, work, sizeof(info), cudaMemcpyDeviceToHost, st);
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err == cudaSuccess) err = cudaGetLastError();
    cudaFree(work);
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "plan kernels");
        cudaFree(plan->row_order);
        delete plan;
        return DLSPM_ERR_CUDA;
    }
    plan->sorted_rows = info[kBins];
    plan->max_row_len = info[kBins + 1];
    *out = plan;
    return DLSPM_OK;
}

extern "C" int dlspm_plan_row_order(const dlspm_plan *plan, int *order, void *stream)
{
    if (!plan || (plan->M > 0 && !order)) return DLSPM_ERR_INVALID_ARGUMENT;
    if (plan->M == 0) return DLSPM_OK;
    dlspm_ctx *ctx = plan->ctx;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(order, plan->row_order, sizeof(int) * (size_t)plan->M, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

extern "C" int dlspm_plan_destroy(dlspm_plan *plan)
{
    if (!plan) return DLSPM_OK;
    if (plan->row_order) {
        cudaSetDevice(plan->ctx->device);
        cudaFree(plan->row_order);
    }
    delete plan;
    return DLSPM_OK;
}
