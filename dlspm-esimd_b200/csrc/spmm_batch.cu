// Grouped launch over many independent SpMMs for sm_100a: the persistent row-gather kernel that pulls
// tiles from a device counter, the analysis of a batch (row order by length, sortedness), prepared
// batches with the optional tiled kernel, the one-shot launch and the variant that allocates nothing.
#include <algorithm>
#include <atomic>
#include <new>
#include <vector>

#include "common.cuh"
#include "spmm_device.cuh"
#include "spmm_tile.cuh"

using namespace dlspm;

// ---- grouped launch ---------------------------------------------------------------------------
namespace {

struct BatchProblem {
    const float *values;
    const int *row_offsets;
    const int *cols;
    const float *B;
    float *C;
    int M, N;
    int row_groups;
    int vec;     // 1, 2 or 4
    int chunks;  // column chunks per slab: 1, 2 or 4
    int K;
    const int *row_order;  // rows from the longest to the shortest (nullptr: natural order)
    int nnz;
    int rows_per_tile;  // 8 (one row per warp) or 64 (each warp walks eight rows, served by the coarse launch)
};

template <int VEC, bool STRICT, bool PRE>
__device__ __forceinline__ void batched_tile(const BatchProblem &p, int slab, int row, int start,
                                             int end, int lane, int2 *stage, int2 first)
{
    float *Crow = p.C + (size_t)row * (size_t)p.N;
    const int n0 = slab * 32 * VEC * p.chunks;
    if (p.chunks == 4)
        spmm_warp_row_slab<VEC, 4, STRICT, 0, PRE>(p.values, p.cols, start, end, p.B, Crow, p.N, n0, lane, stage, first);
    else if (p.chunks == 2)
        spmm_warp_row_slab<VEC, 2, STRICT, 0, PRE>(p.values, p.cols, start, end, p.B, Crow, p.N, n0, lane, stage, first);
    else
        spmm_warp_row_slab<VEC, 1, STRICT, 0, PRE>(p.values, p.cols, start, end, p.B, Crow, p.N, n0, lane, stage, first);
}

// Warps (= rows of a fine tile) per thread block of the grouped launch.
#ifndef DLSPM_BATCH_WARPS
#define DLSPM_BATCH_WARPS 8
#endif
constexpr int kBatchWarps = DLSPM_BATCH_WARPS;
constexpr int kCoarseRows = 64 > 2 * kBatchWarps ? 64 : 2 * kBatchWarps;  // rows per tile of the coarse launch

template <bool STRICT>
__device__ __forceinline__ void batched_row(const BatchProblem &p, int slab, int slot, int lane, int2 *stage)
{
    const int row = p.row_order ? __ldg(p.row_order + slot) : slot;
    const int start = __ldg(p.row_offsets + row), end = __ldg(p.row_offsets + row + 1);
    const int2 none = make_int2(0, 0);
    if (p.vec == 4) batched_tile<4, STRICT, false>(p, slab, row, start, end, lane, stage, none);
    else if (p.vec == 2) batched_tile<2, STRICT, false>(p, slab, row, start, end, lane, stage, none);
    else batched_tile<1, STRICT, false>(p, slab, row, start, end, lane, stage, none);
}

// The rows first + warp, first + warp + 8, ... (below `last`) of a coarse tile, walked by one warp.
// Rows of such tiles hold a handful of nonzeros, so a row on its own is a chain of four dependent
// loads (row number, offsets, pairs, rows of B) in front of very little arithmetic.  Here lane i
// fetches the number and the offsets of the warp's i-th row (one chain for all eight rows), and the
// pairs of the next row are asked for before the current row is computed, so that a row waits for its
// gathers from B only.
template <bool STRICT>
__device__ __forceinline__ void batched_rows_coarse(const BatchProblem &p, int slab, int first, int last, int warp,
                                                    int lane, int2 *stage)
{
    constexpr int kRows = kCoarseRows / kBatchWarps;
    static_assert(kRows <= 32, "one lane per row of the warp");
    int my_row = -1, my_start = 0, my_end = 0;
    {
        const int slot = first + warp + kBatchWarps * lane;
        if (lane < kRows && slot < last) {
            my_row = p.row_order ? __ldg(p.row_order + slot) : slot;
            my_start = __ldg(p.row_offsets + my_row);
            my_end = __ldg(p.row_offsets + my_row + 1);
        }
    }
    int row = __shfl_sync(0xffffffffu, my_row, 0);
    int start = __shfl_sync(0xffffffffu, my_start, 0), end = __shfl_sync(0xffffffffu, my_end, 0);
    int2 pairs = make_int2(0, 0);
    if (row >= 0) pairs = spmm_first_pairs(p.values, p.cols, start, end, lane);
#pragma unroll 1
    for (int i = 0; i < kRows && row >= 0; i++) {
        const int nxt = min(i + 1, kRows - 1);
        int nrow = __shfl_sync(0xffffffffu, my_row, nxt);
        const int nstart = __shfl_sync(0xffffffffu, my_start, nxt), nend = __shfl_sync(0xffffffffu, my_end, nxt);
        if (i + 1 >= kRows) nrow = -1;
        int2 npairs = make_int2(0, 0);
        if (nrow >= 0) npairs = spmm_first_pairs(p.values, p.cols, nstart, nend, lane);
        if (p.vec == 4) batched_tile<4, STRICT, true>(p, slab, row, start, end, lane, stage, pairs);
        else if (p.vec == 2) batched_tile<2, STRICT, true>(p, slab, row, start, end, lane, stage, pairs);
        else batched_tile<1, STRICT, true>(p, slab, row, start, end, lane, stage, pairs);
        row = nrow;
        start = nstart;
        end = nend;
        pairs = npairs;
    }
}

// Persistent thread blocks pull tile numbers from a device counter.  tile_start[i] is the first
// tile of problem i (problems are stored from the most to the least work), tile_start[count] the
// total.
// COARSE: the tiles of this launch cover 64 rows (each warp walks eight of them) instead of 8; a
// build of its own, because the extra loop costs the common build registers it does not have.
template <bool STRICT, bool COARSE>
__global__ void __launch_bounds__(kBatchWarps * 32)
spmm_batched_kernel(const BatchProblem *__restrict__ problems, const long long *__restrict__ tile_start,
                    int count, unsigned long long *counter)
{
    __shared__ int2 stage[kBatchWarps][32];
    __shared__ unsigned long long s_tile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total = tile_start[count];
    for (;;) {
        if (threadIdx.x == 0) s_tile = atomicAdd(counter, 1ull);
        __syncthreads();
        const long long tile = (long long)s_tile;
        __syncthreads();
        if (tile >= total) break;
        int lo = 0, hi = count - 1;  // last problem whose first tile is <= tile
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(tile_start + mid) <= tile) lo = mid;
            else hi = mid - 1;
        }
        const BatchProblem p = problems[lo];
        const long long t = tile - __ldg(tile_start + lo);
        const int slab = (int)(t / p.row_groups);
        if constexpr (COARSE) {
            const int first = (int)(t - (long long)slab * p.row_groups) * kCoarseRows;
            const int last = min(first + kCoarseRows, p.M);
            batched_rows_coarse<STRICT>(p, slab, first, last, warp, lane, stage[warp]);
        } else {
            const int slot = (int)(t - (long long)slab * p.row_groups) * kBatchWarps + warp;
            if (slot < p.M) batched_row<STRICT>(p, slab, slot, lane, stage[warp]);
        }
    }
}

}  // namespace

namespace {

// Rows per tile of a problem.  A tile of eight rows with a handful of nonzeros each moves a few
// KiB, less than the latency chain of drawing it costs, so the grouped launch reached only 46 to
// 62 % of the HBM rate on batches of small, very sparse problems; with 64 rows per tile that
// overhead is paid an eighth as often.  Long rows keep 8 rows per tile (their tiles are large enough,
// and finer tiles balance better).
inline int rows_per_tile_for(const dlspm_problem &q, bool allow_coarse)
{
    if (!allow_coarse || q.M <= kBatchWarps) return kBatchWarps;
    return (double)q.nnz <= 32.0 * (double)q.M ? kCoarseRows : kBatchWarps;
}

// (One-chunk slabs for such problems, so that the slab of B would stay in L1 for the 64 rows of a
// tile, were measured and lost: 0.87 -> 0.50 of the HBM rate on 64 x 64 at 2 %, N = 1024.)
// Coarse tiles are used only when the batch still yields about four of them per SM; a smaller batch
// keeps the finest tiling so that it fills the device.  (Measured with batches of one shape, as a
// fraction of the HBM copy rate, fine / coarse tiles: 1894 problems of 64 x 64 at 10 %, N = 1024
// 0.46 / 0.58; 311 problems of 64 x 64 at 2 %, N = 3136 0.56 / 0.77; 476 of 64 x 64 at 2 %, N = 1024
// 0.47 / 0.66; below four tiles per SM coarse tiles lose as often as they win.)
bool coarse_tiles_pay(const dlspm_ctx *ctx, int count, const dlspm_problem *problems)
{
    long long tiles = 0;
    for (int i = 0; i < count; i++) {
        const dlspm_problem &q = problems[i];
        if (q.M <= 0 || q.N <= 0) continue;
        const int vec = dlspm_vec_width(q.N, q.B, q.C);
        const int slabs = dlspm_ceil_div(q.N, 32 * vec * spmm_slab_chunks(q.N, vec));
        tiles += (long long)dlspm_ceil_div(q.M, rows_per_tile_for(q, true)) * slabs;
    }
    return tiles >= 4LL * ctx->sm_count;
}

// Table entry of one problem (natural row order).
BatchProblem make_batch_problem(const dlspm_problem &q, bool allow_coarse)
{
    BatchProblem b;
    b.values = q.values;
    b.row_offsets = q.row_offsets;
    b.cols = q.column_indices;
    b.B = q.B;
    b.C = q.C;
    b.M = q.M;
    b.N = q.N;
    b.rows_per_tile = rows_per_tile_for(q, allow_coarse);
    b.row_groups = dlspm_ceil_div(q.M, b.rows_per_tile);
    b.vec = dlspm_vec_width(q.N, q.B, q.C);
    b.chunks = spmm_slab_chunks(q.N, b.vec);
    // Coarse tiles whose rows of B are gathered several times over (nnz / K times on average): with
    // slabs of 512 columns the slabs of B under the resident tiles (plus the C they write) exceed L2
    // and B is fetched from DRAM 1.4 to 1.6 times (ncu); slabs of 256 columns halve that footprint.
    // Measured as a fraction of the HBM copy rate, 512 / 256 / 128 columns: 64 x 64 at 10 %, N = 1024
    // 0.61 / 0.63 / 0.39; 256 x 256 at 2 %, N = 3136 0.59 / 0.63 / 0.37; 256 x 256 at 5 %, N = 1024
    // 0.35 / 0.43 / 0.24.  Without that reuse the narrower slab only doubles the row visits
    // (64 x 64 at 2 %: 0.94 -> 0.84), so those keep the wide slab.
    if (b.rows_per_tile > kBatchWarps && b.chunks > 2 && (double)q.nnz >= 3.0 * (double)q.K) b.chunks = 2;
    b.K = q.K;
    b.row_order = nullptr;
    b.nnz = q.nnz;
    return b;
}

// The one-shot grouped launches copy their tables from host memory that does not outlive the call,
// so they cannot be recorded into a CUDA graph (a replay would read a dead buffer): on a capturing
// stream they refuse before anything is enqueued.  Prepared batches (dlspm_batch_create +
// dlspm_batch_launch) keep their tables on the device and are the form to capture.
int reject_capturing_stream(dlspm_ctx *ctx, cudaStream_t st, const char *who)
{
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    cudaError_t err = cudaStreamIsCapturing(st, &status);
    if (err != cudaSuccess) {
        // the legacy default stream cannot be queried while another stream of the thread captures
        (void)cudaGetLastError();
        status = cudaStreamCaptureStatusActive;
    }
    if (status != cudaStreamCaptureStatusNone) {
        snprintf(ctx->last_error, sizeof(ctx->last_error),
                 "%s: the stream is being captured; one-shot grouped launches copy tables from host memory and cannot be "
                 "recorded, use dlspm_batch_create + dlspm_batch_launch", who);
        return DLSPM_ERR_UNSUPPORTED;
    }
    return DLSPM_OK;
}

// How a table of row-gather problems is cut between the two launches: the first `fine` entries have
// tiles of 8 rows, the `coarse` ones after them tiles of 64 rows.  The tile index holds the fine
// part (fine + 1 entries) followed by the coarse part (coarse + 1 entries).
struct GatherSplit {
    int fine, coarse;
    long long tiles_fine, tiles_coarse;
};

// Orders a table (already sorted by decreasing work) fine problems first and builds its tile index.
void finish_gather_tables(std::vector<BatchProblem> &tab, std::vector<long long> &starts, GatherSplit &split)
{
    std::stable_partition(tab.begin(), tab.end(), [](const BatchProblem &b) { return b.rows_per_tile == kBatchWarps; });
    starts.clear();
    split = GatherSplit{0, 0, 0, 0};
    for (const BatchProblem &b : tab) split.fine += b.rows_per_tile == kBatchWarps ? 1 : 0;
    split.coarse = (int)tab.size() - split.fine;
    long long run = 0;
    for (int i = 0; i < split.fine; i++) {
        const BatchProblem &b = tab[(size_t)i];
        starts.push_back(run);
        run += (long long)b.row_groups * dlspm_ceil_div(b.N, 32 * b.vec * b.chunks);
    }
    starts.push_back(run);
    split.tiles_fine = run;
    run = 0;
    for (size_t i = (size_t)split.fine; i < tab.size(); i++) {
        starts.push_back(run);
        run += (long long)tab[i].row_groups * dlspm_ceil_div(tab[i].N, 32 * tab[i].vec * tab[i].chunks);
    }
    starts.push_back(run);
    split.tiles_coarse = run;
}

// Builds the host-side tables for a batch: problems ordered by decreasing nnz*N.
int build_tables(const dlspm_ctx *ctx, int count, const dlspm_problem *problems, std::vector<BatchProblem> &tab,
                 std::vector<long long> &starts, GatherSplit &split)
{
    std::vector<int> order;
    order.reserve(count);
    for (int i = 0; i < count; i++) {
        const dlspm_problem &q = problems[i];
        int rc = check_spmm_args(q.M, q.K, q.N, q.nnz, q.values, q.row_offsets, q.column_indices,
                                 q.B, q.C);
        if (rc) return rc;
        if (q.M > 0 && q.N > 0) order.push_back(i);
    }
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) {
        return (double)problems[x].nnz * problems[x].N > (double)problems[y].nnz * problems[y].N;
    });
    tab.clear();
    const bool coarse = coarse_tiles_pay(ctx, count, problems);
    for (int i : order) tab.push_back(make_batch_problem(problems[i], coarse));
    finish_gather_tables(tab, starts, split);
    return DLSPM_OK;
}

}  // namespace

// ---- analysis of a batch: row order by length and sortedness, one thread block per problem -------
namespace {

constexpr int kLenBins = 4096;  // counting sort on min(row length, 4095)

// flags[i] bit 0: every row of problem i has strictly ascending columns.
__global__ void __launch_bounds__(256) batch_analyze_kernel(const BatchProblem *__restrict__ problems, int count,
                                                           int *__restrict__ flags)
{
    __shared__ int hist[kLenBins];
    __shared__ int warp_tot[8];
    __shared__ int s_sorted;
    for (int pi = blockIdx.x; pi < count; pi += gridDim.x) {
        const BatchProblem p = problems[pi];
        for (int b = threadIdx.x; b < kLenBins; b += blockDim.x) hist[b] = 0;
        if (threadIdx.x == 0) s_sorted = 1;
        __syncthreads();
        bool sorted = true;
        for (int r = threadIdx.x; r < p.M; r += blockDim.x) {
            const int s = p.row_offsets[r], e = p.row_offsets[r + 1];
            atomicAdd(&hist[min(max(e - s, 0), kLenBins - 1)], 1);
            for (int q = s + 1; q < e; q++) sorted &= p.cols[q - 1] < p.cols[q];
        }
        if (!sorted) s_sorted = 0;
        __syncthreads();
        // exclusive scan over the bins from the longest to the shortest: 16 bins per thread
        const int per = kLenBins / 256;
        int local[per];
        int sum = 0;
        for (int i = 0; i < per; i++) {
            local[i] = hist[kLenBins - 1 - (threadIdx.x * per + i)];
            sum += local[i];
        }
        int incl = sum;
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if ((threadIdx.x & 31) >= d) incl += o;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = incl;
        __syncthreads();
        int before = incl - sum;
        for (int w = 0; w < (int)(threadIdx.x >> 5); w++) before += warp_tot[w];
        __syncthreads();
        for (int i = 0; i < per; i++) {
            hist[kLenBins - 1 - (threadIdx.x * per + i)] = before;  // first slot of the bin
            before += local[i];
        }
        __syncthreads();
        if (p.row_order) {
            // Rows of one length keep their ascending order: the rows are placed chunk by chunk, the
            // warps of the block one after the other, each row at its rank among the rows of the same
            // length before it.  (Handing the slots out with atomics gave an order, and kernel times,
            // that changed from run to run.)
            int *order = const_cast<int *>(p.row_order);
            const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            for (int base = 0; base < p.M; base += blockDim.x) {  // same trip count for the whole block
                const int r = base + threadIdx.x;
                const bool have = r < p.M;
                const int bin = have ? min(max(p.row_offsets[r + 1] - p.row_offsets[r], 0), kLenBins - 1) : 0;
                const unsigned active = __ballot_sync(0xffffffffu, have);
                for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
                    if (warp == w && have) {
                        const unsigned peers = __match_any_sync(active, bin);
                        const int leader = __ffs(peers) - 1;
                        int slot = 0;
                        if (lane == leader) {
                            slot = hist[bin];
                            hist[bin] = slot + __popc(peers);
                        }
                        slot = __shfl_sync(peers, slot, leader);
                        order[slot + __popc(peers & ((1u << lane) - 1u))] = r;
                    }
                    __syncthreads();
                }
            }
        }
        if (threadIdx.x == 0) flags[pi] = s_sorted;
        __syncthreads();
    }
}

}  // namespace

struct dlspm_batch {
    dlspm_ctx *ctx;
    // row-gather part
    int count;
    GatherSplit split;            // fine and coarse launches over `problems`
    BatchProblem *problems;       // device
    long long *tile_start;        // device, count + 2 (fine part, coarse part)
    // tiled part (denser problems)
    int tcount;
    long long ttiles;
    TileProblem *tproblems;       // device
    long long *ttile_start;       // device, tcount + 1
    unsigned long long *counters; // device: [0] row-gather, [1] tiled
    int *row_order_pool;          // device: row orders of all row-gather problems
    int *error;                   // device: set by a kernel whose bounded wait ran out
    double stats[4];              // 2*nnz*N and algorithmic bytes: row-gather part, tiled part
};

namespace {

// d_counter: two work counters (fine launch, coarse launch).
int batch_launch_tables(dlspm_ctx *ctx, const BatchProblem *d_tab, const long long *d_starts,
                        unsigned long long *d_counter, const GatherSplit &split, cudaStream_t st)
{
    if (split.tiles_fine == 0 && split.tiles_coarse == 0) return DLSPM_OK;
    DLSPM_CUDA_TRY(ctx, cudaMemsetAsync(d_counter, 0, 2 * sizeof(unsigned long long), st));
    dim3 block(kBatchWarps * 32);
    if (split.fine > 0 && split.tiles_fine > 0) {
        dim3 grid((unsigned)std::min<long long>(split.tiles_fine, (long long)ctx->sm_count * (64 / kBatchWarps)));
        if (ctx->strict_fp32) spmm_batched_kernel<true, false><<<grid, block, 0, st>>>(d_tab, d_starts, split.fine, d_counter);
        else spmm_batched_kernel<false, false><<<grid, block, 0, st>>>(d_tab, d_starts, split.fine, d_counter);
    }
    if (split.coarse > 0 && split.tiles_coarse > 0) {
        dim3 grid((unsigned)std::min<long long>(split.tiles_coarse, (long long)ctx->sm_count * (64 / kBatchWarps)));
        const BatchProblem *tab = d_tab + split.fine;
        const long long *starts = d_starts + split.fine + 1;
        if (ctx->strict_fp32) spmm_batched_kernel<true, true><<<grid, block, 0, st>>>(tab, starts, split.coarse, d_counter + 1);
        else spmm_batched_kernel<false, true><<<grid, block, 0, st>>>(tab, starts, split.coarse, d_counter + 1);
    }
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

int tile_launch_tables(dlspm_ctx *ctx, const TileProblem *d_tab, const long long *d_starts, int *d_error, int count,
                       long long tiles, cudaStream_t st)
{
    if (count == 0 || tiles == 0) return DLSPM_OK;
    static std::atomic<bool> attr_set[64];
    const size_t smem = sizeof(TileSmem);
    if (ctx->device >= 64 || !attr_set[ctx->device].load(std::memory_order_acquire)) {
        DLSPM_CUDA_TRY(ctx, cudaFuncSetAttribute(spmm_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        DLSPM_CUDA_TRY(ctx, cudaFuncSetAttribute(spmm_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (ctx->device < 64) attr_set[ctx->device].store(true, std::memory_order_release);
    }
    // one block per SM (its shared memory fills the SM); blocks deal the tiles out among themselves
    const long long want = std::min<long long>(tiles, (long long)ctx->sm_count);
    dim3 grid((unsigned)want), block(kTileThreads);
    // kernel choice 2: present entries only, under a mask, in every chunk; otherwise absent entries
    // are multiplied as zeros except in chunks of B that hold a non-finite value
    const int force_masked = ctx->spmm_kernel == 2 ? 1 : 0;
    if (ctx->strict_fp32) spmm_tile_kernel<true><<<grid, block, smem, st>>>(d_tab, d_starts, count, force_masked, d_error);
    else spmm_tile_kernel<false><<<grid, block, smem, st>>>(d_tab, d_starts, count, force_masked, d_error);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

// Kernel choice for one problem of a prepared batch.  The tiled kernel needs 16-byte aligned rows
// of B and C (N % 4 == 0) and strictly ascending columns; it pays off once a B row loaded into shared
// memory is used by more than one of a warp's 8 rows often enough, i.e. from a density threshold.
bool prefer_tiled(const dlspm_ctx *ctx, const dlspm_problem &q, int vec, bool sorted)
{
    if (ctx->spmm_kernel == 1 || vec != 4 || !sorted || q.nnz == 0) return false;
    const double density = (double)q.nnz / ((double)q.M * (double)q.K);
    // choices 2 and 3 take every eligible problem unless a density threshold was set as well
    if (ctx->spmm_kernel >= 2)
        return !ctx->tile_min_density_set || ctx->tile_min_density_permille > 1000 ||
               density * 1000.0 >= (double)ctx->tile_min_density_permille;
    return density * 1000.0 >= (double)ctx->tile_min_density_permille && q.M >= 16 && q.N >= 64;
}

}  // namespace

// DLSPM_OPT_CHECK_INPUT for a table of SpMM problems with device pointers.
static int check_batch_input(dlspm_ctx *ctx, int count, const dlspm_problem *problems, cudaStream_t st)
{
    for (int i = 0; i < count && ctx->check_input; i++) {
        const dlspm_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.nnz < 0 || (q.nnz > 0 && !q.column_indices)) return DLSPM_ERR_INVALID_ARGUMENT;
        const int rc = dlspm_check_input(ctx, q.M, q.K, q.nnz, q.row_offsets, q.column_indices, st);
        if (rc) return rc;
    }
    return DLSPM_OK;
}

extern "C" int dlspm_batch_create(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                                  dlspm_batch **out)
{
    if (!ctx || !out || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = check_batch_input(ctx, count, problems, nullptr);
    if (rc) return rc;
    std::vector<BatchProblem> tab;
    std::vector<long long> starts;
    GatherSplit all_split;
    rc = build_tables(ctx, count, problems, tab, starts, all_split);  // validates; all problems, most work first
    if (rc) return rc;
    dlspm_batch *b = new (std::nothrow) dlspm_batch();
    if (!b) return DLSPM_ERR_NOMEM;
    memset(b, 0, sizeof(*b));
    b->ctx = ctx;
    const size_t n = tab.size();
    // pass 1: analyse every problem on the device (row order by length, sortedness)
    size_t rows_total = 0;
    for (const BatchProblem &t : tab) rows_total += (size_t)t.M;
    int *d_flags = nullptr;
    BatchProblem *d_all = nullptr;
    std::vector<int> flags(n, 0);
    cudaError_t err = cudaMalloc(&b->row_order_pool, sizeof(int) * std::max<size_t>(rows_total, 1));
    if (err == cudaSuccess) err = cudaMalloc(&b->counters, 4 * sizeof(unsigned long long));
    if (err == cudaSuccess) err = cudaMalloc(&b->error, sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(b->error, 0, sizeof(int));
    if (err == cudaSuccess && n) {
        size_t off = 0;
        for (BatchProblem &t : tab) {
            t.row_order = b->row_order_pool + off;
            off += (size_t)t.M;
        }
        err = cudaMalloc(&d_all, sizeof(BatchProblem) * n);
        if (err == cudaSuccess) err = cudaMalloc(&d_flags, sizeof(int) * n);
        if (err == cudaSuccess) err = cudaMemcpy(d_all, tab.data(), sizeof(BatchProblem) * n, cudaMemcpyHostToDevice);
        if (err == cudaSuccess) {
            const int blocks = (int)std::min<size_t>(n, (size_t)ctx->sm_count * 8);
            batch_analyze_kernel<<<blocks, 256>>>(d_all, (int)n, d_flags);
            err = cudaMemcpy(flags.data(), d_flags, sizeof(int) * n, cudaMemcpyDeviceToHost);
        }
        if (d_flags) cudaFree(d_flags);
        if (d_all) cudaFree(d_all);
    }
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "batch analysis");
        dlspm_batch_destroy(b);
        return DLSPM_ERR_CUDA;
    }
    // pass 2: split into the tiled and the row-gather tables
    std::vector<BatchProblem> gtab;
    std::vector<long long> gstarts;
    std::vector<TileProblem> ttab;
    std::vector<long long> tstarts;
    long long trun = 0;
    for (size_t i = 0; i < n; i++) {
        const BatchProblem &t = tab[i];
        dlspm_problem q;
        q.M = t.M; q.K = t.K; q.N = t.N;
        q.nnz = t.nnz;
        const double fl = 2.0 * (double)t.nnz * t.N;
        const double by = 4.0 * (t.M + 1) + 8.0 * t.nnz + 4.0 * (double)t.K * t.N + 4.0 * (double)t.M * t.N;
        const bool tiled = prefer_tiled(ctx, q, t.vec, flags[i] & 1);
        b->stats[tiled ? 2 : 0] += fl;
        b->stats[tiled ? 3 : 1] += by;
        if (tiled) {
            TileProblem tp;
            tp.values = t.values; tp.row_offsets = t.row_offsets; tp.cols = t.cols; tp.B = t.B; tp.C = t.C;
            tp.row_order = t.row_order;
            tp.M = t.M; tp.K = t.K; tp.N = t.N;
            tp.row_blocks = dlspm_ceil_div(t.M, kTileM);
            tp.col_blocks = dlspm_ceil_div(t.N, kTileN);
            tp.pad = 0;
            ttab.push_back(tp);
        } else {
            gtab.push_back(t);
        }
    }
    finish_gather_tables(gtab, gstarts, b->split);
    // A tile of the tiled kernel costs ceil(K / 32) equal steps: with the problems in order of
    // decreasing K the fixed deal of tiles to thread blocks (block b takes tiles b, b + blocks, ...)
    // hands every block the same mix, the longest tiles first.
    std::stable_sort(ttab.begin(), ttab.end(), [](const TileProblem &x, const TileProblem &y) { return x.K > y.K; });
    for (const TileProblem &tp : ttab) {
        tstarts.push_back(trun);
        trun += (long long)tp.row_blocks * tp.col_blocks;
    }
    tstarts.push_back(trun);
    b->count = (int)gtab.size();
    b->tcount = (int)ttab.size();
    b->ttiles = trun;
    err = cudaMalloc(&b->problems, sizeof(BatchProblem) * std::max<size_t>(gtab.size(), 1));
    if (err == cudaSuccess) err = cudaMalloc(&b->tile_start, sizeof(long long) * gstarts.size());
    if (err == cudaSuccess) err = cudaMalloc(&b->tproblems, sizeof(TileProblem) * std::max<size_t>(ttab.size(), 1));
    if (err == cudaSuccess) err = cudaMalloc(&b->ttile_start, sizeof(long long) * tstarts.size());
    if (err == cudaSuccess && !gtab.empty())
        err = cudaMemcpy(b->problems, gtab.data(), sizeof(BatchProblem) * gtab.size(), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMemcpy(b->tile_start, gstarts.data(), sizeof(long long) * gstarts.size(), cudaMemcpyHostToDevice);
    if (err == cudaSuccess && !ttab.empty())
        err = cudaMemcpy(b->tproblems, ttab.data(), sizeof(TileProblem) * ttab.size(), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMemcpy(b->ttile_start, tstarts.data(), sizeof(long long) * tstarts.size(), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "batch tables");
        dlspm_batch_destroy(b);
        return DLSPM_ERR_CUDA;
    }
    *out = b;
    return DLSPM_OK;
}

extern "C" int dlspm_batch_launch_part(dlspm_ctx *ctx, const dlspm_batch *batch, int part, void *stream)
{
    if (!ctx || !batch || batch->ctx != ctx || part < 0 || part > 2) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (part != 1) {
        rc = tile_launch_tables(ctx, batch->tproblems, batch->ttile_start, batch->error, batch->tcount, batch->ttiles, st);
        if (rc) return rc;
    }
    if (part != 2) {
        rc = batch_launch_tables(ctx, batch->problems, batch->tile_start, batch->counters, batch->split, st);
    }
    return rc;
}

extern "C" int dlspm_batch_launch(dlspm_ctx *ctx, const dlspm_batch *batch, void *stream)
{
    return dlspm_batch_launch_part(ctx, batch, 0, stream);
}

// Number of problems served by each kernel (for reports) and the device-side error word.
extern "C" int dlspm_batch_info(dlspm_ctx *ctx, const dlspm_batch *batch, int *gather_problems,
                                int *tiled_problems, int *device_error, double *stats4)
{
    if (!ctx || !batch || batch->ctx != ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (gather_problems) *gather_problems = batch->count;
    if (tiled_problems) *tiled_problems = batch->tcount;
    if (stats4) memcpy(stats4, batch->stats, sizeof(batch->stats));
    if (device_error) {
        DLSPM_CUDA_TRY(ctx, cudaDeviceSynchronize());
        DLSPM_CUDA_TRY(ctx, cudaMemcpy(device_error, batch->error, sizeof(int), cudaMemcpyDeviceToHost));
    }
    return DLSPM_OK;
}

extern "C" int dlspm_batch_destroy(dlspm_batch *b)
{
    if (!b) return DLSPM_OK;
    cudaSetDevice(b->ctx->device);
    if (b->problems) cudaFree(b->problems);
    if (b->tile_start) cudaFree(b->tile_start);
    if (b->tproblems) cudaFree(b->tproblems);
    if (b->ttile_start) cudaFree(b->ttile_start);
    if (b->counters) cudaFree(b->counters);
    if (b->row_order_pool) cudaFree(b->row_order_pool);
    if (b->error) cudaFree(b->error);
    (void)cudaGetLastError();
    delete b;
    return DLSPM_OK;
}

// Bytes of device memory the tables of a one-shot grouped launch of `count` problems need.
size_t dlspm_batched_table_bytes(int count)
{
    const size_t tab = (sizeof(BatchProblem) * (size_t)count + 255) & ~(size_t)255;
    const size_t st = (sizeof(long long) * ((size_t)count + 2) + 255) & ~(size_t)255;
    return tab + st + 256;
}

// One-shot grouped launch with its tables placed at `tables` (device memory of at least
// dlspm_batched_table_bytes(count) bytes, owned by the caller until the launch has finished).
int dlspm_spmm_batched_at(dlspm_ctx *ctx, int count, const dlspm_problem *problems, void *tables, cudaStream_t st,
                          void *pinned)
{
    std::vector<BatchProblem> tab;
    std::vector<long long> starts;
    GatherSplit split;
    int rc = build_tables(ctx, count, problems, tab, starts, split);
    if (rc) return rc;
    if (tab.empty()) return DLSPM_OK;
    const size_t tab_bytes = sizeof(BatchProblem) * tab.size();
    const size_t st_off = (sizeof(BatchProblem) * (size_t)count + 255) & ~(size_t)255;
    const size_t st_bytes = sizeof(long long) * starts.size();
    const size_t cnt_off = st_off + ((sizeof(long long) * ((size_t)count + 2) + 255) & ~(size_t)255);
    char *base = (char *)tables;
    const void *src_tab = tab.data(), *src_starts = starts.data();
    if (pinned) {
        memcpy(pinned, tab.data(), tab_bytes);
        memcpy((char *)pinned + st_off, starts.data(), st_bytes);
        src_tab = pinned;
        src_starts = (char *)pinned + st_off;
    }
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(base, src_tab, tab_bytes, cudaMemcpyHostToDevice, st));
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(base + st_off, src_starts, st_bytes, cudaMemcpyHostToDevice, st));
    return batch_launch_tables(ctx, (const BatchProblem *)base, (const long long *)(base + st_off),
                               (unsigned long long *)(base + cnt_off), split, st);
}

// One-shot grouped launch: tables go to the context's scratch (no allocation once it is large
// enough).  The table copies are stream-ordered cudaMemcpyAsync calls from pageable memory, which
// return once the source has been read, so the host vectors may go out of scope.
extern "C" int dlspm_spmm_batched_f32(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                                      void *stream)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (count == 0) return DLSPM_OK;
    rc = reject_capturing_stream(ctx, (cudaStream_t)stream, "dlspm_spmm_batched_f32");
    if (rc) return rc;
    rc = check_batch_input(ctx, count, problems, (cudaStream_t)stream);
    if (rc) return rc;
    rc = dlspm_scratch_reserve(ctx, dlspm_batched_table_bytes(count));
    if (rc) return rc;
    return dlspm_spmm_batched_at(ctx, count, problems, ctx->scratch, (cudaStream_t)stream);
}

// ---- grouped launch without any allocation ------------------------------------------------------
// Some callers may not allocate device memory at the point where they need a grouped SpMM: a
// plug-in running under a host framework that owns the device heap and hands out fixed buffers, a
// real-time loop that must not take the allocator's lock, or code that runs after the heap has been
// sized to the last byte.  dlspm_spmm_batched_f32 keeps its problem table, tile index and work
// counter in context scratch that grows with cudaMalloc on demand; the variant below keeps them in
// a fixed array that is part of the library image instead, so the call never allocates.  The price
// is a hard limit on the batch size, and that every GPU which loads the library carries the array
// (kStaticScratchBytes = 90 624 bytes, 88.5 KiB) until the process exits.
namespace {

constexpr int kStaticMaxProblems = 1024;
constexpr size_t kStaticTableBytes = sizeof(BatchProblem) * kStaticMaxProblems;
constexpr size_t kStaticStartsOff = (kStaticTableBytes + 255) & ~(size_t)255;
constexpr size_t kStaticStartsBytes = sizeof(long long) * (kStaticMaxProblems + 1);
constexpr size_t kStaticCounterOff = (kStaticStartsOff + kStaticStartsBytes + 255) & ~(size_t)255;
constexpr size_t kStaticScratchBytes = kStaticCounterOff + 256;
// the size quoted in the header and the documentation
static_assert(sizeof(BatchProblem) == 80 && kStaticScratchBytes == 90624, "update the documented size of the static scratch");

// Problem table, tile index and work counter of dlspm_spmm_batched_f32_static.  In host code this
// name is only a handle for cudaGetSymbolAddress, never an address a kernel can use.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Device address of g_static_scratch per device (null until looked up).  Contexts on different host
// threads may get here at the same time: the address is published with release/acquire ordering, and
// two threads that both find it missing both look it up and store the same value.
std::atomic<void *> g_static_scratch_addr[kMaxDevices];

// Looks up the device address of the static scratch on the context's device (which is current),
// once per device.
int static_scratch_address(dlspm_ctx *ctx, unsigned char **out)
{
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return DLSPM_ERR_UNSUPPORTED;
    void *p = g_static_scratch_addr[ctx->device].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (err != cudaSuccess) return dlspm_cuda_fail(ctx, err, "cudaGetSymbolAddress(g_static_scratch)");
        g_static_scratch_addr[ctx->device].store(p, std::memory_order_release);
    }
    *out = (unsigned char *)p;
    return DLSPM_OK;
}

constexpr int kStaticChunk = 32;  // table entries built on the stack and copied at a time

}  // namespace

// Host memory: none from the heap, and about 5 KiB of stack (a 2 KiB order array of 16-bit indices
// and one chunk of kStaticChunk table entries), so the call also fits the small stacks of plug-in
// and real-time threads.  The table is sent in chunks; every cudaMemcpyAsync here has a pageable
// source of a few KiB, which the runtime copies out before it returns, so the chunk buffer can be
// reused at once.  Because of these copies the call cannot be recorded into a CUDA graph: on a
// capturing stream it returns DLSPM_ERR_UNSUPPORTED before anything is enqueued.
extern "C" int dlspm_spmm_batched_f32_static(dlspm_ctx *ctx, int count, const dlspm_problem *problems,
                                             void *stream)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    if (count > kStaticMaxProblems) {
        snprintf(ctx->last_error, sizeof(ctx->last_error),
                 "dlspm_spmm_batched_f32_static: %d problems exceed the fixed limit of %d", count,
                 kStaticMaxProblems);
        return DLSPM_ERR_UNSUPPORTED;
    }
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    rc = reject_capturing_stream(ctx, st, "dlspm_spmm_batched_f32_static");
    if (rc) return rc;
    unsigned char *base = nullptr;
    rc = static_scratch_address(ctx, &base);
    if (rc) return rc;

    // Same order as the allocating entry point: decreasing nnz*N, the lower index first on ties.
    unsigned short order[kStaticMaxProblems];
    int used = 0;
    for (int i = 0; i < count; i++) {
        const dlspm_problem &q = problems[i];
        rc = check_spmm_args(q.M, q.K, q.N, q.nnz, q.values, q.row_offsets, q.column_indices, q.B, q.C);
        if (rc) return rc;
        if (q.M > 0 && q.N > 0) order[used++] = (unsigned short)i;
    }
    if (used == 0) return DLSPM_OK;
    std::sort(order, order + used, [&](unsigned short x, unsigned short y) {
        const double wx = (double)problems[x].nnz * problems[x].N, wy = (double)problems[y].nnz * problems[y].N;
        return wx != wy ? wx > wy : x < y;
    });

    BatchProblem *d_tab = (BatchProblem *)base;
    long long *d_starts = (long long *)(base + kStaticStartsOff);
    unsigned long long *d_counter = (unsigned long long *)(base + kStaticCounterOff);
    // The array keeps what the previous call left in it: the tables are overwritten here and the
    // work counter is cleared by batch_launch_tables before the kernel starts.
    BatchProblem tab[kStaticChunk];
    long long starts[kStaticChunk + 1];
    long long run = 0;
    for (int s0 = 0; s0 < used; s0 += kStaticChunk) {
        const int n = std::min(kStaticChunk, used - s0);
        for (int s = 0; s < n; s++) {
            tab[s] = make_batch_problem(problems[order[s0 + s]], false);
            starts[s] = run;
            run += (long long)tab[s].row_groups * dlspm_ceil_div(tab[s].N, 32 * tab[s].vec * tab[s].chunks);
        }
        const bool last = s0 + n == used;
        if (last) starts[n] = run;
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_tab + s0, tab, sizeof(BatchProblem) * (size_t)n, cudaMemcpyHostToDevice, st));
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_starts + s0, starts, sizeof(long long) * (size_t)(n + (last ? 1 : 0)),
                                            cudaMemcpyHostToDevice, st));
    }
    return batch_launch_tables(ctx, d_tab, d_starts, d_counter, GatherSplit{used, 0, run, 0}, st);
}
