// Grouped launches over many independent SDDMMs and fused SDDMM -> SpMM chains for sm_100a.
//
// A layer-sized pattern (a few hundred to a few thousand rows) is launch-bound on its own: the lone
// launches of the reference's batch scripts (SDDMM/batch-run-sddmm_fromfile:31-47,
// FUSED/batch-run-fused:22-34) spend more time between kernels than in them.  Here all problems of a
// batch that share a register layout (group width G and chunks per lane R, which follow from the
// inner dimension, see sddmm_device.cuh) run in ONE persistent launch: warps pull rows from a device
// counter (thread blocks pull tiles of eight where the fused chain shares rows between warps), one
// warp per row, and every row is processed exactly as in the
// single-matrix kernels (same passes, same butterfly, same order of additions), so results have the
// same bits (one exception: rows of exactly 32 floats in single-matrix launches of 8192 rows or more use
// 256-bit loads there and can differ in the last place).  A batch with one inner dimension is one
// launch; a mixed batch is at most twelve.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "fused_device.cuh"
#include "sddmm_device.cuh"

using namespace dlspm;

namespace {

constexpr int kWarps = 8;
constexpr int kClasses = 12;  // the six (G, R) layouts of sddmm_layout (0..5), then SDDMM rows beyond 1024 floats in segments
                              // of 1024 / 512 floats, one warp per row (6, 7) or rows shared between warps (8, 9), then
                              // rows of up to 16 / 32 floats in groups of four lanes (10, 11)
constexpr int kOpSddmm = 0, kOpFused = 1, kOpSddmmLong = 2, kOpSddmmLongShared = 3;

struct RowProblem {
    const int *row_offsets;
    const int *cols;
    const float *a;     // lhs (SDDMM) or C (fused): M x N
    const float *b;     // rhs or B: K x N
    const float *d;     // fused only: D, K x N
    const float *mask;  // SDDMM only: factors per stored entry or nullptr
    float *out;         // out_values (SDDMM) or E (fused)
    int M;
    int chunks;         // N / 4
    int shift;          // SDDMM: 1 << shift warps share a row (its passes in turn; for rows beyond 1024
                        // floats the nonzeros inside every pass), see choose_sharing
};

// `sub` of 1 << p.shift warps that share the row: this warp takes the passes sub, sub + (1 << shift), ...
template <int G, int R>
__device__ __forceinline__ void sddmm_one_row(const RowProblem &p, int row, int sub, int lane)
{
    const int g = lane / G, t = lane % G;
    const int stride = 32 << p.shift;
    const int start = __ldg(p.row_offsets + row) + 32 * sub, end = __ldg(p.row_offsets + row + 1);
    if (start >= end) return;
    const float4 *lhs4 = reinterpret_cast<const float4 *>(p.a) + (size_t)row * (size_t)p.chunks;
    const float4 *rhs4 = reinterpret_cast<const float4 *>(p.b);
    float4 a[R];
    load_row_chunks<G, R>(lhs4, p.chunks, t, a);
    int col_next = start + lane < end ? __ldg(p.cols + start + lane) : -1;
    for (int base = start; base < end; base += stride) {
        const int q = base + lane;
        const int col = col_next;
        col_next = q + stride < end ? __ldg(p.cols + q + stride) : -1;
        const float r = sddmm_pass_dealt<G, R>(a, rhs4, p.chunks, col, g, t);
        const int o = base + sddmm_dealt_slot(G, g, t);  // the nonzero whose dot product this lane holds
        if (o < end) p.out[o] = p.mask ? __ldg(p.mask + o) * r : r;
    }
}

// Inner dimension beyond 1024: the partial dot products of a pass are accumulated over segments of
// 32*R float4 of the two rows and reduced once per pass, as in the single-matrix kernel for long rows.
// `sub` of 1 << p.shift warps that share the row: this warp takes every (1 << shift)-th nonzero of a pass.
template <int R, bool KSPLIT>
__device__ __forceinline__ void sddmm_one_row_long(const RowProblem &p, int row, int sub, int lane)
{
    constexpr int G = 32, kSeg = G * R;
    const int kmask = (1 << p.shift) - 1;
    const int start = __ldg(p.row_offsets + row), end = __ldg(p.row_offsets + row + 1);
    if (start >= end) return;
    const float4 *lhs4 = reinterpret_cast<const float4 *>(p.a) + (size_t)row * (size_t)p.chunks;
    const float4 *rhs4 = reinterpret_cast<const float4 *>(p.b);
    int col_next = start + lane < end ? __ldg(p.cols + start + lane) : -1;
    for (int base = start; base < end; base += 32) {
        const int q = base + lane;
        const int col = col_next;
        col_next = q + 32 < end ? __ldg(p.cols + q + 32) : -1;
        float part[G];
#pragma unroll
        for (int k = 0; k < G; k++) part[k] = 0.f;
        for (int seg = 0; seg < p.chunks; seg += kSeg) {
            const int len = min(kSeg, p.chunks - seg);
            float4 a[R];
            load_row_chunks<G, R>(lhs4 + seg, len, lane, a);
            sddmm_accumulate<G, R, KSPLIT>(part, a, rhs4 + seg, len, p.chunks, col, 0, lane, kmask, sub);
        }
        group_transpose_reduce<G>(part, lane);
        if (q < end && (!KSPLIT || (lane & kmask) == sub)) p.out[q] = p.mask ? __ldg(p.mask + q) * part[0] : part[0];
    }
}

// `sub` of 1 << p.shift warps of the thread block that share the row: this warp takes the passes sub,
// sub + (1 << shift), ...; the partial rows of the others are handed to the row's first warp through
// `part` ([kWarps][G * R] float4 of shared memory) and added in a fixed order, as in the single-matrix
// kernel for patterns with few rows.  Every warp of the block calls this for the same tile (warps
// without a row included), because of the barrier inside.
template <int G, int R, bool SHARED>
__device__ __forceinline__ void fused_one_row(const RowProblem &p, int row, int sub, bool has_row, int warp, int lane,
                                              float4 *part)
{
    const int g = lane / G, t = lane % G;
    float4 acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_row) {
        const int start = __ldg(p.row_offsets + row) + 32 * sub, end = __ldg(p.row_offsets + row + 1);
        if (start < end) {
            const float4 *c4 = reinterpret_cast<const float4 *>(p.a) + (size_t)row * (size_t)p.chunks;
            float4 q[R];
            load_row_chunks<G, R>(c4, p.chunks, t, q);
            float run_max = -INFINITY, run_sum = 0.f;
            fused_row_passes<G, R, kPlain>(p.cols, q, reinterpret_cast<const float4 *>(p.b),
                                           reinterpret_cast<const float4 *>(p.d), p.chunks, start, end, 32 << p.shift, 1.f,
                                           lane, acc, run_max, run_sum);
        }
    }
    if (SHARED && p.shift > 0) {  // uniform over the block
        if (sub != 0 && g == 0) {
#pragma unroll
            for (int r = 0; r < R; r++) part[warp * (G * R) + r * G + t] = acc[r];
        }
        __syncthreads();
        if (sub == 0 && g == 0) {
            for (int o = 1; o < (1 << p.shift); o++) {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const float4 v = part[(warp + o) * (G * R) + r * G + t];
                    acc[r].x += v.x;
                    acc[r].y += v.y;
                    acc[r].z += v.z;
                    acc[r].w += v.w;
                }
            }
        }
        __syncthreads();  // `part` is reused by the block's next tile
    }
    if (has_row && sub == 0 && g == 0) {  // rows without entries are written as zeros
        float4 *e4 = reinterpret_cast<float4 *>(p.out) + (size_t)row * (size_t)p.chunks;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int idx = r * G + t;
            if (idx < p.chunks) e4[idx] = acc[r];
        }
    }
}

// Persistent launch over the rows of all problems of one class.  A tile is eight slots (rows, or
// parts of rows where warps share them) of one problem; tile_start[i] is the first tile of problem i,
// tile_start[count] the total.  BLOCK: a thread block pulls a tile from the device counter and its
// warps take the eight slots together, which the fused chain needs where warps share rows (partial
// rows meet in shared memory behind a barrier).  Otherwise every warp pulls one slot at a time for
// itself (the counter counts slots): no barrier, so a warp with a short row does not wait for the
// longest row of its tile.
template <int G, int R, int OP, bool BLOCK>
__global__ void __launch_bounds__(kWarps * 32)
rows_batched_kernel(const RowProblem *__restrict__ problems, const long long *__restrict__ tile_start, int count,
                    unsigned long long *counter)
{
    __shared__ unsigned long long s_tile;
    __shared__ float4 part[OP == kOpFused && BLOCK ? kWarps * G * R : 1];  // partial rows of warps that share a row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total = tile_start[count];
    for (;;) {
        long long tile;
        int in_tile;
        if constexpr (BLOCK) {
            if (threadIdx.x == 0) s_tile = atomicAdd(counter, 1ull);
            __syncthreads();
            tile = (long long)s_tile;
            in_tile = warp;
            __syncthreads();
        } else {
            unsigned long long s = 0;
            if (lane == 0) s = atomicAdd(counter, 1ull);
            s = __shfl_sync(0xffffffffu, s, 0);
            tile = (long long)(s / kWarps);
            in_tile = (int)(s % kWarps);
        }
        if (tile >= total) break;
        int lo = 0, hi = count - 1;  // last problem whose first tile is <= tile
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(tile_start + mid) <= tile) lo = mid;
            else hi = mid - 1;
        }
        const RowProblem p = problems[lo];
        const int slot = (int)(tile - __ldg(tile_start + lo)) * kWarps + in_tile;
        const int row = slot >> p.shift, sub = slot & ((1 << p.shift) - 1);
        if constexpr (OP == kOpFused) {
            if (BLOCK || row < p.M) fused_one_row<G, R, BLOCK>(p, row, sub, row < p.M, warp, lane, part);
        } else if (row < p.M) {
            if constexpr (OP == kOpSddmmLongShared) sddmm_one_row_long<R, true>(p, row, sub, lane);
            else if constexpr (OP == kOpSddmmLong) sddmm_one_row_long<R, false>(p, row, 0, lane);
            else sddmm_one_row<G, R>(p, row, sub, lane);
        }
    }
}

int layout_class(int G, int R)
{
    if (G == 8) return R == 1 ? 0 : R == 2 ? 1 : 2;
    if (G == 16) return 3;
    return R == 4 ? 4 : 5;
}

template <int G, int R, int OP, bool BLOCK>
int launch_kernel(dlspm_ctx *ctx, const RowProblem *d_tab, const long long *d_starts, int count, long long tiles,
                  unsigned long long *d_counter, cudaStream_t st)
{
    int per_sm = 0;
    DLSPM_CUDA_TRY(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rows_batched_kernel<G, R, OP, BLOCK>,
                                                                      kWarps * 32, 0));
    const long long want = std::min<long long>(tiles, (long long)ctx->sm_count * std::max(per_sm, 1));
    rows_batched_kernel<G, R, OP, BLOCK><<<(unsigned)want, kWarps * 32, 0, st>>>(d_tab, d_starts, count, d_counter);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

// `shared`: some problem of the class has warps sharing rows.  Only the fused chain needs the
// block-wide form for that.
template <int G, int R, int OP>
int launch_class(dlspm_ctx *ctx, const RowProblem *d_tab, const long long *d_starts, int count, long long tiles,
                 unsigned long long *d_counter, bool shared, cudaStream_t st)
{
    if constexpr (OP == kOpFused) {
        if (shared) return launch_kernel<G, R, OP, true>(ctx, d_tab, d_starts, count, tiles, d_counter, st);
    }
    return launch_kernel<G, R, OP, false>(ctx, d_tab, d_starts, count, tiles, d_counter, st);
}

template <int OP>
int launch_class_by_index(dlspm_ctx *ctx, int cls, const RowProblem *d_tab, const long long *d_starts, int count,
                          long long tiles, unsigned long long *d_counter, bool shared, cudaStream_t st)
{
    switch (cls) {
    case 0: return launch_class<8, 1, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 1: return launch_class<8, 2, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 2: return launch_class<8, 4, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 3: return launch_class<16, 4, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 4: return launch_class<32, 4, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 5: return launch_class<32, 8, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 6: return launch_class<32, 8, kOpSddmmLong>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 7: return launch_class<32, 4, kOpSddmmLong>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 8: return launch_class<32, 8, kOpSddmmLongShared>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 9: return launch_class<32, 4, kOpSddmmLongShared>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    case 10: return launch_class<4, 1, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    default: return launch_class<4, 2, OP>(ctx, d_tab, d_starts, count, tiles, d_counter, shared, st);
    }
}

int side_streams_init(dlspm_ctx *ctx)
{
    if (ctx->side_ready) return DLSPM_OK;
    for (int i = 0; i < kSideStreams; i++) {
        DLSPM_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->side_stream[i], cudaStreamNonBlocking));
        DLSPM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->side_join[i], cudaEventDisableTiming));
    }
    DLSPM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->side_fork, cudaEventDisableTiming));
    ctx->side_ready = 1;
    return DLSPM_OK;
}

struct HostEntry {
    RowProblem p;
    double work;
    double avg_row;
    int index;
};

// Classes with too few rows to fill the device with one warp per row: rows are shared between 2, 4 or
// 8 warps, as the single-matrix launchers do for lone patterns (SDDMM: the outputs of different
// nonzeros are independent, nothing is combined; fused chain: partial rows are added through shared
// memory).  Register-resident rows (classes 0..5, 10, 11) deal out
// the passes of 32 nonzeros, as long as a warp keeps about one pass; rows beyond 1024 floats (classes
// 6, 7) deal out the nonzeros inside every pass and move to the classes 8, 9, whose kernels carry the
// extra test.
void choose_sharing(const dlspm_ctx *ctx, std::vector<HostEntry> (&by_class)[kClasses])
{
    const long long want = (long long)ctx->sm_count * 32;
    for (int c = 0; c < kClasses; c++) {
        if (c == 8 || c == 9) continue;  // filled below from 6 and 7
        std::vector<HostEntry> &v = by_class[c];
        long long rows = 0;
        for (const HostEntry &e : v) rows += e.p.M;
        if (v.empty() || rows * 4 >= want * 3) continue;
        int cls_shift = 0;
        while (cls_shift < 3 && (rows << cls_shift) < want) cls_shift++;
        for (HostEntry &e : v) {
            int s = 0;
            if (c < 6 || c >= 10) {
                while (s < cls_shift && e.avg_row > 32.0 * (1 << s)) s++;
            } else {
                s = cls_shift;
            }
            e.p.shift = s;
        }
        if (c == 6 || c == 7) {  // shared long rows run on the kernels with the extra test
            for (HostEntry &e : v)
                if (e.p.shift > 0) by_class[c + 2].push_back(e);
            v.erase(std::remove_if(v.begin(), v.end(), [](const HostEntry &e) { return e.p.shift > 0; }), v.end());
        }
    }
}

// Device layout of the tables of one call inside `tables`: per class its problems, then its tile
// index, then all counters.
size_t padded256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace

// Bytes of device memory the tables of a grouped SDDMM / fused launch of `count` problems need.
size_t dlspm_rows_batched_table_bytes(int count)
{
    return padded256(sizeof(RowProblem) * (size_t)count) + (size_t)kClasses * 256 +
           padded256(sizeof(long long) * ((size_t)count + kClasses)) + 256 * (size_t)kClasses + 256;
}

namespace {

// Launches the grouped kernels for the entries (already validated, all eligible for the 128-bit
// path) with their tables at `tables`; `pinned` (optional) is host memory of the same size to build
// the tables in, for asynchronous copies.
template <int OP>
int rows_batched_at(dlspm_ctx *ctx, std::vector<HostEntry> (&by_class)[kClasses], void *tables, void *pinned,
                    cudaStream_t st)
{
    size_t total = 0;
    for (int c = 0; c < kClasses; c++) total += by_class[c].size();
    if (total == 0) return DLSPM_OK;
    // host image of the tables
    const size_t tab_bytes = padded256(sizeof(RowProblem) * total) + (size_t)kClasses * 256;
    const size_t starts_bytes = padded256(sizeof(long long) * (total + kClasses)) + 256 * (size_t)kClasses;
    const size_t image_bytes = tab_bytes + starts_bytes;
    std::vector<unsigned char> local;
    unsigned char *img = (unsigned char *)pinned;
    if (!img) {
        local.resize(image_bytes);
        img = local.data();
    }
    size_t tab_off[kClasses], st_off[kClasses];
    long long tiles[kClasses];
    bool shared[kClasses];
    size_t toff = 0, soff = tab_bytes;
    for (int c = 0; c < kClasses; c++) {
        std::vector<HostEntry> &v = by_class[c];
        std::stable_sort(v.begin(), v.end(), [](const HostEntry &x, const HostEntry &y) { return x.work > y.work; });
        tab_off[c] = toff;
        st_off[c] = soff;
        RowProblem *tab = (RowProblem *)(img + toff);
        long long *starts = (long long *)(img + soff);
        long long run = 0;
        shared[c] = false;
        for (size_t i = 0; i < v.size(); i++) {
            tab[i] = v[i].p;
            shared[c] = shared[c] || v[i].p.shift > 0;
            starts[i] = run;
            run += (long long)((((long long)v[i].p.M << v[i].p.shift) + kWarps - 1) / kWarps);
        }
        starts[v.size()] = run;
        tiles[c] = run;
        toff += padded256(sizeof(RowProblem) * v.size());
        soff += padded256(sizeof(long long) * (v.size() + 1));
    }
    char *base = (char *)tables;
    unsigned long long *d_counters = (unsigned long long *)(base + image_bytes);
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(base, img, image_bytes, cudaMemcpyHostToDevice, st));
    DLSPM_CUDA_TRY(ctx, cudaMemsetAsync(d_counters, 0, 256, st));
    // The launches of the classes are independent: the first runs on the caller's stream, the others
    // on side streams forked from it after the table copy and joined back afterwards, so that a batch
    // with several inner dimensions takes about as long as its slowest class, not the sum.
    int live = 0;
    for (int c = 0; c < kClasses; c++) live += (!by_class[c].empty() && tiles[c] > 0) ? 1 : 0;
    if (live > 1) {
        int rc = side_streams_init(ctx);
        if (rc) return rc;
        DLSPM_CUDA_TRY(ctx, cudaEventRecord(ctx->side_fork, st));
    }
    int used = 0;
    for (int c = 0; c < kClasses; c++) {
        if (by_class[c].empty() || tiles[c] == 0) continue;
        cudaStream_t sc = used == 0 ? st : ctx->side_stream[used - 1];
        if (used > 0) DLSPM_CUDA_TRY(ctx, cudaStreamWaitEvent(sc, ctx->side_fork, 0));
        int rc = launch_class_by_index<OP>(ctx, c, (const RowProblem *)(base + tab_off[c]),
                                           (const long long *)(base + st_off[c]), (int)by_class[c].size(), tiles[c],
                                           d_counters + c, shared[c], sc);
        if (rc) return rc;
        if (used > 0) {
            DLSPM_CUDA_TRY(ctx, cudaEventRecord(ctx->side_join[used - 1], sc));
            DLSPM_CUDA_TRY(ctx, cudaStreamWaitEvent(st, ctx->side_join[used - 1], 0));
        }
        used++;
    }
    return DLSPM_OK;
}

int reject_capture(dlspm_ctx *ctx, cudaStream_t st, const char *who)
{
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &status) != cudaSuccess) {
        (void)cudaGetLastError();
        status = cudaStreamCaptureStatusActive;
    }
    if (status != cudaStreamCaptureStatusNone) {
        snprintf(ctx->last_error, sizeof(ctx->last_error),
                 "%s: the stream is being captured; grouped launches copy tables from host memory and cannot be recorded",
                 who);
        return DLSPM_ERR_UNSUPPORTED;
    }
    return DLSPM_OK;
}

}  // namespace

// SDDMM: classifies the problems; eligible ones go to the grouped kernels (tables at `tables`), the
// others run one by one through the single-matrix entry point on the same stream.
int dlspm_sddmm_batched_at(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems, void *tables, void *pinned,
                           cudaStream_t st)
{
    std::vector<HostEntry> by_class[kClasses];
    for (int i = 0; i < count; i++) {
        const dlspm_sddmm_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || q.nnz < 0 || (q.M > 0 && !q.row_offsets) ||
            (q.nnz > 0 && (!q.column_indices || !q.out_values)) || (q.nnz > 0 && q.N > 0 && (!q.lhs || !q.rhs)))
            return DLSPM_ERR_INVALID_ARGUMENT;
    }
    for (int i = 0; i < count; i++) {
        const dlspm_sddmm_problem &q = problems[i];
        if (q.M == 0 || q.nnz == 0) continue;
        int G = 0, R = 0;
        const bool wide = q.N > 0 && dlspm_vec_width(q.N, q.lhs, q.rhs) == 4;
        if (wide) {
            HostEntry e;
            e.p = RowProblem{q.row_offsets, q.column_indices, q.lhs, q.rhs, nullptr, q.mask_values, q.out_values, q.M, q.N / 4, 0};
            e.avg_row = (double)q.nnz / (double)q.M;
            e.work = (double)q.nnz * q.N;
            e.index = i;
            // beyond the register-resident layouts: segments of 1024 floats, of 512 from N = 2052 on
            // (the choice of the single-matrix launcher)
            // rows of up to 32 floats: groups of four lanes, as in the single-matrix launcher
            const int cls = q.N <= 16 ? 10 : q.N <= 32 ? 11 : sddmm_layout(q.N / 4, &G, &R) ? layout_class(G, R) : (q.N > 2048 ? 7 : 6);
            by_class[cls].push_back(e);
        } else {
            int rc = dlspm_sddmm_csr_masked_f32(ctx, q.M, q.K, q.N, q.nnz, q.row_offsets, q.column_indices, q.mask_values,
                                                q.lhs, q.rhs, q.out_values, st);
            if (rc) return rc;
        }
    }
    choose_sharing(ctx, by_class);
    return rows_batched_at<kOpSddmm>(ctx, by_class, tables, pinned, st);
}

int dlspm_fused_batched_at(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems, void *tables, void *pinned,
                           cudaStream_t st)
{
    std::vector<HostEntry> by_class[kClasses];
    for (int i = 0; i < count; i++) {
        const dlspm_fused_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || q.nnz < 0 || (q.M > 0 && !q.row_offsets) || (q.nnz > 0 && !q.column_indices) ||
            (q.M > 0 && q.N > 0 && (!q.C || !q.E)) || (q.nnz > 0 && q.N > 0 && (!q.B || !q.D)))
            return DLSPM_ERR_INVALID_ARGUMENT;
    }
    for (int i = 0; i < count; i++) {
        const dlspm_fused_problem &q = problems[i];
        if (q.M == 0 || q.N == 0) continue;
        int G = 0, R = 0;
        if (dlspm_vec_width(q.N, q.C, q.B, q.D, q.E) == 4 && sddmm_layout(q.N / 4, &G, &R)) {
            HostEntry e;
            e.p = RowProblem{q.row_offsets, q.column_indices, q.C, q.B, q.D, nullptr, q.E, q.M, q.N / 4, 0};
            e.avg_row = (double)q.nnz / (double)q.M;
            e.work = (double)q.nnz * q.N + (double)q.M;  // rows without entries still cost a store
            e.index = i;
            by_class[q.N <= 16 ? 10 : q.N <= 32 ? 11 : layout_class(G, R)].push_back(e);
        } else {
            int rc = dlspm_fused_sddmm_spmm_f32(ctx, q.M, q.K, q.N, q.nnz, q.row_offsets, q.column_indices, q.C, q.B, q.D,
                                                q.E, st);
            if (rc) return rc;
        }
    }
    choose_sharing(ctx, by_class);  // the classes 6..9 are never filled for the fused chain
    return rows_batched_at<kOpFused>(ctx, by_class, tables, pinned, st);
}

extern "C" int dlspm_sddmm_batched_f32(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems, void *stream)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (count == 0) return DLSPM_OK;
    rc = reject_capture(ctx, (cudaStream_t)stream, "dlspm_sddmm_batched_f32");
    if (rc) return rc;
    for (int i = 0; i < count && ctx->check_input; i++) {  // DLSPM_OPT_CHECK_INPUT
        const dlspm_sddmm_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.nnz < 0 || (q.nnz > 0 && !q.column_indices)) return DLSPM_ERR_INVALID_ARGUMENT;
        rc = dlspm_check_input(ctx, q.M, q.K, q.nnz, q.row_offsets, q.column_indices, (cudaStream_t)stream);
        if (rc) return rc;
    }
    rc = dlspm_scratch_reserve(ctx, dlspm_rows_batched_table_bytes(count));
    if (rc) return rc;
    return dlspm_sddmm_batched_at(ctx, count, problems, ctx->scratch, nullptr, (cudaStream_t)stream);
}

extern "C" int dlspm_fused_batched_f32(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems, void *stream)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (count == 0) return DLSPM_OK;
    rc = reject_capture(ctx, (cudaStream_t)stream, "dlspm_fused_batched_f32");
    if (rc) return rc;
    for (int i = 0; i < count && ctx->check_input; i++) {  // DLSPM_OPT_CHECK_INPUT
        const dlspm_fused_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.nnz < 0 || (q.nnz > 0 && !q.column_indices)) return DLSPM_ERR_INVALID_ARGUMENT;
        rc = dlspm_check_input(ctx, q.M, q.K, q.nnz, q.row_offsets, q.column_indices, (cudaStream_t)stream);
        if (rc) return rc;
    }
    rc = dlspm_scratch_reserve(ctx, dlspm_rows_batched_table_bytes(count));
    if (rc) return rc;
    return dlspm_fused_batched_at(ctx, count, problems, ctx->scratch, nullptr, (cudaStream_t)stream);
}
