// Sampled dense-dense matrix multiplication on a CSR pattern for sm_100a.
//
// One warp per row of the pattern.  The lhs row lives in registers for the whole row; rhs rows are
// gathered with 128-bit loads; dot products are finished with a transposing butterfly (see
// sddmm_device.cuh), and the 32 results of a pass are written with one coalesced store.  There are
// no atomics (the reference's v4 kernel adds partial sums atomically and needs a zeroed output,
// SDDMM/sddmm-esimd-fromfile_v4.hpp:161), so results are deterministic and every output element is
// written exactly once.
#include <cstdint>

#include "common.cuh"
#include "sddmm_device.cuh"

using namespace dlspm;

namespace {

constexpr int kWarps = 8;

// `mask` (may be null) holds one factor per stored entry: out[p] = mask[p] * dot.
// CAP: compiled for eight resident thread blocks (32 registers).  For the two-chunk layout (inner
// dimension 36 to 64) that is 1.5 to 1.65x faster once the pattern has more rows than fit the device
// at once (8192 x 8192, N = 64: 156 -> 94 us) and 13 % slower below that (4096 rows), so the launcher
// picks by the number of warps.  The one-chunk layout needs 32 registers anyway.  The 32-lane layouts
// are held to five (four chunks per lane) and four (eight chunks) resident blocks: 8192 x 2048 with
// N = 512 went 296 -> 255 us, with N = 1024 754 -> 480 us; one block more lost 15 to 35 % again.
template <int G, int R, bool KSPLIT, bool CAP = false, bool WIDE = false>
__global__ void __launch_bounds__(kWarps * 32, CAP ? 8 : ((G == 32 && R == 4 && !KSPLIT) ? 5 : ((G == 32 && R == 8 && !KSPLIT) ? 4 : 0)))
sddmm_rows_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                  const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out,
                  int M, int chunks, const float *__restrict__ mask, int split_shift, int k_shift)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // (1 << split_shift) * (1 << k_shift) warps share a row: the passes of 32 nonzeros are dealt
    // out in turn, and within a pass a warp takes every (1 << k_shift)-th nonzero of each lane
    // group.  The outputs of different nonzeros are independent, so nothing is combined afterwards.
    const int slot = (blockIdx.x * kWarps + warp) >> k_shift;
    const int kmask = (1 << k_shift) - 1, ksub = (blockIdx.x * kWarps + warp) & kmask;
    const int row = slot >> split_shift;
    if (row >= M) return;
    const int stride = 32 << split_shift;
    const int g = lane / G, t = lane % G;
    const float4 *lhs4 = reinterpret_cast<const float4 *>(lhs) + (size_t)row * (size_t)chunks;
    const float4 *rhs4 = reinterpret_cast<const float4 *>(rhs);
    const int start = __ldg(row_offsets + row) + 32 * (slot & ((1 << split_shift) - 1));
    const int end = __ldg(row_offsets + row + 1);
    if (start >= end) return;
    float4 a[R];
    if constexpr (WIDE) load_row_pair(lhs4, t, a);  // N = 32, 32-byte aligned operands: see sddmm_pass_dealt_wide
    else load_row_chunks<G, R>(lhs4, chunks, t, a);
    // the column indices of the next pass are fetched before this pass is computed, so that their
    // latency does not sit in front of the rhs gathers of every pass
    int col_next = start + lane < end ? __ldg(cols + start + lane) : -1;
    for (int base = start; base < end; base += stride) {
        const int p = base + lane;
        const int col = col_next;
        col_next = p + stride < end ? __ldg(cols + p + stride) : -1;
        if constexpr (KSPLIT) {
            const float r = sddmm_pass<G, R, true>(a, rhs4, chunks, col, g, t, kmask, ksub);
            if (p < end && (t & kmask) == ksub) out[p] = mask ? __ldg(mask + p) * r : r;
        } else {
            // nonzeros dealt to the lane groups in turn: this lane ends up with nonzero `q` of the row
            float r;
            if constexpr (WIDE) r = sddmm_pass_dealt_wide(a, rhs4, col, g, t);
            else r = sddmm_pass_dealt<G, R>(a, rhs4, chunks, col, g, t);
            const int q = base + sddmm_dealt_slot(G, g, t);
            if (q < end) out[q] = mask ? __ldg(mask + q) * r : r;
        }
    }
}

// Inner dimension beyond 1024 (16-byte aligned rows): the lanes' partial dot products of a pass are
// accumulated over segments of 32*R float4 and reduced once at the end of the pass; the lhs segment
// is re-read from L1 for every pass, which adds 3 % to the rhs traffic.
// (512-float segments: held to four resident blocks, 8192 x 2048 with N = 3136 1766 -> 1629 us.)
template <int R, bool KSPLIT>
__global__ void __launch_bounds__(kWarps * 32, (R == 4 && !KSPLIT) ? 4 : 0)
sddmm_rows_long_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                       const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out,
                       int M, int chunks, const float *__restrict__ mask, int k_shift)
{
    constexpr int G = 32, kSeg = G * R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1 << k_shift warps share a row, each taking every (1 << k_shift)-th nonzero of a pass
    const int slot = blockIdx.x * kWarps + warp;
    const int kmask = (1 << k_shift) - 1, ksub = slot & kmask;
    const int row = slot >> k_shift;
    if (row >= M) return;
    const float4 *lhs4 = reinterpret_cast<const float4 *>(lhs) + (size_t)row * (size_t)chunks;
    const float4 *rhs4 = reinterpret_cast<const float4 *>(rhs);
    const int start = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
    int col_next = start + lane < end ? __ldg(cols + start + lane) : -1;
    for (int base = start; base < end; base += 32) {
        const int p = base + lane;
        const int col = col_next;
        col_next = p + 32 < end ? __ldg(cols + p + 32) : -1;
        float part[G];
#pragma unroll
        for (int k = 0; k < G; k++) part[k] = 0.f;
        for (int seg = 0; seg < chunks; seg += kSeg) {
            const int len = min(kSeg, chunks - seg);
            float4 a[R];
            load_row_chunks<G, R>(lhs4 + seg, len, lane, a);
            sddmm_accumulate<G, R, KSPLIT>(part, a, rhs4 + seg, len, chunks, col, 0, lane, kmask, ksub);
        }
        group_transpose_reduce<G>(part, lane);
        if (p < end && (!KSPLIT || (lane & kmask) == ksub)) out[p] = mask ? __ldg(mask + p) * part[0] : part[0];
    }
}

// Any N and alignment: each lane strides over the row; one full-warp reduction per nonzero.
template <int VEC>
__global__ void __launch_bounds__(kWarps * 32)
sddmm_generic_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                     const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out,
                     int M, int N, const float *__restrict__ mask)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + warp;
    if (row >= M) return;
    const float *arow = lhs + (size_t)row * (size_t)N;
    const int start = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
    for (int base = start; base < end; base += 32) {
        const int p = base + lane;
        const int col = p < end ? __ldg(cols + p) : 0;
        const int cnt = min(32, end - base);
        float mine = 0.f;
        for (int k = 0; k < cnt; k++) {
            const int c = __shfl_sync(0xffffffffu, col, k);
            const float *brow = rhs + (size_t)c * (size_t)N;
            float acc = 0.f;
            for (int l = lane * VEC; l < N; l += 32 * VEC) {
                if constexpr (VEC == 4) {
                    acc = dot4(__ldg(reinterpret_cast<const float4 *>(arow + l)),
                               __ldg(reinterpret_cast<const float4 *>(brow + l)), acc);
                } else if constexpr (VEC == 2) {
                    const float2 x = __ldg(reinterpret_cast<const float2 *>(arow + l));
                    const float2 y = __ldg(reinterpret_cast<const float2 *>(brow + l));
                    acc = fmaf(x.x, y.x, acc);
                    acc = fmaf(x.y, y.y, acc);
                } else {
                    acc = fmaf(__ldg(arow + l), __ldg(brow + l), acc);
                }
            }
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
            if (lane == k) mine = acc;
        }
        if (p < end) out[p] = mask ? __ldg(mask + p) * mine : mine;
    }
}

// Rows that rule out 128-bit loads (N not a multiple of 4, or unaligned operands) up to 256 floats:
// the group layout of the fast path with scalar elements.  Lane t of a group of G lanes owns the
// elements e*G + t (e = 0..E-1) of a dense row, so a group reads G consecutive floats per load; the
// lhs row stays in registers, the nonzeros of a pass are dealt to the groups in turn and the
// transposing butterfly finishes G dot products with G-1 shuffles per lane.  The any-width kernel
// above re-reads the lhs row and runs a full-warp reduction (five shuffles) for every nonzero; at
// N = 49, a width of the data set's own table, that is three times the instructions.
template <int G, int E>
__global__ void __launch_bounds__(kWarps * 32)
sddmm_rows_scalar_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                         const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out,
                         int M, int N, const float *__restrict__ mask, int split_shift)
{
    constexpr int NG = 32 / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1 << split_shift warps share a row and take its passes in turn (patterns with few rows)
    const int slot = blockIdx.x * kWarps + warp;
    const int row = slot >> split_shift;
    if (row >= M) return;
    const int g = lane / G, t = lane % G;
    const int stride = 32 << split_shift;
    const int start = __ldg(row_offsets + row) + 32 * (slot & ((1 << split_shift) - 1));
    const int end = __ldg(row_offsets + row + 1);
    if (start >= end) return;
    const float *arow = lhs + (size_t)row * (size_t)N;
    float a[E];
#pragma unroll
    for (int e = 0; e < E; e++) {
        const int idx = e * G + t;
        a[e] = idx < N ? __ldg(arow + idx) : 0.f;
    }
    int col_next = start + lane < end ? __ldg(cols + start + lane) : -1;
    for (int base = start; base < end; base += stride) {
        const int col = col_next;
        col_next = base + stride + lane < end ? __ldg(cols + base + stride + lane) : -1;
        float part[G];
#pragma unroll
        for (int k = 0; k < G; k++) {
            const int c = __shfl_sync(0xffffffffu, col, k * NG + g);
            float acc = 0.f;
            if (c >= 0) {
                const float *brow = rhs + (size_t)c * (size_t)N;
#pragma unroll
                for (int e = 0; e < E; e++) {
                    const int idx = e * G + t;
                    if (idx < N) acc = fmaf(a[e], __ldg(brow + idx), acc);
                }
            }
            part[k] = acc;
        }
        group_transpose_reduce<G>(part, t);
        const int q = base + sddmm_dealt_slot(G, g, t);
        if (q < end) out[q] = mask ? __ldg(mask + q) * part[0] : part[0];
    }
}

template <int G>
void launch_scalar(const int *ro, const int *ci, const float *lhs, const float *rhs, float *out, int M, int N,
                   const float *mask, int split_shift, cudaStream_t st)
{
    const unsigned blocks = (unsigned)((((long long)M << split_shift) + kWarps - 1) / kWarps);
    const int per_lane = dlspm_ceil_div(N, G);
    if (per_lane <= 2) sddmm_rows_scalar_kernel<G, 2><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, N, mask, split_shift);
    else if (per_lane <= 4) sddmm_rows_scalar_kernel<G, 4><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, N, mask, split_shift);
    else sddmm_rows_scalar_kernel<G, 8><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, N, mask, split_shift);
}

// Patterns of one to a few waves of thread blocks: the last wave is often nearly empty (6144 rows are
// 768 blocks for 592 resident ones, i.e. two waves for 1.3 waves of work).  Two or four warps per
// row make the blocks shorter and the waves finer; a shared row costs about 8 % per doubling (every
// warp loads the lhs row, shorter runs per warp).  Returns the shift with the least estimated time.
inline int sddmm_wave_shift(long long blocks, long long resident, double avg_row)
{
    if (blocks <= resident) {
        // Less than one wave (4096 rows with N = 32 are 512 blocks for 1184 resident ones): the device
        // is partly empty and the launch lasts as long as one warp needs for its row, so rows are
        // shared while the launch still fits in one wave and a warp keeps more than one pass.
        int s = 0;
        while (s < 2 && (blocks << (s + 1)) <= resident && avg_row > 64.0 * (1 << s)) s++;
        return s;
    }
    if (blocks > 8 * resident) return 0;
    int best = 0;
    double best_cost = 1e30;
    for (int s = 0; s <= 2 && avg_row > 32.0 * (1 << s); s++) {
        const long long waves = ((blocks << s) + resident - 1) / resident;
        const double cost = (double)waves / (double)(1 << s) * (1.0 + 0.08 * s);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

template <int G, int R>
void launch_fast(const int *ro, const int *ci, const float *lhs, const float *rhs, float *out, int M,
                 int chunks, const float *mask, int split_shift, int k_shift, int sm_count, cudaStream_t st,
                 double avg_row = 0.0, bool wide = false)
{
    if (split_shift == 0 && k_shift == 0 && avg_row > 0.0) {
        static int per_sm = 0;  // resident blocks of the plain build of this layout
        if (per_sm == 0) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sddmm_rows_kernel<G, R, false>, kWarps * 32, 0) != cudaSuccess) {
                (void)cudaGetLastError();
                n = 4;
            }
            per_sm = n > 0 ? n : 4;
        }
        split_shift = sddmm_wave_shift(((long long)M + kWarps - 1) / kWarps, (long long)per_sm * sm_count, avg_row);
    }
    const long long warps = (long long)M << (split_shift + k_shift);
    const unsigned blocks = (unsigned)((warps + kWarps - 1) / kWarps);
    if constexpr (G == 8 && R == 2) {
        // the capped build pays when it saves a wave of thread blocks (eight instead of six per SM)
        const long long w6 = (blocks + 6LL * sm_count - 1) / (6LL * sm_count), w8 = (blocks + 8LL * sm_count - 1) / (8LL * sm_count);
        if (k_shift == 0 && (double)w8 * 8.0 * 1.07 < (double)w6 * 6.0) {
            sddmm_rows_kernel<G, R, false, true><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, chunks, mask, split_shift, 0);
            return;
        }
    }
    if constexpr (G == 4 && R == 2) {
        if (wide && k_shift == 0) {
            sddmm_rows_kernel<G, R, false, false, true><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, chunks, mask, split_shift, 0);
            return;
        }
    }
    if (k_shift > 0)
        sddmm_rows_kernel<G, R, true><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, chunks, mask, split_shift, k_shift);
    else
        sddmm_rows_kernel<G, R, false><<<blocks, kWarps * 32, 0, st>>>(ro, ci, lhs, rhs, out, M, chunks, mask, split_shift, 0);
}

// Warps per row (as a shift) for a pattern with few rows: one warp per row would leave most of the
// device idle and walk the row's passes one after the other, so rows are shared until about 32
// warps per SM exist or a warp would get less than one full pass.  Measured (lone launches, warm
// L2, before -> after): 2048 x 512 at 20 %, N = 128: 12.6 -> 10.0 us; 1024 x 1024 at 10 %: 14.8 ->
// 7.1 us; 512 x 2048 at 10 %, N = 256: 34.5 -> 8.0 us; 4096-row patterns lost 15 % when shared and
// are left alone.
int sddmm_split_shift(const dlspm_ctx *ctx, int M, int nnz)
{
    const long long want = (long long)ctx->sm_count * 32;
    const double avg = (double)nnz / (double)(M > 0 ? M : 1);
    if ((long long)M * 4 >= want * 3) return 0;  // nearly one full wave already: sharing only adds a second one
    int shift = 0;
    while (shift < 3 && ((long long)M << shift) < want && avg > 32.0 * (1 << shift)) shift++;
    return shift;
}

// Further sharing inside a pass for patterns that are still far from filling the device (few and
// short rows, e.g. a 64 x 576 layer with a long inner dimension): each of 2, 4 or 8 warps takes
// every 2nd, 4th or 8th nonzero of a lane group.  `shared` = warps per row already decided.
// `min_row`: shortest average row for which this is done.  Every sharing warp loads the lhs row and
// runs the butterfly again, and the kernel with the extra test batches fewer loads; measured on the
// register-resident path, 512 x 128 at 10 % (13 nonzeros per row, N = 784) lost 16 to 35 % at any
// sharing factor while 128 x 512 (51 per row) gained 2.2x, so short rows are left alone there.
// With a long inner dimension (segmented kernel) every case measured gained (64 x 576, N = 3136:
// 112 -> 43 us; 64 x 64: 23 -> 15 us).
int sddmm_k_shift(const dlspm_ctx *ctx, int M, int nnz, int shared_shift, double min_row)
{
    const long long want = (long long)ctx->sm_count * 32;
    const double avg = (double)nnz / (double)(M > 0 ? M : 1);
    if (avg < min_row) return 0;
    int k = 0;
    while (k < 3 && ((long long)M << (shared_shift + k)) * 2 <= want) k++;
    return k;
}

int sddmm_launch(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                 const int *column_indices, const float *mask, const float *lhs, const float *rhs,
                 float *out_values, void *stream)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (M > 0 && !row_offsets) return DLSPM_ERR_INVALID_ARGUMENT;
    if (nnz > 0 && (!column_indices || !out_values)) return DLSPM_ERR_INVALID_ARGUMENT;
    if (nnz > 0 && N > 0 && (!lhs || !rhs)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    rc = dlspm_check_input(ctx, M, K, nnz, row_offsets, column_indices, st);
    if (rc) return rc;
    if (M == 0 || nnz == 0) return DLSPM_OK;
    if (N == 0) {  // empty dot products
        DLSPM_CUDA_TRY(ctx, cudaMemsetAsync(out_values, 0, sizeof(float) * (size_t)nnz, st));
        return DLSPM_OK;
    }
    const int vec = dlspm_vec_width(N, lhs, rhs);
    int G = 0, R = 0;
    const int blocks = dlspm_ceil_div(M, kWarps);
    if (vec == 4 && sddmm_layout(N / 4, &G, &R)) {
        const int chunks = N / 4;
        const int shift = sddmm_split_shift(ctx, M, nnz);
        const int kshift = sddmm_k_shift(ctx, M, nnz, shift, 16.0);
        const double avg_row = (double)nnz / (double)M;
#ifndef DLSPM_NO_NARROW_GROUPS
        // Rows of up to 32 floats: groups of 4 lanes (8 nonzeros in flight per step instead of 4, a
        // butterfly of 3 shuffles instead of 7).  Warps that share the nonzeros inside a pass select
        // by the index within a group, so at most 4 warps can do that with groups of 4.
        if (chunks <= 8 && kshift <= 2) {
            if (chunks <= 4) launch_fast<4, 1>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, avg_row);
            else {
                // N = 32 with 32-byte aligned operands: one 256-bit load per lane and nonzero.  That build
                // needs 42 registers instead of 32 (five resident blocks instead of eight), which costs a
                // launch of less than about a wave more than the halved L1 traffic gains (GFLOP/s at 30 %
                // nonzeros: 1024 x 1024 1977 -> 1557, 4096 x 4096 6336 -> 5898, but 8192 x 8192
                // 6498 -> 7182, 16384 x 4096 6862 -> 9398, 32768 x 8192 7133 -> 8979): from 8192 rows on.
                const bool wide = chunks == 8 && ((uintptr_t)lhs % 32) == 0 && ((uintptr_t)rhs % 32) == 0 &&
                                  (long long)blocks * 10 >= 69LL * ctx->sm_count;
                launch_fast<4, 2>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, avg_row, wide);
            }
            DLSPM_CUDA_TRY(ctx, cudaGetLastError());
            return DLSPM_OK;
        }
#endif
        if (G == 8 && R == 1) launch_fast<8, 1>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 8 && R == 2) launch_fast<8, 2>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 8 && R == 4) launch_fast<8, 4>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 16) launch_fast<16, 4>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 32 && R == 4) launch_fast<32, 4>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
        else launch_fast<32, 8>(row_offsets, column_indices, lhs, rhs, out_values, M, chunks, mask, shift, kshift, ctx->sm_count, st, (double)nnz / (double)M);
    } else if (vec == 4) {
        // measured: 512-float segments (80 registers, 3 blocks per SM) win from N = 3136, 1024-float
        // segments below that
        const int kshift = sddmm_k_shift(ctx, M, nnz, 0, 0.0);
        const unsigned lblocks = (unsigned)((((long long)M << kshift) + kWarps - 1) / kWarps);
        if (N > 2048 && kshift > 0) sddmm_rows_long_kernel<4, true><<<lblocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N / 4, mask, kshift);
        else if (N > 2048) sddmm_rows_long_kernel<4, false><<<lblocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N / 4, mask, 0);
        else if (kshift > 0) sddmm_rows_long_kernel<8, true><<<lblocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N / 4, mask, kshift);
        else sddmm_rows_long_kernel<8, false><<<lblocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N / 4, mask, 0);
    } else if (N <= 256) {  // no 128-bit loads: the group layout with scalar elements
        const int shift = sddmm_split_shift(ctx, M, nnz);
        if (N <= 64) launch_scalar<8>(row_offsets, column_indices, lhs, rhs, out_values, M, N, mask, shift, st);
        else if (N <= 128) launch_scalar<16>(row_offsets, column_indices, lhs, rhs, out_values, M, N, mask, shift, st);
        else launch_scalar<32>(row_offsets, column_indices, lhs, rhs, out_values, M, N, mask, shift, st);
    } else if (vec == 2) {
        sddmm_generic_kernel<2><<<blocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N, mask);
    } else {
        sddmm_generic_kernel<1><<<blocks, kWarps * 32, 0, st>>>(row_offsets, column_indices, lhs, rhs, out_values, M, N, mask);
    }
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

}  // namespace

extern "C" int dlspm_sddmm_csr_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                                   const int *column_indices, const float *lhs, const float *rhs,
                                   float *out_values, void *stream)
{
    return sddmm_launch(ctx, M, K, N, nnz, row_offsets, column_indices, nullptr, lhs, rhs, out_values, stream);
}

extern "C" int dlspm_sddmm_csr_masked_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                                          const int *column_indices, const float *mask_values,
                                          const float *lhs, const float *rhs, float *out_values, void *stream)
{
    return sddmm_launch(ctx, M, K, N, nnz, row_offsets, column_indices, mask_values, lhs, rhs, out_values, stream);
}
