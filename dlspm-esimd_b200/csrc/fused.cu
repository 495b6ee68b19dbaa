// Fused SDDMM -> SpMM for sm_100a: E = (pattern(A) .* (C * B^T)) * D, the sampled products never
// leave the registers.
//
// One warp per row.  A pass takes 32 nonzeros: their dot products are formed exactly as in the
// SDDMM kernel (group layout and transposing butterfly of sddmm_device.cuh), which leaves the score
// of nonzero `lane` on that lane.  The same lane groups then gather the D rows of their own
// nonzeros and accumulate score * D[col, :] into R float4 registers per lane; when the row is done
// the 32/G group partial sums are added with shuffles and one group stores the row of E.
// The reference keeps a 32-score vector per row in registers in the same way
// (FUSED/fused-esimd_cb.cpp:130-154); it needs a zeroed E for empty rows, this kernel writes them.
//
// The same kernels carry two optional steps between the two products (template parameter MODE):
// a scale factor on the sampled products, and a softmax over the stored entries of each row
// (sparse attention).  The softmax is the streaming form: a running maximum and a running sum per
// row, and the partial output row is rescaled whenever the maximum grows, so a row is still read
// once and nothing is written besides the output row.
#include <cstdint>

#include "common.cuh"
#include "fused_device.cuh"
#include "sddmm_device.cuh"

using namespace dlspm;

namespace {

constexpr int kWarps = 8;

// CAP: second builds with a register cap, chosen per launch.
//  - one chunk per lane (d <= 32): 32 registers for eight resident blocks instead of six.  It pays
//    when it saves a wave of thread blocks: 8192 rows are 1.15 waves of six blocks per SM but fit
//    one wave of eight (55 -> 33 us at 8192 x 2048, d = 32); with both in one wave (4096 rows) or
//    many waves (32768 rows) the 40-register build is 7 to 8 % faster.
//  - 32 lanes x four chunks (d = 260..512): 64 registers for four resident blocks instead of two:
//    1.3 to 1.5x faster once the pattern has more rows than the uncapped build keeps resident
//    (8192 x 2048, d = 512: 637 -> 479 us), 12 % slower below that.
template <int G, int R, int MODE, bool CAP = false, bool WIDE = false>
__global__ void __launch_bounds__(kWarps * 32, CAP ? (G == 8 ? 8 : 4) : 0)
fused_rows_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                  const float *__restrict__ c, const float *__restrict__ b, const float *__restrict__ d,
                  float *__restrict__ e, int M, int chunks, float scale)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + warp;
    if (row >= M) return;
    const int g = lane / G, t = lane % G;
    const float4 *c4 = reinterpret_cast<const float4 *>(c) + (size_t)row * (size_t)chunks;
    float4 q[R];
    if constexpr (WIDE) load_row_pair(c4, t, q);  // rows of 32 floats, 32-byte aligned: lane t owns chunks 2t, 2t + 1
    else load_row_chunks<G, R>(c4, chunks, t, q);
    float4 acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    float run_max = -INFINITY, run_sum = 0.f;
    fused_row_passes<G, R, MODE, WIDE>(cols, q, reinterpret_cast<const float4 *>(b), reinterpret_cast<const float4 *>(d),
                                       chunks, __ldg(row_offsets + row), __ldg(row_offsets + row + 1), 32, scale, lane,
                                       acc, run_max, run_sum);
    if constexpr (MODE == kSoftmax) {
        const float inv = run_sum > 0.f ? 1.f / run_sum : 0.f;  // empty row: zeros
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r].x *= inv;
            acc[r].y *= inv;
            acc[r].z *= inv;
            acc[r].w *= inv;
        }
    }
    if (g == 0) {
        float4 *e4 = reinterpret_cast<float4 *>(e) + (size_t)row * (size_t)chunks;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int idx = WIDE ? 2 * t + r : r * G + t;
            if (idx < chunks) e4[idx] = acc[r];
        }
    }
}

// Patterns with few rows: 1 << split_shift warps of a thread block share a row and take its passes
// in turn; their partial rows (and, for the softmax, their running maxima and sums) are combined
// through shared memory in a fixed order by the first warp of the row.
template <int G, int R, int MODE>
__global__ void __launch_bounds__(kWarps * 32)
fused_rows_split_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                        const float *__restrict__ c, const float *__restrict__ b, const float *__restrict__ d,
                        float *__restrict__ e, int M, int chunks, float scale, int split_shift)
{
    extern __shared__ float4 part[];  // [kWarps][G * R]
    __shared__ float stat[kWarps][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = blockIdx.x * kWarps + warp;
    const int row = slot >> split_shift, sub = slot & ((1 << split_shift) - 1);
    const bool active = row < M;
    const int g = lane / G, t = lane % G;
    float4 acc[R];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
    float run_max = -INFINITY, run_sum = 0.f;
    if (active) {
        const int start = __ldg(row_offsets + row) + 32 * sub, end = __ldg(row_offsets + row + 1);
        if (start < end) {
            const float4 *c4 = reinterpret_cast<const float4 *>(c) + (size_t)row * (size_t)chunks;
            float4 q[R];
            load_row_chunks<G, R>(c4, chunks, t, q);
            fused_row_passes<G, R, MODE>(cols, q, reinterpret_cast<const float4 *>(b),
                                         reinterpret_cast<const float4 *>(d), chunks, start, end, 32 << split_shift,
                                         scale, lane, acc, run_max, run_sum);
        }
    }
    if (sub != 0 && g == 0) {
#pragma unroll
        for (int r = 0; r < R; r++) part[warp * (G * R) + r * G + t] = acc[r];
    }
    if (lane == 0) {
        stat[warp][0] = run_max;
        stat[warp][1] = run_sum;
    }
    __syncthreads();
    if (!active || sub != 0 || g != 0) return;
    const int others = (1 << split_shift) - 1;
    if constexpr (MODE == kSoftmax) {
        float top = run_max;
        for (int s = 1; s <= others; s++) top = fmaxf(top, stat[warp + s][0]);
        if (top == -INFINITY) {  // empty row: zeros
            run_sum = 0.f;
        } else {
            const float own = expf(run_max - top);
            run_sum *= own;
#pragma unroll
            for (int r = 0; r < R; r++) {
                acc[r].x *= own;
                acc[r].y *= own;
                acc[r].z *= own;
                acc[r].w *= own;
            }
            for (int s = 1; s <= others; s++) {
                const float w = expf(stat[warp + s][0] - top);  // 0 for a warp that had no pass
                run_sum += stat[warp + s][1] * w;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const float4 v = part[(warp + s) * (G * R) + r * G + t];
                    acc[r].x = fmaf(w, v.x, acc[r].x);
                    acc[r].y = fmaf(w, v.y, acc[r].y);
                    acc[r].z = fmaf(w, v.z, acc[r].z);
                    acc[r].w = fmaf(w, v.w, acc[r].w);
                }
            }
        }
        const float inv = run_sum > 0.f ? 1.f / run_sum : 0.f;
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r].x *= inv;
            acc[r].y *= inv;
            acc[r].z *= inv;
            acc[r].w *= inv;
        }
    } else {
        for (int s = 1; s <= others; s++) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float4 v = part[(warp + s) * (G * R) + r * G + t];
                acc[r].x += v.x;
                acc[r].y += v.y;
                acc[r].z += v.z;
                acc[r].w += v.w;
            }
        }
    }
    float4 *e4 = reinterpret_cast<float4 *>(e) + (size_t)row * (size_t)chunks;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int idx = r * G + t;
        if (idx < chunks) e4[idx] = acc[r];
    }
}

// Any N and alignment.  The output row is produced in slabs of 128 columns per pass over the row's
// nonzeros; scores are recomputed for every slab, so nothing is spilled to memory.
template <int MODE>
__global__ void __launch_bounds__(kWarps * 32)
fused_generic_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                     const float *__restrict__ c, const float *__restrict__ b, const float *__restrict__ d,
                     float *__restrict__ e, int M, int N, float scale)
{
    constexpr int U = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + warp;
    if (row >= M) return;
    const float *crow = c + (size_t)row * (size_t)N;
    const int start = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
    for (int n0 = 0; n0 < N; n0 += 32 * U) {
        float acc[U];
#pragma unroll
        for (int u = 0; u < U; u++) acc[u] = 0.f;
        [[maybe_unused]] float run_max = -INFINITY, run_sum = 0.f;
        for (int base = start; base < end; base += 32) {
            const int p = base + lane;
            const int col = p < end ? __ldg(cols + p) : 0;
            const int cnt = min(32, end - base);
            for (int k = 0; k < cnt; k++) {
                const int cc = __shfl_sync(0xffffffffu, col, k);
                const float *brow = b + (size_t)cc * (size_t)N;
                float s = 0.f;
                for (int l = lane; l < N; l += 32) s = fmaf(__ldg(crow + l), __ldg(brow + l), s);
#pragma unroll
                for (int w = 16; w >= 1; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
                if constexpr (MODE == kScaled) s *= scale;
                if constexpr (MODE == kSoftmax) {
                    const float x = s * scale;
                    const float m_new = fmaxf(run_max, x);
                    const float corr = expf(run_max - m_new);
                    s = expf(x - m_new);
                    run_sum = run_sum * corr + s;
                    run_max = m_new;
#pragma unroll
                    for (int u = 0; u < U; u++) acc[u] *= corr;
                }
                const float *drow = d + (size_t)cc * (size_t)N;
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = n0 + u * 32 + lane;
                    if (j < N) acc[u] = fmaf(s, __ldg(drow + j), acc[u]);
                }
            }
        }
        [[maybe_unused]] const float inv = run_sum > 0.f ? 1.f / run_sum : 0.f;
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int j = n0 + u * 32 + lane;
            if constexpr (MODE == kSoftmax) acc[u] *= inv;
            if (j < N) e[(size_t)row * (size_t)N + j] = acc[u];
        }
    }
}

// Widths that rule out 128-bit loads (N not a multiple of 4, or unaligned operands) up to 256 floats:
// the group layout of the fast path with scalar elements, as in the SDDMM kernel for such widths.
// Lane t of a group of G lanes owns the elements e*G + t of a dense row; the row of C stays in
// registers, scores are formed with dealt passes and the transposing butterfly, every lane group
// gathers the D rows of its own nonzeros, and the groups' partial rows are added with shuffles when
// the row is done.  The any-width kernel above runs a full-warp reduction per nonzero and re-reads
// the row of C every time.
template <int G, int E, int MODE>
__global__ void __launch_bounds__(kWarps * 32)
fused_rows_scalar_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                         const float *__restrict__ c, const float *__restrict__ b, const float *__restrict__ d,
                         float *__restrict__ e, int M, int N, float scale)
{
    constexpr int NG = 32 / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarps + warp;
    if (row >= M) return;
    const int g = lane / G, t = lane % G;
    const int start = __ldg(row_offsets + row), end = __ldg(row_offsets + row + 1);
    const float *crow = c + (size_t)row * (size_t)N;
    float q[E], acc[E];
#pragma unroll
    for (int i = 0; i < E; i++) {
        const int idx = i * G + t;
        q[i] = idx < N ? __ldg(crow + idx) : 0.f;
        acc[i] = 0.f;
    }
    [[maybe_unused]] float run_max = -INFINITY, run_sum = 0.f;
    int col_next = start + lane < end ? __ldg(cols + start + lane) : -1;
    for (int base = start; base < end; base += 32) {
        const int col = col_next;
        col_next = base + 32 + lane < end ? __ldg(cols + base + 32 + lane) : -1;
        float part[G];
#pragma unroll
        for (int k = 0; k < G; k++) {
            const int cc = __shfl_sync(0xffffffffu, col, k * NG + g);
            float dot = 0.f;
            if (cc >= 0) {
                const float *brow = b + (size_t)cc * (size_t)N;
#pragma unroll
                for (int i = 0; i < E; i++) {
                    const int idx = i * G + t;
                    if (idx < N) dot = fmaf(q[i], __ldg(brow + idx), dot);
                }
            }
            part[k] = dot;
        }
        group_transpose_reduce<G>(part, t);
        float score = part[0];  // of nonzero base + sddmm_dealt_slot(G, g, t), whose column sits on that lane
        if constexpr (MODE == kScaled) score *= scale;
        if constexpr (MODE == kSoftmax) {
            const bool stored = base + sddmm_dealt_slot(G, g, t) < end;
            const float x = stored ? score * scale : -INFINITY;
            const float m_new = fmaxf(run_max, warp_max(x));
            const float corr = expf(run_max - m_new);
            score = stored ? expf(x - m_new) : 0.f;
            run_sum = run_sum * corr + warp_sum(score);
            run_max = m_new;
#pragma unroll
            for (int i = 0; i < E; i++) acc[i] *= corr;
        }
#pragma unroll
        for (int k = 0; k < G; k++) {
            const int cc = __shfl_sync(0xffffffffu, col, k * NG + g);  // the group's k-th nonzero
            const float s = __shfl_sync(0xffffffffu, score, g * G + k);
            if (cc >= 0) {
                const float *drow = d + (size_t)cc * (size_t)N;
#pragma unroll
                for (int i = 0; i < E; i++) {
                    const int idx = i * G + t;
                    if (idx < N) acc[i] = fmaf(s, __ldg(drow + idx), acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int s = G; s < 32; s <<= 1) {
#pragma unroll
        for (int i = 0; i < E; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], s);
    }
    [[maybe_unused]] const float inv = run_sum > 0.f ? 1.f / run_sum : 0.f;  // empty row: zeros
    if (g == 0) {
#pragma unroll
        for (int i = 0; i < E; i++) {
            const int idx = i * G + t;
            if constexpr (MODE == kSoftmax) acc[i] *= inv;
            if (idx < N) e[(size_t)row * (size_t)N + idx] = acc[i];
        }
    }
}

template <int G, int MODE>
void launch_scalar(const int *ro, const int *ci, const float *c, const float *b, const float *d, float *e, int M, int N,
                   float scale, cudaStream_t st)
{
    const unsigned blocks = (unsigned)dlspm_ceil_div(M, kWarps);
    const int per_lane = dlspm_ceil_div(N, G);
    if (per_lane <= 2) fused_rows_scalar_kernel<G, 2, MODE><<<blocks, kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, N, scale);
    else if (per_lane <= 4) fused_rows_scalar_kernel<G, 4, MODE><<<blocks, kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, N, scale);
    else fused_rows_scalar_kernel<G, 8, MODE><<<blocks, kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, N, scale);
}

// Patterns of one to a few waves of thread blocks, as in the SDDMM launcher: two or four warps per row
// make the waves finer where the last one would be nearly empty (6144 or 12288 rows).  A shared row
// costs more here than in SDDMM (every warp loads the row of C, partial rows are combined through
// shared memory): 15 % per doubling in the estimate.
inline int fused_wave_shift(long long blocks, long long resident, double avg_row)
{
    if (blocks <= resident || blocks > 8 * resident) return 0;
    int best = 0;
    double best_cost = 1e30;
    for (int s = 0; s <= 2 && avg_row > 32.0 * (1 << s); s++) {
        const long long waves = ((blocks << s) + resident - 1) / resident;
        const double cost = (double)waves / (double)(1 << s) * (1.0 + 0.15 * s);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

template <int G, int R, int MODE>
void launch_fast(const int *ro, const int *ci, const float *c, const float *b, const float *d, float *e,
                 int M, int chunks, float scale, int split_shift, int sm_count, cudaStream_t st, double avg_row = 0.0,
                 bool wide = false)
{
    if (split_shift == 0 && avg_row > 0.0) {
        static int per_sm = 0;  // resident blocks of the plain build of this layout
        if (per_sm == 0) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fused_rows_kernel<G, R, MODE>, kWarps * 32, 0) != cudaSuccess) {
                (void)cudaGetLastError();
                n = 4;
            }
            per_sm = n > 0 ? n : 4;
            if (G == 8 && R == 1) per_sm = 8;  // this layout has a capped build for eight resident blocks (below)
        }
        split_shift = fused_wave_shift(((long long)M + kWarps - 1) / kWarps, (long long)per_sm * sm_count, avg_row);
    }
    if (split_shift > 0) {
        const long long warps = (long long)M << split_shift;
        const size_t smem = sizeof(float4) * (size_t)kWarps * G * R;
        fused_rows_split_kernel<G, R, MODE><<<(unsigned)((warps + kWarps - 1) / kWarps), kWarps * 32, smem, st>>>(
            ro, ci, c, b, d, e, M, chunks, scale, split_shift);
        return;
    }
    if constexpr (G == 32 && R == 4) {
        if ((long long)M > 2LL * kWarps * sm_count) {  // more rows than two resident blocks per SM hold
            fused_rows_kernel<G, R, MODE, true><<<dlspm_ceil_div(M, kWarps), kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, chunks, scale);
            return;
        }
    }
    if constexpr (G == 8 && R == 1) {
        // waves of thread blocks times blocks per wave, the capped build 7 % slower per block
        const long long blocks = dlspm_ceil_div(M, kWarps);
        const long long w6 = (blocks + 6LL * sm_count - 1) / (6LL * sm_count), w8 = (blocks + 8LL * sm_count - 1) / (8LL * sm_count);
        if ((double)w8 * 8.0 * 1.07 < (double)w6 * 6.0) {
            fused_rows_kernel<G, R, MODE, true><<<(unsigned)blocks, kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, chunks, scale);
            return;
        }
    }
    if constexpr (G == 4 && R == 2) {
        if (wide) {  // rows of 32 floats, 32-byte aligned operands, a long launch: 256-bit loads
            fused_rows_kernel<G, R, MODE, false, true><<<dlspm_ceil_div(M, kWarps), kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, chunks, scale);
            return;
        }
    }
    fused_rows_kernel<G, R, MODE><<<dlspm_ceil_div(M, kWarps), kWarps * 32, 0, st>>>(ro, ci, c, b, d, e, M, chunks, scale);
}

// Warps per row (as a shift) for a pattern with few rows, by the rule of the SDDMM kernel: share
// rows until about 32 warps per SM exist or a warp would get less than one full pass; leave
// patterns alone that nearly fill one wave as they are.
int fused_split_shift(const dlspm_ctx *ctx, int M, int N, int nnz)
{
    // two gathers per nonzero make a warp's pass heavier than in SDDMM: from N = 128 on, half as
    // many warps already keep the L1 pipe busy (2048 x 512 at 20 %, N = 128 lost 17 % with more)
    const long long want = (long long)ctx->sm_count * (N >= 128 ? 16 : 32);
    if ((long long)M * 4 >= want * 3) return 0;
    const double avg = (double)nnz / (double)(M > 0 ? M : 1);
    int shift = 0;
    while (shift < 3 && ((long long)M << shift) < want && avg > 32.0 * (1 << shift)) shift++;
    return shift;
}

template <int MODE>
int fused_launch(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                 const int *column_indices, const float *C, const float *B, const float *D, float *E,
                 float scale, void *stream)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (M > 0 && !row_offsets) return DLSPM_ERR_INVALID_ARGUMENT;
    if (nnz > 0 && !column_indices) return DLSPM_ERR_INVALID_ARGUMENT;
    if (M > 0 && N > 0 && (!C || !E)) return DLSPM_ERR_INVALID_ARGUMENT;
    if (nnz > 0 && N > 0 && (!B || !D)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = dlspm_check_input(ctx, M, K, nnz, row_offsets, column_indices, (cudaStream_t)stream);
    if (rc) return rc;
    if (M == 0 || N == 0) return DLSPM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = dlspm_vec_width(N, C, B, D, E);
    int G = 0, R = 0;
    if (vec == 4 && sddmm_layout(N / 4, &G, &R)) {
        const int chunks = N / 4;
        const int shift = fused_split_shift(ctx, M, N, nnz);
        if (chunks <= 8) {  // rows of up to 32 floats: groups of four lanes, as in the SDDMM kernel (16384 x 4096 at
                            // 30 %, d = 16: 389 -> 184 us; 8192 x 8192 at 30 %, d = 32: 462 -> 357 us)
            if (chunks <= 4) launch_fast<4, 1, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
            else {
                const bool wide = chunks == 8 && ((uintptr_t)C % 32) == 0 && ((uintptr_t)B % 32) == 0 && ((uintptr_t)D % 32) == 0 &&
                                  (long long)M * 10 >= 69LL * kWarps * ctx->sm_count;
                launch_fast<4, 2, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M, wide);
            }
            DLSPM_CUDA_TRY(ctx, cudaGetLastError());
            return DLSPM_OK;
        }
        if (G == 8 && R == 1) launch_fast<8, 1, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 8 && R == 2) launch_fast<8, 2, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 8 && R == 4) launch_fast<8, 4, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 16) launch_fast<16, 4, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
        else if (G == 32 && R == 4) launch_fast<32, 4, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
        else launch_fast<32, 8, MODE>(row_offsets, column_indices, C, B, D, E, M, chunks, scale, shift, ctx->sm_count, st, (double)nnz / (double)M);
    } else if (N <= 256) {  // no 128-bit loads: the group layout with scalar elements
        if (N <= 64) launch_scalar<8, MODE>(row_offsets, column_indices, C, B, D, E, M, N, scale, st);
        else if (N <= 128) launch_scalar<16, MODE>(row_offsets, column_indices, C, B, D, E, M, N, scale, st);
        else launch_scalar<32, MODE>(row_offsets, column_indices, C, B, D, E, M, N, scale, st);
    } else {
        fused_generic_kernel<MODE><<<dlspm_ceil_div(M, kWarps), kWarps * 32, 0, st>>>(row_offsets, column_indices, C, B, D, E, M, N, scale);
    }
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    return DLSPM_OK;
}

}  // namespace

extern "C" int dlspm_fused_sddmm_spmm_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                          const int *row_offsets, const int *column_indices,
                                          const float *C, const float *B, const float *D, float *E,
                                          void *stream)
{
    return fused_launch<kPlain>(ctx, M, K, N, nnz, row_offsets, column_indices, C, B, D, E, 1.f, stream);
}

extern "C" int dlspm_fused_attention_f32(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                         const int *row_offsets, const int *column_indices,
                                         const float *Q, const float *Kmat, const float *V, float *O,
                                         float scale, unsigned flags, void *stream)
{
    if (flags & ~(unsigned)DLSPM_ATTN_SOFTMAX) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!(scale == scale) || scale - scale != 0.f) return DLSPM_ERR_INVALID_ARGUMENT;  // NaN or infinite
    if (flags & DLSPM_ATTN_SOFTMAX)
        return fused_launch<kSoftmax>(ctx, M, K, N, nnz, row_offsets, column_indices, Q, Kmat, V, O, scale, stream);
    return fused_launch<kScaled>(ctx, M, K, N, nnz, row_offsets, column_indices, Q, Kmat, V, O, scale, stream);
}
