// Tiled SpMM for the denser problems (from roughly 15-20 % nonzeros, rows with strictly ascending
// columns): a thread block owns 64 rows x 256 columns of C and walks K in chunks of 32 rows of B.
//
// The row-gather kernel moves 512 bytes of B through L1 for every nonzero and 128 columns; ncu shows
// it at 87 % of the L1 data-pipe peak, i.e. at its ceiling (about one fifth of the fp32 peak).  The
// way past that ceiling is to load a row of B once and use it for several rows of A.  Here a warp
// owns 8 rows of the tile and all 256 columns (8 per lane):
//   * the B chunk (32 rows x 1 KiB) comes into shared memory by bulk asynchronous copies
//     (cp.async.bulk, one per row, completion counted on an mbarrier), double buffered;
//   * each warp turns the next 32 columns of its 8 rows from CSR into a small dense block plus one
//     32-bit presence mask per row: the <= 32 next entries of a row are fetched with cp.async
//     straight into shared memory while the previous chunk is being computed, then the entries that
//     fall into the chunk (a prefix, since columns ascend) are scattered by column;
//   * per column k of the chunk the warp loads its 8 columns of B[k] once (two 128-bit loads) and
//     walks its 8 rows: the mask bit guards the 8 FMAs of an entry (the compiler predicates them;
//     explicit branches measured slower).  Columns that no row of the warp uses are skipped before
//     the B load.
// Only present entries are multiplied, in ascending column order, so every output element sums the
// same products in the same order as the row-gather kernel and the reference host loop
// (SPMM/spmm-esimd-fromfile.cpp:63-83): results are bit-identical to the row-gather kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dlspm {

constexpr int kTileM = 64, kTileN = 256, kTileK = 32;
constexpr int kTileThreads = 256;
constexpr int kTileRowsPerWarp = kTileM / 8;
constexpr unsigned kWaitLimit = 1u << 24;  // polls of an mbarrier before the kernel gives up

struct TileProblem {
    const float *values;
    const int *row_offsets;
    const int *cols;
    const float *B;
    float *C;
    const int *row_order;  // rows from the longest to the shortest (nullptr: natural order)
    int M, K, N;
    int row_blocks;  // ceil(M / 64)
    int col_blocks;  // ceil(N / 256)
    int pad;
};

struct TileSmem {
    float Bs[2][kTileK][kTileN];          // 64 KiB: B chunk, two stages
    float As[2][kTileM][kTileK];          // 16 KiB: A chunk by (row, column in chunk); only masked entries are valid
    int cand_col[kTileM][32];             //  8 KiB: next <= 32 entries of every row (staged by cp.async)
    float cand_val[kTileM][32];           //  8 KiB
    unsigned Am[2][kTileM];               // presence mask of the chunk per row
    int cursor[kTileM];                   // next unconsumed entry of every row
    int row_end[kTileM];
    int row_id[kTileM];                   // row of C behind every tile slot (-1: none)
    unsigned long long full[2];           // mbarriers: B chunk landed
    unsigned long long tile;
    int abort;                            // set by a thread whose bounded wait ran out
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false after kWaitLimit polls (the caller records the failure and leaves).
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity)
{
    for (unsigned i = 0; i < kWaitLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, unsigned bytes, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void cp_async_4(void *dst, const void *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Issues the B chunk starting at row k0 into stage s (called by warp 0 only).  Rows past the end of
// B (last chunk when K is not a multiple of 32) are written as zeros: the masked inner loop never
// reads them, but the zero-filled variant multiplies every row of the chunk, and stale shared
// memory there could hold a NaN.
__device__ __forceinline__ void tile_load_b(TileSmem &sm, const TileProblem &p, int s, int k0, int n0, int lane)
{
    const int cols = min(kTileN, p.N - n0);
    const unsigned row_bytes = (unsigned)cols * 4u;
    const int rows = min(kTileK, p.K - k0);
    if (rows < kTileK) {
        for (int r = rows; r < kTileK; r++)
            for (int c = lane * 4; c < kTileN; c += 128)
                *reinterpret_cast<float4 *>(&sm.Bs[s][r][c]) = make_float4(0.f, 0.f, 0.f, 0.f);
        fence_async_smem();  // these generic-proxy writes precede later bulk copies into the same rows
        __syncwarp();
    }
    if (lane == 0) mbar_expect_tx(&sm.full[s], row_bytes * (unsigned)rows);
    __syncwarp();
    if (lane < rows)
        bulk_copy_g2s(&sm.Bs[s][lane][0], p.B + (size_t)(k0 + lane) * (size_t)p.N + n0, row_bytes, &sm.full[s]);
}

// Starts the asynchronous fetch of the next <= 32 entries of this warp's rows.
__device__ __forceinline__ void tile_fetch_candidates(TileSmem &sm, const TileProblem &p, int warp, int lane)
{
#pragma unroll
    for (int i = 0; i < kTileRowsPerWarp; i++) {
        const int r = warp * kTileRowsPerWarp + i;
        const int q = sm.cursor[r] + lane;
        if (q < sm.row_end[r]) {
            cp_async_4(&sm.cand_col[r][lane], p.cols + q);
            cp_async_4(&sm.cand_val[r][lane], p.values + q);
        }
    }
}

// Scatters the fetched entries that fall into columns [k0, k0+32) into As[s] and writes the masks.
// DENSE: absent entries are written as zeros, so that the inner loop can run without mask tests.
template <bool DENSE>
__device__ __forceinline__ void tile_expand_a(TileSmem &sm, int s, int k0, int warp, int lane)
{
    cp_async_wait_all();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kTileRowsPerWarp; i++) {
        const int r = warp * kTileRowsPerWarp + i;
        const int cur = sm.cursor[r];
        int c = -1;
        float v = 0.f;
        if (cur + lane < sm.row_end[r]) {
            c = sm.cand_col[r][lane] - k0;
            v = sm.cand_val[r][lane];
        }
        const bool take = (unsigned)c < (unsigned)kTileK;  // columns ascend: the taken ones are a prefix
        if constexpr (DENSE) {
            sm.As[s][r][lane] = 0.f;
            __syncwarp();
        }
        if (take) sm.As[s][r][c] = v;
        const unsigned mask = __reduce_or_sync(0xffffffffu, take ? (1u << c) : 0u);
        if (lane == 0) {
            sm.Am[s][r] = mask;
            sm.cursor[r] = cur + __popc(mask);
        }
    }
    __syncwarp();
}

template <bool STRICT>
__device__ __forceinline__ float tmad(float a, float b, float c)
{
    if constexpr (STRICT) return __fadd_rn(c, __fmul_rn(a, b));
    else return fmaf(a, b, c);
}

template <bool STRICT>
__device__ __forceinline__ void row_update(float (&acc)[8], float av, const float4 &b0, const float4 &b1)
{
    acc[0] = tmad<STRICT>(av, b0.x, acc[0]);
    acc[1] = tmad<STRICT>(av, b0.y, acc[1]);
    acc[2] = tmad<STRICT>(av, b0.z, acc[2]);
    acc[3] = tmad<STRICT>(av, b0.w, acc[3]);
    acc[4] = tmad<STRICT>(av, b1.x, acc[4]);
    acc[5] = tmad<STRICT>(av, b1.y, acc[5]);
    acc[6] = tmad<STRICT>(av, b1.z, acc[6]);
    acc[7] = tmad<STRICT>(av, b1.w, acc[7]);
}

// Persistent thread blocks pull tile numbers from `counter`; tile_start[i] is the first tile of
// problem i.  On an mbarrier timeout error[0] is set to 1 and the block returns.
template <bool STRICT, bool DENSE>
__global__ void __launch_bounds__(kTileThreads, 2)
spmm_tile_kernel(const TileProblem *__restrict__ problems, const long long *__restrict__ tile_start, int count,
                 unsigned long long *counter, int *error)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    TileSmem &sm = *reinterpret_cast<TileSmem *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wr = warp * kTileRowsPerWarp;

    if (tid == 0) {
        mbar_init(&sm.full[0], 1);
        mbar_init(&sm.full[1], 1);
        sm.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    unsigned phase0 = 0, phase1 = 0;  // parity of the next completion of each stage's barrier
    const long long total = tile_start[count];

    for (;;) {
        if (tid == 0) sm.tile = atomicAdd(counter, 1ull);
        __syncthreads();
        const long long tile = (long long)sm.tile;
        if (tile >= total) break;
        int lo = 0, hi = count - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(tile_start + mid) <= tile) lo = mid;
            else hi = mid - 1;
        }
        const TileProblem p = problems[lo];
        const int t = (int)(tile - __ldg(tile_start + lo));
        const int cb = t / p.row_blocks, rb = t - cb * p.row_blocks;
        const int n0 = cb * kTileN;

        if (tid < kTileM) {
            const int slot = rb * kTileM + tid;
            int row = -1, cur = 0, end = 0;
            if (slot < p.M) {
                row = p.row_order ? __ldg(p.row_order + slot) : slot;
                cur = __ldg(p.row_offsets + row);
                end = __ldg(p.row_offsets + row + 1);
            }
            sm.row_id[tid] = row;
            sm.cursor[tid] = cur;
            sm.row_end[tid] = end;
        }
        __syncthreads();

        float acc[kTileRowsPerWarp][8];
#pragma unroll
        for (int i = 0; i < kTileRowsPerWarp; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

        const int nchunks = (p.K + kTileK - 1) / kTileK;
        if (warp == 0) tile_load_b(sm, p, 0, 0, n0, lane);
        tile_fetch_candidates(sm, p, warp, lane);
        tile_expand_a<DENSE>(sm, 0, 0, warp, lane);

        bool aborted = false;
        for (int c = 0; c < nchunks; c++) {
            const int s = c & 1;
            const bool more = c + 1 < nchunks;
            if (more) {
                if (warp == 0) tile_load_b(sm, p, s ^ 1, (c + 1) * kTileK, n0, lane);
                tile_fetch_candidates(sm, p, warp, lane);  // lands while this chunk is computed
            }
            const unsigned parity = s ? phase1 : phase0;
            // A thread whose wait runs out raises the flag and still walks to the barrier below,
            // so that the whole block leaves together.
            if (!mbar_wait(&sm.full[s], parity)) *(volatile int *)&sm.abort = 1;
            if (s) phase1 ^= 1u;
            else phase0 ^= 1u;

            if constexpr (DENSE) {
                // every entry of the 8 x 32 block is multiplied; absent ones are zeros
#pragma unroll 2
                for (int k4 = 0; k4 < kTileK; k4 += 4) {
                    float4 a[kTileRowsPerWarp];
#pragma unroll
                    for (int i = 0; i < kTileRowsPerWarp; i++) a[i] = *reinterpret_cast<const float4 *>(&sm.As[s][wr + i][k4]);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const float4 b0 = *reinterpret_cast<const float4 *>(&sm.Bs[s][k4 + kk][lane * 4]);
                        const float4 b1 = *reinterpret_cast<const float4 *>(&sm.Bs[s][k4 + kk][128 + lane * 4]);
#pragma unroll
                        for (int i = 0; i < kTileRowsPerWarp; i++) {
                            const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
                            row_update<STRICT>(acc[i], av, b0, b1);
                        }
                    }
                }
            } else {
            unsigned m[kTileRowsPerWarp];
            unsigned any = 0;
#pragma unroll
            for (int i = 0; i < kTileRowsPerWarp; i++) {
                m[i] = sm.Am[s][wr + i];
                any |= m[i];
            }
#pragma unroll 1
            for (int k4 = 0; k4 < kTileK; k4 += 4) {
                const unsigned any4 = (any >> k4) & 0xFu;
                if (any4 == 0u) continue;  // none of this warp's rows uses these four columns
                float4 a[kTileRowsPerWarp];
                unsigned mk[kTileRowsPerWarp];
#pragma unroll
                for (int i = 0; i < kTileRowsPerWarp; i++) {
                    a[i] = *reinterpret_cast<const float4 *>(&sm.As[s][wr + i][k4]);
                    mk[i] = m[i] >> k4;
                }
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    if ((any4 >> kk) & 1u) {
                        const float4 b0 = *reinterpret_cast<const float4 *>(&sm.Bs[s][k4 + kk][lane * 4]);
                        const float4 b1 = *reinterpret_cast<const float4 *>(&sm.Bs[s][k4 + kk][128 + lane * 4]);
#pragma unroll
                        for (int i = 0; i < kTileRowsPerWarp; i++) {
                            const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
                            if (mk[i] & (1u << kk)) row_update<STRICT>(acc[i], av, b0, b1);
                        }
                    }
                }
            }
            }
            if (more) tile_expand_a<DENSE>(sm, s ^ 1, (c + 1) * kTileK, warp, lane);
            __syncthreads();  // every warp is done with Bs[s]: it may be refilled in the next round
            if (*(volatile int *)&sm.abort) {
                aborted = true;
                break;
            }
        }
        if (aborted) {
            // Record the failure, give the copies still in flight one more bounded chance to land
            // in this block's shared memory, and leave without storing the tile.
            if (tid == 0) {
                atomicExch(error, 1);
                (void)mbar_wait(&sm.full[0], phase0);
                (void)mbar_wait(&sm.full[1], phase1);
            }
            __syncthreads();
            return;
        }

#pragma unroll
        for (int i = 0; i < kTileRowsPerWarp; i++) {
            const int row = sm.row_id[wr + i];
            if (row >= 0) {
                float *crow = p.C + (size_t)row * (size_t)p.N + n0;
                if (n0 + lane * 4 < p.N)
                    *reinterpret_cast<float4 *>(crow + lane * 4) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                if (n0 + 128 + lane * 4 < p.N)
                    *reinterpret_cast<float4 *>(crow + 128 + lane * 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
            }
        }
    }
}

}  // namespace dlspm
