// Tiled SpMM for the denser problems (from roughly a quarter nonzeros, rows with strictly ascending
// columns): one thread block per SM owns 128 rows x 256 columns of C at a time and walks K in chunks
// of 32 rows of B.
//
// The row-gather kernel moves 512 bytes of B through L1 for every nonzero and 128 columns; ncu shows
// it at 87 % of the L1 data-pipe peak, i.e. at its ceiling (one L1 wavefront per FMA instruction, a
// quarter of the fp32 peak).  The way past that ceiling is to load a row of B once and use it for
// several rows of A from registers.  Roles inside a block of 17 warps, which never meet at a
// block-wide barrier:
//   * one producer warp streams B: the 32 x 256 chunk of every (tile, chunk) step goes into one of
//     four shared-memory stages by bulk asynchronous copies (cp.async.bulk, one per row, completion
//     counted on the stage's `full` mbarrier).  When a chunk has landed the producer tests it for
//     non-finite values (one pass over 32 KiB against the chunk's 524 k multiply-adds), records the
//     answer and arrives on the stage's `ready` mbarrier.  A stage is refilled once all sixteen
//     consumer warps have arrived on its `empty` mbarrier.
//   * sixteen consumer warps own 8 rows of the tile each and all 256 columns (8 per lane, 64
//     accumulators per lane).  Each warp turns the next 32 columns of its 8 rows from CSR into a
//     zero-filled 32 x 8 block in shared memory (private to the warp, double buffered; the next <= 32
//     entries of every row are fetched one chunk ahead with cp.async) plus one presence mask per
//     row.  Per column k of the chunk the warp reads its 8 values of A (two broadcast loads) and its
//     8 columns of B[k] (two 128-bit loads) and issues 64 FMAs.
// Absent entries are multiplied as zeros, which adds +0 to a sum and leaves it unchanged as long as
// B[k] is finite.  For a chunk in which the producer found an infinity or a NaN the consumers run
// the masked loop instead, which multiplies present entries only, so a non-finite value of B
// reaches exactly the rows that reference it, as in the reference host loop
// (SPMM/spmm-esimd-fromfile.cpp:63-83).  Products are added in ascending column order from 0.0f:
// results are bit-identical to the row-gather kernel (the one exception is the sign of a zero: a
// sum that underflowed to -0 becomes +0 when a zero product is added to it).
// Every mbarrier wait is bounded; a wait that runs out raises the block's abort word, which ends
// all roles, sets the error word of the launch and leaves the tile unwritten.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dlspm {

constexpr int kTileN = 256, kTileK = 32;
#ifndef DLSPM_TILE_UNROLL
#define DLSPM_TILE_UNROLL 8
#endif
constexpr int kTileUnroll = DLSPM_TILE_UNROLL;  // columns of a chunk per unrolled step of the multiply loop
#ifndef DLSPM_TILE_CONSUMERS
#define DLSPM_TILE_CONSUMERS 16
#endif
constexpr int kTileConsumers = DLSPM_TILE_CONSUMERS;  // consumer warps per block (a multiple of four)
// Registers per thread: at launch (what a block of this size may have), for the producer's group
// after it has given registers up, and for the consumers after they have taken them.
constexpr int kTileRegsLaunch = kTileConsumers == 16 ? 96 : 128;
constexpr int kTileRegsProducer = kTileConsumers == 16 ? 32 : 40;
constexpr int kTileRegsConsumer = kTileConsumers == 16 ? 112 : 152;
static_assert(kTileConsumers == 16 || kTileConsumers == 12, "register budgets are set for 12 or 16 consumer warps");
static_assert((kTileConsumers + 4) * 32 * kTileRegsLaunch <= 65536 &&
                  kTileConsumers * 32 * kTileRegsConsumer + 128 * kTileRegsProducer <= (kTileConsumers + 4) * 32 * kTileRegsLaunch,
              "register budgets exceed what the block is launched with");
constexpr int kTileRowsPerWarp = 8;
constexpr int kTileM = kTileConsumers * kTileRowsPerWarp;  // 128 rows of C per tile
constexpr int kTileStages = 4;                   // B chunks in flight
// Registers are handed out to a block in units of four warps, so the producer warp costs a whole
// group of four: the block is launched with 20 warps, of which three leave at once.
constexpr int kTileThreads = (kTileConsumers + 4) * 32;
constexpr unsigned kWaitLimit = 1u << 20;  // polls of an mbarrier (a quarter of a microsecond apart) before the kernel gives up

struct TileProblem {
    const float *values;
    const int *row_offsets;
    const int *cols;
    const float *B;
    float *C;
    const int *row_order;  // rows from the longest to the shortest (nullptr: natural order)
    int M, K, N;
    int row_blocks;  // ceil(M / 128)
    int col_blocks;  // ceil(N / 256)
    int pad;
};

struct TileSmem {
    float Bs[kTileStages][kTileK][kTileN];                 // 128 KiB: B chunks
    float As[kTileConsumers][2][kTileK][kTileRowsPerWarp]; //  32 KiB: per warp, A chunk by (column in chunk, row), zero-filled
    int cand_col[kTileConsumers][kTileRowsPerWarp][32];    //  16 KiB: next <= 32 entries of every row (staged by cp.async)
    float cand_val[kTileConsumers][kTileRowsPerWarp][32];  //  16 KiB
    unsigned Am[kTileConsumers][2][kTileRowsPerWarp];      // presence mask of the chunk per row
    unsigned long long full[kTileStages];                  // B chunk landed (transaction bytes)
    unsigned long long ready[kTileStages];                 // B chunk landed and tested (producer arrives)
    unsigned long long empty[kTileStages];                 // all consumer warps are done with the chunk
    int nonfinite[kTileStages];                            // the chunk holds an infinity or a NaN
    int abort;                                             // set by a thread whose bounded wait ran out
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

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up when another thread of the block has raised `abort`.
__device__ __forceinline__ bool mbar_wait_or_abort(unsigned long long *bar, unsigned parity, volatile int *abort)
{
    for (unsigned i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        // a waiting warp must not take issue slots from the warps that compute
        if (i >= 4u) __nanosleep(i < 64u ? 64u : 256u);
        if ((i & 63u) == 63u && *abort) return false;
    }
    return false;
}

// The (tile, chunk) steps of one block in order: tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the
// launch.  Producer and consumers walk the same sequence independently; `g` numbers the chunks of
// the whole sequence and selects stage (g % kTileStages) and barrier parity.
struct TileCursor {
    long long tile;  // current tile number
    int prob;        // its problem
    int rb, n0;      // row block, first column
    int nchunks;     // ceil(K / 32)
};

__device__ __forceinline__ bool tile_cursor_load(TileCursor &tc, const TileProblem *__restrict__ problems,
                                                 const long long *__restrict__ tile_start, int count, long long total,
                                                 TileProblem &p)
{
    if (tc.tile >= total) return false;
    int lo = tc.prob, hi = count - 1;  // tiles only move forward: the search starts at the last problem
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(tile_start + mid) <= tc.tile) lo = mid;
        else hi = mid - 1;
    }
    tc.prob = lo;
    p = problems[lo];
    const int t = (int)(tc.tile - __ldg(tile_start + lo));
    const int cb = t / p.row_blocks;
    tc.rb = t - cb * p.row_blocks;
    tc.n0 = cb * kTileN;
    tc.nchunks = (p.K + kTileK - 1) / kTileK;
    return true;
}

// ---- producer warp --------------------------------------------------------------------------------

// Issues the B chunk starting at row k0 into stage s.  Rows past the end of B (last chunk when K is
// not a multiple of 32) are written as zeros: the zero-filled A block multiplies every row of the
// chunk, and stale shared memory there could hold a NaN.
__device__ __forceinline__ void tile_load_b(TileSmem &sm, const TileProblem &p, int s, int k0, int n0, int lane)
{
    const int cols = min(kTileN, p.N - n0);
    const unsigned row_bytes = (unsigned)cols * 4u;
    const int rows = min(kTileK, p.K - k0);
    if (rows < kTileK) {
        for (int r = rows; r < kTileK; r++)
            for (int c = lane * 4; c < kTileN; c += 128)
                *reinterpret_cast<float4 *>(&sm.Bs[s][r][c]) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // generic-proxy accesses to this stage (the zeros above, the previous test pass) precede the
    // bulk copies, which write through the async proxy
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_expect_tx(&sm.full[s], row_bytes * (unsigned)rows);
    __syncwarp();
    if (lane < rows)
        bulk_copy_g2s(&sm.Bs[s][lane][0], p.B + (size_t)(k0 + lane) * (size_t)p.N + n0, row_bytes, &sm.full[s]);
}

// True if the valid part of the chunk in stage s (rows x cols) holds an infinity or a NaN: the
// largest magnitude bit pattern is compared with that of infinity.
__device__ __forceinline__ bool tile_chunk_nonfinite(const TileSmem &sm, int s, int cols, int lane)
{
    unsigned top = 0u;
    const int c4 = cols >> 2;  // float4 per row that were copied (cols is a multiple of 4)
    if (c4 == kTileN / 4) {
        const uint4 *src = reinterpret_cast<const uint4 *>(&sm.Bs[s][0][0]);
#pragma unroll 8
        for (int i = lane; i < kTileK * kTileN / 4; i += 32) {
            const uint4 v = src[i];
            top = max(top, max(max(v.x & 0x7fffffffu, v.y & 0x7fffffffu), max(v.z & 0x7fffffffu, v.w & 0x7fffffffu)));
        }
    } else {
        for (int r = 0; r < kTileK; r++)
            for (int c = lane; c < c4; c += 32) {
                const uint4 v = *reinterpret_cast<const uint4 *>(&sm.Bs[s][r][c * 4]);
                top = max(top, max(max(v.x & 0x7fffffffu, v.y & 0x7fffffffu), max(v.z & 0x7fffffffu, v.w & 0x7fffffffu)));
            }
    }
    return __any_sync(0xffffffffu, top >= 0x7f800000u);
}

// The producer's whole life: for every chunk of the block's sequence, refill a free stage; one step
// behind, test the chunk that has landed and hand it to the consumers.  Returns false if a wait
// ran out (after the copies still in flight have been given a bounded chance to land).
__device__ __forceinline__ bool tile_producer(TileSmem &sm, const TileProblem *__restrict__ problems,
                                              const long long *__restrict__ tile_start, int count, long long total,
                                              int lane)
{
    volatile int *abort = &sm.abort;
    TileCursor tc{(long long)blockIdx.x, 0, 0, 0, 0};
    TileProblem p;
    bool have = tile_cursor_load(tc, problems, tile_start, count, total, p);
    int c = 0;               // chunk of the current tile to issue next
    unsigned g = 0;          // chunks issued so far
    int prev_cols = 0;       // columns of the chunk issued last (for its test)
    bool ok = true;
    while (have || g > 0) {
        const bool issue = have;
        int cols_now = 0;
        if (issue) {
            const int s = (int)(g % kTileStages);
            if (g >= (unsigned)kTileStages)
                ok = mbar_wait_or_abort(&sm.empty[s], ((g / kTileStages) - 1u) & 1u, abort);
            if (!ok) break;
            tile_load_b(sm, p, s, c * kTileK, tc.n0, lane);
            cols_now = min(kTileN, p.N - tc.n0);
        }
        if (g > 0) {  // the chunk issued one step ago: wait for it, test it, release it to the consumers
            const unsigned gp = g - 1u;
            const int sp = (int)(gp % kTileStages);
            ok = mbar_wait_or_abort(&sm.full[sp], (gp / kTileStages) & 1u, abort);
            if (!ok) {
                g = issue ? g + 1u : g;
                break;
            }
            const bool bad = tile_chunk_nonfinite(sm, sp, prev_cols, lane);
            if (lane == 0) {
                sm.nonfinite[sp] = bad ? 1 : 0;
                mbar_arrive(&sm.ready[sp]);  // release: the flag is visible to whoever sees the phase complete
            }
            __syncwarp();
        }
        if (!issue) break;  // that was the test of the last chunk
        prev_cols = cols_now;
        g++;
        if (++c == tc.nchunks) {
            c = 0;
            tc.tile += gridDim.x;
            have = tile_cursor_load(tc, problems, tile_start, count, total, p);
        }
    }
    if (!ok) {
        *abort = 1;
        // copies that were issued but not seen to land: at most the last two chunks
        for (unsigned back = 1; back <= 2u && back <= g; back++) {
            const unsigned gq = g - back;
            (void)mbar_wait(&sm.full[gq % kTileStages], (gq / kTileStages) & 1u);
        }
    }
    return ok;
}

// ---- consumer warps -------------------------------------------------------------------------------

// Two multiply-adds per instruction (fma.rn.f32x2, new with sm_100): the fp32 pipe does the same
// number of them per cycle, but they take half the issue slots, which leaves room for the shared-
// memory loads and the CSR expansion beside a busy FMA pipe.  Each half rounds exactly like fmaf
// (the strict form keeps scalar multiplies and adds), so results do not change.
template <bool STRICT>
__device__ __forceinline__ float2 tmad2(float2 a, float2 b, float2 c)
{
    // strict: scalar multiply and add with their own roundings (the packed __fmul2_rn / __fadd2_rn
    // pair was seen to be contracted into one packed FMA by the compiler)
    if constexpr (STRICT) return make_float2(__fadd_rn(c.x, __fmul_rn(a.x, b.x)), __fadd_rn(c.y, __fmul_rn(a.y, b.y)));
    else return __ffma2_rn(a, b, c);
}

// acc holds the 8 columns of one row as 4 pairs: columns (0,1) (2,3) of b0, then of b1.
template <bool STRICT>
__device__ __forceinline__ void row_update(float2 (&acc)[4], float av, const float4 &b0, const float4 &b1)
{
    const float2 a2 = make_float2(av, av);
    acc[0] = tmad2<STRICT>(a2, make_float2(b0.x, b0.y), acc[0]);
    acc[1] = tmad2<STRICT>(a2, make_float2(b0.z, b0.w), acc[1]);
    acc[2] = tmad2<STRICT>(a2, make_float2(b1.x, b1.y), acc[2]);
    acc[3] = tmad2<STRICT>(a2, make_float2(b1.z, b1.w), acc[3]);
}

// Row state of a consumer warp: lane r (< 8) holds the state of the warp's row r.
struct TileRows {
    int row;     // row of C (-1: the tile has no such row)
    int cursor;  // next unconsumed entry
    int end;     // end of the row in the CSR arrays
};

__device__ __forceinline__ void tile_rows_setup(TileRows &rs, const TileProblem *__restrict__ pp, int rb, int warp, int lane)
{
    rs.row = -1;
    rs.cursor = 0;
    rs.end = 0;
    if (lane < kTileRowsPerWarp) {
        const int slot = rb * kTileM + warp * kTileRowsPerWarp + lane;
        if (slot < pp->M) {
            const int *order = pp->row_order;
            const int *offsets = pp->row_offsets;
            rs.row = order ? __ldg(order + slot) : slot;
            rs.cursor = __ldg(offsets + rs.row);
            rs.end = __ldg(offsets + rs.row + 1);
        }
    }
}

// Starts the asynchronous fetch of the next <= 32 entries of this warp's rows; slots past the end of
// a row get a column that no chunk contains.
__device__ __forceinline__ void tile_fetch_candidates(TileSmem &sm, const TileProblem *__restrict__ pp, const TileRows &rs,
                                                      int warp, int lane)
{
    // the two array bases are re-read from the problem table (an L1 hit) rather than kept in
    // registers through the multiply loop
    const int *cols = pp->cols;
    const float *values = pp->values;
#pragma unroll
    for (int r = 0; r < kTileRowsPerWarp; r++) {
        const int q = __shfl_sync(0xffffffffu, rs.cursor, r) + lane;
        const int e = __shfl_sync(0xffffffffu, rs.end, r);
        if (q < e) {
            cp_async_4(&sm.cand_col[warp][r][lane], cols + q);
            cp_async_4(&sm.cand_val[warp][r][lane], values + q);
        } else {
            sm.cand_col[warp][r][lane] = 0x7fffffff;
        }
    }
}

// Turns the fetched entries that fall into columns [k0, k0 + 32) into the zero-filled block
// As[warp][buf][column][row] and the presence masks, and moves the rows' cursors past them.  Columns
// ascend, so the entries of the chunk are a prefix of the fetched ones, in column order: lane c
// finds the value of column c at position popc(mask below c).
__device__ __forceinline__ void tile_expand_a(TileSmem &sm, TileRows &rs, int buf, int k0, int warp, int lane)
{
    cp_async_wait_all();
    __syncwarp();
    float v[kTileRowsPerWarp];
    unsigned my_mask = 0u, my_count = 0u;
#pragma unroll
    for (int r = 0; r < kTileRowsPerWarp; r++) {
        const int c = sm.cand_col[warp][r][lane] - k0;
        const float val = sm.cand_val[warp][r][lane];
        const bool take = (unsigned)c < (unsigned)kTileK;
        const unsigned mask = __reduce_or_sync(0xffffffffu, take ? (1u << c) : 0u);
        const float x = __shfl_sync(0xffffffffu, val, __popc(mask & ((1u << lane) - 1u)));
        v[r] = ((mask >> lane) & 1u) ? x : 0.f;
        if (lane == r) {
            my_mask = mask;
            my_count = (unsigned)__popc(mask);
        }
    }
    float4 *dst = reinterpret_cast<float4 *>(&sm.As[warp][buf][lane][0]);
    dst[0] = make_float4(v[0], v[1], v[2], v[3]);
    dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    if (lane < kTileRowsPerWarp) {
        sm.Am[warp][buf][lane] = my_mask;
        rs.cursor += (int)my_count;
    }
    __syncwarp();
}

// One chunk with every entry of the 8 x 32 block multiplied (absent ones are zeros).
template <bool STRICT>
__device__ __forceinline__ void tile_chunk_dense(const TileSmem &sm, int s, int warp, int buf, int lane,
                                                 float2 (&acc)[kTileRowsPerWarp][4])
{
    const float *bs = &sm.Bs[s][0][lane * 4];
    const float *as = &sm.As[warp][buf][0][0];
#pragma unroll(kTileUnroll)
    for (int k = 0; k < kTileK; k++) {
        const float4 a0 = *reinterpret_cast<const float4 *>(as + k * kTileRowsPerWarp);
        const float4 a1 = *reinterpret_cast<const float4 *>(as + k * kTileRowsPerWarp + 4);
        const float4 b0 = *reinterpret_cast<const float4 *>(bs + k * kTileN);
        const float4 b1 = *reinterpret_cast<const float4 *>(bs + k * kTileN + 128);
        row_update<STRICT>(acc[0], a0.x, b0, b1);
        row_update<STRICT>(acc[1], a0.y, b0, b1);
        row_update<STRICT>(acc[2], a0.z, b0, b1);
        row_update<STRICT>(acc[3], a0.w, b0, b1);
        row_update<STRICT>(acc[4], a1.x, b0, b1);
        row_update<STRICT>(acc[5], a1.y, b0, b1);
        row_update<STRICT>(acc[6], a1.z, b0, b1);
        row_update<STRICT>(acc[7], a1.w, b0, b1);
    }
}

// One chunk with present entries only (used for chunks of B that hold a non-finite value, and for
// every chunk when the masked form is asked for).
template <bool STRICT>
__device__ __forceinline__ void tile_chunk_masked(const TileSmem &sm, int s, int warp, int buf, int lane,
                                                  float2 (&acc)[kTileRowsPerWarp][4])
{
    const float *bs = &sm.Bs[s][0][lane * 4];
    const float *as = &sm.As[warp][buf][0][0];
    unsigned m[kTileRowsPerWarp];
    unsigned any = 0u;
#pragma unroll
    for (int i = 0; i < kTileRowsPerWarp; i++) {
        m[i] = sm.Am[warp][buf][i];
        any |= m[i];
    }
#pragma unroll 1
    for (int k = 0; k < kTileK; k++) {
        if (!((any >> k) & 1u)) continue;  // none of this warp's rows uses the column
        const float4 a0 = *reinterpret_cast<const float4 *>(as + k * kTileRowsPerWarp);
        const float4 a1 = *reinterpret_cast<const float4 *>(as + k * kTileRowsPerWarp + 4);
        const float4 b0 = *reinterpret_cast<const float4 *>(bs + k * kTileN);
        const float4 b1 = *reinterpret_cast<const float4 *>(bs + k * kTileN + 128);
        if ((m[0] >> k) & 1u) row_update<STRICT>(acc[0], a0.x, b0, b1);
        if ((m[1] >> k) & 1u) row_update<STRICT>(acc[1], a0.y, b0, b1);
        if ((m[2] >> k) & 1u) row_update<STRICT>(acc[2], a0.z, b0, b1);
        if ((m[3] >> k) & 1u) row_update<STRICT>(acc[3], a0.w, b0, b1);
        if ((m[4] >> k) & 1u) row_update<STRICT>(acc[4], a1.x, b0, b1);
        if ((m[5] >> k) & 1u) row_update<STRICT>(acc[5], a1.y, b0, b1);
        if ((m[6] >> k) & 1u) row_update<STRICT>(acc[6], a1.z, b0, b1);
        if ((m[7] >> k) & 1u) row_update<STRICT>(acc[7], a1.w, b0, b1);
    }
}

// The consumers' view of a tile: where it is, without a copy of the problem record.
__device__ __forceinline__ bool tile_cursor_locate(TileCursor &tc, const TileProblem *__restrict__ problems,
                                                   const long long *__restrict__ tile_start, int count, long long total)
{
    if (tc.tile >= total) return false;
    int lo = tc.prob, hi = count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(tile_start + mid) <= tc.tile) lo = mid;
        else hi = mid - 1;
    }
    tc.prob = lo;
    const int t = (int)(tc.tile - __ldg(tile_start + lo));
    const int row_blocks = problems[lo].row_blocks;
    const int cb = t / row_blocks;
    tc.rb = t - cb * row_blocks;
    tc.n0 = cb * kTileN;
    tc.nchunks = (problems[lo].K + kTileK - 1) / kTileK;
    return true;
}

template <bool STRICT>
__device__ __forceinline__ bool tile_consumer(TileSmem &sm, const TileProblem *__restrict__ problems,
                                              const long long *__restrict__ tile_start, int count, long long total,
                                              bool force_masked, int warp, int lane)
{
    volatile int *abort = &sm.abort;
    TileCursor tc{(long long)blockIdx.x, 0, 0, 0, 0};
    unsigned g = 0;  // chunks consumed so far (the same numbering as the producer's)
    while (tile_cursor_locate(tc, problems, tile_start, count, total)) {
        const TileProblem *pp = problems + tc.prob;
        TileRows rs;
        tile_rows_setup(rs, pp, tc.rb, warp, lane);
        // a warp whose 8 row slots all lie past the last row only keeps the barriers moving
        const bool idle = tc.rb * kTileM + warp * kTileRowsPerWarp >= pp->M;
        float2 acc[kTileRowsPerWarp][4];
#pragma unroll
        for (int i = 0; i < kTileRowsPerWarp; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = make_float2(0.f, 0.f);
        if (!idle) {
            tile_fetch_candidates(sm, pp, rs, warp, lane);
            tile_expand_a(sm, rs, (int)(g & 1u), 0, warp, lane);
        }
        for (int c = 0; c < tc.nchunks; c++, g++) {
            const int s = (int)(g % kTileStages);
            const int buf = (int)(g & 1u);
            const bool more = c + 1 < tc.nchunks;
            if (more && !idle) tile_fetch_candidates(sm, pp, rs, warp, lane);  // lands while this chunk is computed
            if (!mbar_wait_or_abort(&sm.ready[s], (g / kTileStages) & 1u, abort)) return false;
            if (!idle) {
                if (force_masked || sm.nonfinite[s]) tile_chunk_masked<STRICT>(sm, s, warp, buf, lane, acc);
                else tile_chunk_dense<STRICT>(sm, s, warp, buf, lane, acc);
                if (more) tile_expand_a(sm, rs, buf ^ 1, (c + 1) * kTileK, warp, lane);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[s]);  // this warp is done with the stage
        }
        if (!idle) {
            float *cbase = pp->C;
            const int ncols = pp->N;
#pragma unroll
            for (int i = 0; i < kTileRowsPerWarp; i++) {
                const int row = __shfl_sync(0xffffffffu, rs.row, i);
                if (row >= 0) {
                    float *crow = cbase + (size_t)row * (size_t)ncols + tc.n0;
                    if (tc.n0 + lane * 4 < ncols)
                        *reinterpret_cast<float4 *>(crow + lane * 4) = make_float4(acc[i][0].x, acc[i][0].y, acc[i][1].x, acc[i][1].y);
                    if (tc.n0 + 128 + lane * 4 < ncols)
                        *reinterpret_cast<float4 *>(crow + 128 + lane * 4) = make_float4(acc[i][2].x, acc[i][2].y, acc[i][3].x, acc[i][3].y);
                }
            }
        }
        tc.tile += gridDim.x;
    }
    return true;
}

// One thread block per SM; block b takes the tiles b, b + gridDim.x, ... (tile_start[i] is the first
// tile of problem i; tiles of a problem are numbered column block by column block, so blocks that
// run side by side read the same columns of B).  A tile costs ceil(K / 32) equal steps whatever its
// pattern, and the problems are stored from the most to the least work, so this fixed deal is
// balanced to within one tile.  On an mbarrier timeout error[0] is set to 1.
template <bool STRICT>
__global__ void __launch_bounds__(kTileThreads, 1)
spmm_tile_kernel(const TileProblem *__restrict__ problems, const long long *__restrict__ tile_start, int count,
                 int force_masked, int *error)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    TileSmem &sm = *reinterpret_cast<TileSmem *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kTileStages; s++) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.ready[s], 1);
            mbar_init(&sm.empty[s], kTileConsumers);
            sm.nonfinite[s] = 0;
        }
        sm.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long total = tile_start[count];
    // Registers move from the producer's group of four warps to the consumers (see kTileRegsLaunch): the producer's loop needs few, the consumers hold 64 accumulators each.
    bool ok = true;
    if (warp >= kTileConsumers) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTileRegsProducer));
        // the producer and the three spare warps of its group, which leave at once
        if (warp == kTileConsumers) ok = tile_producer(sm, problems, tile_start, count, total, lane);
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTileRegsConsumer));
        ok = tile_consumer<STRICT>(sm, problems, tile_start, count, total, force_masked != 0, warp, lane);
    }
    if (!ok) {
        *(volatile int *)&sm.abort = 1;
        if (lane == 0) atomicExch(error, 1);
    }
}

}  // namespace dlspm
