// Device-side building block of the row-gather SpMM: one warp computes one row of C for one
// slab of 32*VEC*U consecutive columns.
//
// Work layout: lane l owns the columns n0 + (u*32 + l)*VEC .. +VEC-1 for u = 0..U-1, so every
// warp-wide load of a B row is one contiguous run of 32*VEC floats (512 bytes for VEC = 4).
// The row's (column, value) pairs are staged 32 at a time in shared memory with one coalesced
// load per array and read back as a broadcast, which costs one shared-memory wavefront per
// nonzero instead of two shuffles.  Each output element accumulates its products in CSR order
// starting from 0.0f, the same order as the reference host loop
// (SPMM/spmm-esimd-fromfile.cpp:63-83), so STRICT = true (separate multiply and add) gives its
// bits exactly.
#pragma once
#include <cuda_runtime.h>

namespace dlspm {

constexpr int kWarpsPerCta = 8;

template <int VEC>
__device__ __forceinline__ void load_vec(const float *__restrict__ p, float (&v)[VEC])
{
    if constexpr (VEC == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if constexpr (VEC == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2 *>(p));
        v[0] = t.x; v[1] = t.y;
    } else {
        v[0] = __ldg(p);
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float *__restrict__ p, const float (&v)[VEC])
{
    if constexpr (VEC == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else if constexpr (VEC == 2) {
        *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]);
    } else {
        p[0] = v[0];
    }
}

// The same store marked as streaming (evicted from L2 first): for output that is written once and
// not read again by the kernel, so that it does not push the rows of B that are still needed out
// of L2.
template <int VEC>
__device__ __forceinline__ void store_vec_streaming(float *__restrict__ p, const float (&v)[VEC])
{
#ifdef DLSPM_NO_STREAMING_STORES
    store_vec<VEC>(p, v);
#else
    if constexpr (VEC == 4) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    } else if constexpr (VEC == 2) {
        __stcs(reinterpret_cast<float2 *>(p), make_float2(v[0], v[1]));
    } else {
        __stcs(p, v[0]);
    }
#endif
}

template <bool STRICT>
__device__ __forceinline__ float mad(float a, float b, float c)
{
    if constexpr (STRICT) return __fadd_rn(c, __fmul_rn(a, b));
    else return fmaf(a, b, c);
}

// Adds the products of `cnt` staged (column, value) pairs to the accumulators of one warp slab, in
// the order of the pairs.  J = 0: the plain loop, unrolled four times.  J > 0: J nonzeros are taken
// at once, all their loads first and their products afterwards (still in pair order), which keeps
// J*U loads in flight per lane; a lone small matrix is bound by exactly that latency chain.
template <int VEC, int U, bool STRICT, int J>
__device__ __forceinline__ void spmm_accumulate_staged(const int2 *stage, int cnt, const float *__restrict__ B,
                                                       int N, const int (&cidx)[U], float (&acc)[U][VEC])
{
    if constexpr (J <= 1) {
#pragma unroll 4
        for (int j = 0; j < cnt; j++) {
            const int2 e = stage[j];
            const float a = __int_as_float(e.y);
            const float *brow = B + (size_t)e.x * (size_t)N;
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (cidx[u] < N) {
                    float b[VEC];
                    load_vec<VEC>(brow + cidx[u], b);
#pragma unroll
                    for (int v = 0; v < VEC; v++) acc[u][v] = mad<STRICT>(a, b[v], acc[u][v]);
                }
            }
        }
    } else {
        for (int j = 0; j < cnt; j += J) {
            float b[J][U][VEC];
            float a[J];
#pragma unroll
            for (int jj = 0; jj < J; jj++) {
                const bool live = j + jj < cnt;
                const int2 e = stage[(j + jj) & 31];
                a[jj] = __int_as_float(e.y);
                const float *brow = B + (size_t)e.x * (size_t)N;
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (live && cidx[u] < N) load_vec<VEC>(brow + cidx[u], b[jj][u]);
                }
            }
#pragma unroll
            for (int jj = 0; jj < J; jj++) {
                if (j + jj < cnt) {
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        if (cidx[u] < N) {
#pragma unroll
                            for (int v = 0; v < VEC; v++) acc[u][v] = mad<STRICT>(a[jj], b[jj][u][v], acc[u][v]);
                        }
                    }
                }
            }
        }
    }
}

// Nonzeros taken at once by a lone launch (0: the plain unrolled loop): 8 loads in flight per lane
// for the one- and two-chunk slabs.  Measured on lone matrices of 256 to 2048 rows: 512 x 512 at
// 10 %, N = 128 went from 7.7 to 5.2 us, 1024 x 1024 at 30 % from 20.5 to 17.5 us; 16 nonzeros at
// once (one-chunk) or 8 (two-chunk) lost again through registers.  The grouped launch keeps the
// plain loop for every width: it holds all three widths in one kernel, its occupancy is what
// hides the latency there, and the batched loads would cost it registers.
template <int U>
constexpr int kLoneBatch = U == 1 ? 8 : U == 2 ? 4 : 0;

// The (column, value) pair of nonzero start + lane of a row, (0, 0) beyond its end: what the first
// staging step of spmm_warp_row_slab loads.  A caller that walks several rows can ask for the next
// row's pairs before it computes the current row and hand them over (PRE = true), which takes that
// load out of the next row's chain of dependent latencies.
__device__ __forceinline__ int2 spmm_first_pairs(const float *__restrict__ values, const int *__restrict__ cols,
                                                 int start, int end, int lane)
{
    const int p = start + lane;
    return p < end ? make_int2(__ldg(cols + p), __float_as_int(__ldg(values + p))) : make_int2(0, 0);
}

// The sums of one row for one slab: acc[u][v] for the columns cidx[u] + v (computed here), products
// added in CSR order from 0.0f.  stage: 32 int2 slots private to this warp.  PRE: `first` holds
// spmm_first_pairs of this row.
template <int VEC, int U, bool STRICT, int J, bool PRE>
__device__ __forceinline__ void spmm_warp_row_sums(const float *__restrict__ values, const int *__restrict__ cols,
                                                   int start, int end, const float *__restrict__ B, int N, int n0,
                                                   int lane, int2 *stage, int2 first, int (&cidx)[U],
                                                   float (&acc)[U][VEC])
{
#pragma unroll
    for (int u = 0; u < U; u++) {
        cidx[u] = n0 + (u * 32 + lane) * VEC;
#pragma unroll
        for (int v = 0; v < VEC; v++) acc[u][v] = 0.0f;
    }
    for (int base = start; base < end; base += 32) {
        const int p = base + lane;
        int2 cv = make_int2(0, 0);
        if (PRE && base == start) cv = first;
        else if (p < end) cv = make_int2(__ldg(cols + p), __float_as_int(__ldg(values + p)));
        stage[lane] = cv;
        __syncwarp();
        spmm_accumulate_staged<VEC, U, STRICT, J>(stage, min(32, end - base), B, N, cidx, acc);
        __syncwarp();
    }
}

// One row of C for one slab, written to Crow.  stage: 32 int2 slots private to this warp.  PRE: `first`
// holds spmm_first_pairs of this row.
template <int VEC, int U, bool STRICT, int J = 0, bool PRE = false>
__device__ __forceinline__ void spmm_warp_row_slab(const float *__restrict__ values,
                                                   const int *__restrict__ cols, int start, int end,
                                                   const float *__restrict__ B, float *__restrict__ Crow,
                                                   int N, int n0, int lane, int2 *stage,
                                                   int2 first = make_int2(0, 0))
{
    float acc[U][VEC];
    int cidx[U];
    spmm_warp_row_sums<VEC, U, STRICT, J, PRE>(values, cols, start, end, B, N, n0, lane, stage, first, cidx, acc);
#pragma unroll
    for (int u = 0; u < U; u++) {
        if (cidx[u] < N) store_vec_streaming<VEC>(Crow + cidx[u], acc[u]);
    }
}

// Column chunks (of 32*vec columns) per warp slab: 1, 2 or 4.  Wider slabs amortise the staging of a
// row's indices over more B traffic; beyond 4 chunks the accumulators push the kernel past 64
// registers and the lost occupancy costs far more than the staging saves (measured: 8 chunks ran
// 30 % slower).  A partly filled last slab costs little: its idle chunks issue no loads, and the
// kernel is bound by L1 traffic, not by issue slots.  (Narrowing the slabs of a lone small matrix
// to get more warps was tried and lost: 512 x 2048, N = 3136 went from 119 to 153 us.)
__host__ __device__ inline int spmm_slab_chunks(int N, int vec)
{
    const int total = (N + 32 * vec - 1) / (32 * vec);
    return total > 4 ? 4 : total > 1 ? 2 : 1;
}

}  // namespace dlspm
