// Device-side building blocks shared by the SDDMM and the fused SDDMM->SpMM kernels.
//
// Lane layout of the fast path (rows of N = 4*chunks floats, 16-byte aligned): the warp is cut
// into 32/G groups of G lanes.  Lane t of a group owns the float4 chunks r*G + t (r = 0..R-1) of a
// dense row, so a group reads G*16 contiguous bytes of a row per load (from G = 8 on at least one
// full 128-byte line; rows of up to 32 floats use G = 4, see the launchers).  One pass handles 32
// nonzeros, G per group, and every lane keeps G partial dot products.  In sddmm_pass (used where
// warps share the nonzeros inside a pass) group g takes the nonzeros g*G .. g*G+G-1; in
// sddmm_pass_dealt (everywhere else) the nonzeros are dealt to the groups in turn.  A transposing
// butterfly then leaves one finished dot product on every lane: G-1 shuffles per lane for G results,
// instead of log2(G) shuffles per result.
#pragma once
#include <cuda_runtime.h>

namespace dlspm {

__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc)
{
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// v[0..G-1] per lane -> v[0] on lane t (within its group of G lanes) = sum over the group's
// lanes of v[t].
template <int G>
__device__ __forceinline__ void group_transpose_reduce(float (&v)[G], int t)
{
#pragma unroll
    for (int s = G / 2; s >= 1; s >>= 1) {
        const bool upper = (t & s) != 0;
#pragma unroll
        for (int k = 0; k < s; k++) {
            const float send = upper ? v[k] : v[k + s];
            const float keep = upper ? v[k + s] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
}

// Loads the R chunks of row `row4` (a float4 pointer to the start of the row) owned by lane t.
template <int G, int R>
__device__ __forceinline__ void load_row_chunks(const float4 *__restrict__ row4, int chunks, int t,
                                                float4 (&a)[R])
{
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int idx = r * G + t;
        a[r] = idx < chunks ? __ldg(row4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// 32 bytes in one load (sm_100 has 256-bit global loads).  `p` must be 32-byte aligned.
__device__ __forceinline__ void ldg256(const float4 *__restrict__ p, float4 &lo, float4 &hi)
{
    asm("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(lo.x), "=f"(lo.y), "=f"(lo.z), "=f"(lo.w), "=f"(hi.x), "=f"(hi.y), "=f"(hi.z), "=f"(hi.w)
                 : "l"(p));
}

// Rows of exactly 32 floats (eight chunks) whose operands are 32-byte aligned, groups of four lanes:
// lane t owns the chunks 2t and 2t+1, i.e. 32 consecutive bytes, and fetches them with ONE 256-bit
// load, so a group reads a whole 128-byte row per load instruction.  With 16-byte loads (chunks t and
// 4+t) a warp-wide load touches eight rows but uses only half of each 128-byte line, twice the L1
// wavefronts per nonzero: the N = 32 launches sat at 88 % of the L1 data pipe.  Same dealing of the
// nonzeros and same result placement as sddmm_pass_dealt<4, 2>; the lanes' partial sums cover other
// elements, so the bits can differ from the 16-byte form in the last place.
__device__ __forceinline__ void load_row_pair(const float4 *__restrict__ row4, int t, float4 (&a)[2])
{
    a[0] = __ldg(row4 + 2 * t);
    a[1] = __ldg(row4 + 2 * t + 1);
}

__device__ __forceinline__ float sddmm_pass_dealt_wide(const float4 (&a)[2], const float4 *__restrict__ rhs4,
                                                       int col, int g, int t)
{
    constexpr int G = 4, NG = 8, kChunks = 8;
    float part[G];
#pragma unroll
    for (int k = 0; k < G; k++) {
        const int c = __shfl_sync(0xffffffffu, col, k * NG + g);
        float acc = 0.f;
        if (c >= 0) {
            float4 lo, hi;
            ldg256(rhs4 + (size_t)c * kChunks + 2 * t, lo, hi);
            acc = dot4(a[0], lo, acc);
            acc = dot4(a[1], hi, acc);
        }
        part[k] = acc;
    }
    group_transpose_reduce<G>(part, t);
    return part[0];
}

// One pass of sampled dot products: col = this lane's column index of nonzero base+lane (or -1
// past the end of the row).  On return part0 on lane g*G+t is dot(lhs_row, rhs[col of that lane]).
// Adds to part[k] the partial dot product of this lane for the k-th nonzero of its group.  `chunks`
// is the number of float4 of the row (or row segment) that take part, `stride4` the row stride of
// rhs in float4 (they differ when a long row is processed in segments).
// With kmask != 0 only the nonzeros whose index k within the group has (k & kmask) == ksub are
// computed: several warps then share one pass, each taking every (kmask+1)-th nonzero, and the
// results of the others stay zero on this warp.
// (KSPLIT is a template parameter: with the test compiled into the common path the compiler batches
// fewer loads and large patterns ran 30 to 40 % slower.)
template <int G, int R, bool KSPLIT = false>
__device__ __forceinline__ void sddmm_accumulate(float (&part)[G], const float4 (&a)[R],
                                                 const float4 *__restrict__ rhs4, int chunks, int stride4,
                                                 int col, int g, int t, int kmask = 0, int ksub = 0)
{
#pragma unroll
    for (int k = 0; k < G; k++) {
        const int c = __shfl_sync(0xffffffffu, col, g * G + k);
        float acc = part[k];
        bool take = c >= 0;
        if constexpr (KSPLIT) take = take && (k & kmask) == ksub;
        if (take) {
            const float4 *brow = rhs4 + (size_t)c * (size_t)stride4;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int idx = r * G + t;
                if (idx < chunks) acc = dot4(a[r], __ldg(brow + idx), acc);
            }
        }
        part[k] = acc;
    }
}

template <int G, int R, bool KSPLIT = false>
__device__ __forceinline__ float sddmm_pass(const float4 (&a)[R], const float4 *__restrict__ rhs4,
                                            int chunks, int col, int g, int t, int kmask = 0, int ksub = 0)
{
    float part[G];
#pragma unroll
    for (int k = 0; k < G; k++) part[k] = 0.f;
    sddmm_accumulate<G, R, KSPLIT>(part, a, rhs4, chunks, chunks, col, g, t, kmask, ksub);
    group_transpose_reduce<G>(part, t);
    return part[0];
}

// The same pass with the nonzeros DEALT to the groups in turn: nonzero i of the pass (its column on
// lane i, -1 past the end of the row) goes to group i % (32/G) as that group's (i / (32/G))-th.  In a
// pass with few nonzeros (the last pass of every row, the only pass of a short row) every group then
// has work in the first ceil(cnt / (32/G)) steps only and the remaining steps are skipped by all
// lanes, where with blocks of G the first group worked through min(cnt, G) nonzeros alone.
// Returns, on lane g*G + t, the dot product of nonzero sddmm_dealt_slot(G, g, t) of the pass.  Every
// dot product is summed in the same order as in sddmm_pass, so the two give the same bits.
template <int G, int R>
__device__ __forceinline__ float sddmm_pass_dealt(const float4 (&a)[R], const float4 *__restrict__ rhs4,
                                                  int chunks, int col, int g, int t)
{
    constexpr int NG = 32 / G;
    float part[G];
#pragma unroll
    for (int k = 0; k < G; k++) {
        const int c = __shfl_sync(0xffffffffu, col, k * NG + g);
        float acc = 0.f;
        if (c >= 0) {
            const float4 *brow = rhs4 + (size_t)c * (size_t)chunks;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int idx = r * G + t;
                if (idx < chunks) acc = dot4(a[r], __ldg(brow + idx), acc);
            }
        }
        part[k] = acc;
    }
    group_transpose_reduce<G>(part, t);
    return part[0];
}

__device__ __forceinline__ int sddmm_dealt_slot(int G, int g, int t) { return t * (32 / G) + g; }

// Group width and chunks per lane for a row of `chunks` float4: G*R >= chunks with G >= 8 (the
// launchers take G = 4 for rows of up to 32 floats by themselves).
// Returns false when the row is too long for the register-resident path.
__host__ __device__ inline bool sddmm_layout(int chunks, int *G, int *R)
{
    if (chunks <= 32) { *G = 8; }        // N <= 128
    else if (chunks <= 64) { *G = 16; }  // N <= 256
    else if (chunks <= 256) { *G = 32; } // N <= 1024
    else return false;
    const int need = (chunks + *G - 1) / *G;
    *R = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    return true;
}

}  // namespace dlspm
