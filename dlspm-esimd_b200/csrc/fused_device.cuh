// Device-side building block of the fused SDDMM -> SpMM kernels (single-matrix and grouped
// launches): the passes of one row.  Scores are formed as in the SDDMM kernel (sddmm_device.cuh) and
// consumed at once by the lane groups that gather the D rows of their own nonzeros; the reference
// keeps a 32-score vector per row in registers in the same way (FUSED/fused-esimd_cb.cpp:130-154).
#pragma once
#include <cuda_runtime.h>
#include <math.h>

#include "sddmm_device.cuh"

namespace dlspm {

constexpr int kPlain = 0, kScaled = 1, kSoftmax = 2;

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

// The passes base, base + stride, ... of one row: scores as in the SDDMM kernel, then the update of
// the lane's partial output row.  On return acc holds this lane group's partial sums (relative to
// run_max in softmax mode).
template <int G, int R, int MODE, bool WIDE = false>
__device__ __forceinline__ void fused_row_passes(const int *__restrict__ cols, const float4 (&q)[R],
                                                 const float4 *__restrict__ b4, const float4 *__restrict__ d4,
                                                 int chunks, int start, int end, int stride, float scale, int lane,
                                                 float4 (&acc)[R], float &run_max, float &run_sum)
{
    const int g = lane / G, t = lane % G;
    // column indices of the next pass are fetched one pass ahead
    int col_next = start + lane < end ? __ldg(cols + start + lane) : -1;
    for (int base = start; base < end; base += stride) {
        const int p = base + lane;
        const int col = col_next;
        col_next = p + stride < end ? __ldg(cols + p + stride) : -1;
        // nonzeros dealt to the lane groups in turn (see sddmm_pass_dealt): this lane's score belongs
        // to nonzero base + sddmm_dealt_slot of the row, whose column sits on lane sddmm_dealt_slot
        float score;
        if constexpr (WIDE) score = sddmm_pass_dealt_wide(q, b4, col, g, t);  // G = 4, R = 2, rows of 32 floats
        else score = sddmm_pass_dealt<G, R>(q, b4, chunks, col, g, t);
        if constexpr (MODE == kScaled) score *= scale;
        if constexpr (MODE == kSoftmax) {
            // streaming softmax: weights relative to the running maximum; the partial row and the
            // running sum are rescaled when the maximum grows
            const bool stored = base + sddmm_dealt_slot(G, g, t) < end;
            const float x = stored ? score * scale : -INFINITY;
            const float m_new = fmaxf(run_max, warp_max(x));  // finite: a pass has a stored entry
            const float corr = expf(run_max - m_new);         // 0 on the first pass
            score = stored ? expf(x - m_new) : 0.f;
            run_sum = run_sum * corr + warp_sum(score);
            run_max = m_new;
#pragma unroll
            for (int r = 0; r < R; r++) {
                acc[r].x *= corr;
                acc[r].y *= corr;
                acc[r].z *= corr;
                acc[r].w *= corr;
            }
        }
#pragma unroll
        for (int k = 0; k < G; k++) {
            const int cc = __shfl_sync(0xffffffffu, col, k * (32 / G) + g);  // the group's k-th nonzero
            const float s = __shfl_sync(0xffffffffu, score, g * G + k);
            if constexpr (WIDE) {
                // lane t owns the chunks 2t and 2t + 1 of the row: one 256-bit load (see sddmm_pass_dealt_wide)
                if (cc >= 0) {
                    float4 lo, hi;
                    ldg256(d4 + (size_t)cc * 8 + 2 * t, lo, hi);
                    acc[0].x = fmaf(s, lo.x, acc[0].x);
                    acc[0].y = fmaf(s, lo.y, acc[0].y);
                    acc[0].z = fmaf(s, lo.z, acc[0].z);
                    acc[0].w = fmaf(s, lo.w, acc[0].w);
                    acc[R - 1].x = fmaf(s, hi.x, acc[R - 1].x);
                    acc[R - 1].y = fmaf(s, hi.y, acc[R - 1].y);
                    acc[R - 1].z = fmaf(s, hi.z, acc[R - 1].z);
                    acc[R - 1].w = fmaf(s, hi.w, acc[R - 1].w);
                }
            } else if (cc >= 0) {
                const float4 *drow = d4 + (size_t)cc * (size_t)chunks;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int idx = r * G + t;
                    if (idx < chunks) {
                        const float4 v = __ldg(drow + idx);
                        acc[r].x = fmaf(s, v.x, acc[r].x);
                        acc[r].y = fmaf(s, v.y, acc[r].y);
                        acc[r].z = fmaf(s, v.z, acc[r].z);
                        acc[r].w = fmaf(s, v.w, acc[r].w);
                    }
                }
            }
        }
    }
    // add the partial rows of the 32/G groups: afterwards every lane holds the sums of its chunks
#pragma unroll
    for (int s = G; s < 32; s <<= 1) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            acc[r].x += __shfl_xor_sync(0xffffffffu, acc[r].x, s);
            acc[r].y += __shfl_xor_sync(0xffffffffu, acc[r].y, s);
            acc[r].z += __shfl_xor_sync(0xffffffffu, acc[r].z, s);
            acc[r].w += __shfl_xor_sync(0xffffffffu, acc[r].w, s);
        }
    }
}

}  // namespace dlspm
