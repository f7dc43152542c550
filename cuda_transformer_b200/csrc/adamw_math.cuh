// adamw_math.cuh: what the pass-2 kernels share: the per-element update, the tensor table
// in shared memory and the cursor that turns a position into a decay flag.
#pragma once

#include <climits>

#include "internal.cuh"

namespace b200amp
{

// One element, the arithmetic of the reference (cuda/kernels/adamw_multi.cu:20-29): decay the
// parameter, m += (1-b1)(g-m), v = v*b2 + ((1-b2)*g)*g, denom = sqrt(v)/bc2_sqrt + eps,
// p = decayed - step_size*(m/denom). Written as plain expressions and built with nvcc's
// defaults (fused multiply-add contraction on, IEEE sqrt and division: no fast-math, as the
// reference's Makefile:44-46), so the compiler rounds them the way it rounds the reference's.
__device__ __forceinline__ void adamw_element(float &p, float &m, float &v, float g, float w1, float w2, float b2,
                                              float eps, float decay, float step_size, float bc2_sqrt)
{
    const float decayed = p * decay;
    m = m + w1 * (g - m);
    v = v * b2 + w2 * g * g;
    const float denom = sqrtf(v) / bc2_sqrt + eps;
    p = decayed - step_size * (m / denom);
}

// Tensor table in shared memory + the cursor over it.
struct TensorTable
{
    long long first[B200AMP_MAX_TENSORS];
    unsigned char decay[B200AMP_MAX_TENSORS];
};

__device__ __forceinline__ void table_load(TensorTable &tab, const b200amp_tensor_info *tensors, int ntensors)
{
    for (int k = threadIdx.x; k < ntensors; k += blockDim.x)
    {
        tab.first[k] = tensors[k].offset;
        tab.decay[k] = tensors[k].decay ? 1 : 0;
    }
    __syncthreads();
}

struct Cursor
{
    int k;              // the last tensor whose first element is <= the position (0 if none is)
    long long next;     // first element of tensor k + 1, LLONG_MAX past the end
};

__device__ __forceinline__ long long table_next(const TensorTable &tab, int ntensors, int k)
{
    return k + 1 < ntensors ? tab.first[k + 1] : LLONG_MAX;
}

__device__ __forceinline__ Cursor cursor_seek(const TensorTable &tab, int ntensors, long long at)
{
    int lo = 0, hi = ntensors - 1;
    while (lo < hi)
    {
        const int mid = (lo + hi + 1) >> 1;
        if (tab.first[mid] <= at)
        {
            lo = mid;
        }
        else
        {
            hi = mid - 1;
        }
    }
    Cursor c;
    c.k = lo;
    c.next = table_next(tab, ntensors, lo);
    return c;
}

__device__ __forceinline__ void cursor_advance(Cursor &c, const TensorTable &tab, int ntensors, long long at)
{
    while (at >= c.next)
    {
        c.k += 1;
        c.next = table_next(tab, ntensors, c.k);
    }
}

// Decay factors of the two quads of the 8-element group that starts at `at`. Tensor
// offsets are multiples of 4, so a quad never straddles two tensors but a group can.
__device__ __forceinline__ void group_decay(Cursor &c, const TensorTable &tab, int ntensors, long long at,
                                            float wd_decay, float &lo, float &hi)
{
    cursor_advance(c, tab, ntensors, at);
    lo = tab.decay[c.k] ? wd_decay : 1.0f;
    hi = lo;
    if (at + 4 >= c.next)
    {
        Cursor c2 = c;
        cursor_advance(c2, tab, ntensors, at + 4);
        hi = tab.decay[c2.k] ? wd_decay : 1.0f;
    }
}

} // namespace b200amp
