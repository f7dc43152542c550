// adamw_math.cuh: what the pass-2 kernels share: the per-element update, the tensor table
// in shared memory and the cursor that turns a position into a decay flag.
#pragma once

#include <climits>

#include "internal.cuh"

namespace b200amp
{

// One element, the arithmetic of the reference (cuda/kernels/adamw_multi.cu:20-29): decay the
// parameter, m += (1-b1)(g-m), v = v*b2 + ((1-b2)*g)*g, denom = sqrt(v)/bc2_sqrt + eps,
// p = decayed - step_size*(m/denom). The reference builds with nvcc's defaults (fused
// multiply-add contraction on; IEEE sqrt and division, no fast-math: Makefile:44-46). The
// fusions nvcc 12.9 picks for those expressions are written out here with intrinsics, so every
// kernel that inlines this function rounds identically whatever code surrounds it: the single
// fusion of m + w1*(g-m); in v, the product (w2*g)*g fused and v*b2 rounded; in p, the product
// step_size*(m/denom) fused and p*decay rounded. The GPU tests hold this to the bits of the
// reference's own kernels compiled from its sources.
__device__ __forceinline__ void adamw_element(float &p, float &m, float &v, float g, float w1, float w2, float b2,
                                              float eps, float decay, float step_size, float bc2_sqrt)
{
    const float decayed = __fmul_rn(p, decay);
    m = __fmaf_rn(w1, __fsub_rn(g, m), m);
    v = __fmaf_rn(__fmul_rn(w2, g), g, __fmul_rn(v, b2));
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), bc2_sqrt), eps);
    p = __fmaf_rn(-step_size, __fdiv_rn(m, denom), decayed);
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
    float factor;       // what a parameter of tensor k is multiplied by: the step's decay, or 1
};

__device__ __forceinline__ long long table_next(const TensorTable &tab, int ntensors, int k)
{
    return k + 1 < ntensors ? tab.first[k + 1] : LLONG_MAX;
}

__device__ __forceinline__ Cursor cursor_seek(const TensorTable &tab, int ntensors, long long at, float wd_decay)
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
    c.factor = tab.decay[lo] ? wd_decay : 1.0f;
    return c;
}

// Positions only grow. Nothing to do (one compare, no shared-memory access) while the
// position stays inside tensor k, which is the case for all but a few hundred trips.
__device__ __forceinline__ void cursor_advance(Cursor &c, const TensorTable &tab, int ntensors, long long at,
                                               float wd_decay)
{
    if (at >= c.next)
    {
        do
        {
            c.k += 1;
            c.next = table_next(tab, ntensors, c.k);
        } while (at >= c.next);
        c.factor = tab.decay[c.k] ? wd_decay : 1.0f;
    }
}

// Decay factors of the two quads of the 8-element group that starts at `at`. Tensor
// offsets are multiples of 4, so a quad never straddles two tensors but a group can.
// The usual case, the whole group inside the cursor's tensor, costs one compare.
__device__ __forceinline__ void group_decay(Cursor &c, const TensorTable &tab, int ntensors, long long at,
                                            float wd_decay, float &lo, float &hi)
{
    if (at + 8 <= c.next)
    {
        lo = c.factor;
        hi = c.factor;
        return;
    }
    cursor_advance(c, tab, ntensors, at, wd_decay);
    lo = c.factor;
    hi = c.factor;
    if (at + 4 >= c.next)
    {
        Cursor c2 = c;
        cursor_advance(c2, tab, ntensors, at + 4, wd_decay);
        hi = c2.factor;
    }
}

} // namespace b200amp
