// pass1_common.cuh: what every kernel that computes the gradient norm shares: the fixed
// virtual partition of a range, the workspace layout, and the accumulation of 8 fp16 values.
#pragma once

#include "internal.cuh"

namespace b200amp
{

constexpr int P1_THREADS = 256;
constexpr int P1_WARPS = P1_THREADS / 32;
constexpr int P1_UNROLL = 4;                    // independent 16-byte loads (and accumulators) per thread
constexpr int P1_MAX_VBLOCKS = 148 * 32;        // virtual blocks at most: 4736
constexpr long long P1_MIN_VEC_PER_VBLOCK = P1_THREADS * P1_UNROLL;

// Workspace layout. sums comes first so a rank can all-gather its first 16 bytes.
struct Workspace
{
    double sums[2];                 // out: squared norm of the range, flag as 0.0 / 1.0
    unsigned int ticket;            // blocks finished so far; the last one resets it
    int bad;                        // any block saw an inf/NaN; the last one resets it
    unsigned int pad[2];
    double partial[P1_MAX_VBLOCKS]; // one fp64 sum per virtual block
};

// How the arena is cut into virtual blocks: a function of n alone.
struct P1Partition
{
    int vblocks;
    long long vec_per_vblock;       // 16-byte vectors (8 fp16) per virtual block, the last may be short
};

__host__ __device__ inline P1Partition p1_partition(long long n8)
{
    P1Partition p;
    long long per = (n8 + P1_MAX_VBLOCKS - 1) / P1_MAX_VBLOCKS;
    if (per < P1_MIN_VEC_PER_VBLOCK)
    {
        per = P1_MIN_VEC_PER_VBLOCK;
    }
    // whole trips of the unrolled loop, so only the arena's end needs bounds checks
    per = (per + P1_MIN_VEC_PER_VBLOCK - 1) / P1_MIN_VEC_PER_VBLOCK * P1_MIN_VEC_PER_VBLOCK;
    p.vec_per_vblock = per;
    p.vblocks = static_cast<int>((n8 + per - 1) / per);
    return p;
}

// Squares of 8 unscaled gradients added to acc in element order; nonfinite bits or-ed into bad.
__device__ __forceinline__ void accumulate_h8(const uint4 &w, float inv, float &acc, uint32_t &bad)
{
    bad |= half2_nonfinite_bits(w.x) | half2_nonfinite_bits(w.y) | half2_nonfinite_bits(w.z) |
           half2_nonfinite_bits(w.w);
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; k++)
    {
        float2 f = half2_bits_to_float2(words[k]);
        const float a = f.x * inv;              // exact: inv is a power of two
        const float b = f.y * inv;
        acc = fmaf(a, a, acc);
        acc = fmaf(b, b, acc);
    }
}

// The sum of one virtual block: the threads' fp32 sums go to fp64, are added over the warp by
// butterfly and over the block's warps in warp order by thread 0, which stores partial[vb].
// warp_part: shared memory for P1_WARPS doubles. Every thread of the block must call this.
__device__ __forceinline__ void vblock_store_partial(float mine, double *warp_part, Workspace *ws, int vb)
{
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const double total = warp_sum_f64(static_cast<double>(mine));
    if (lane == 0)
    {
        warp_part[warp] = total;
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        double block_total = 0.0;
#pragma unroll
        for (int w = 0; w < P1_WARPS; w++)
        {
            block_total += warp_part[w];
        }
        ws->partial[vb] = block_total;
    }
    __syncthreads();                            // warp_part is reused by the next virtual block
}

// After a CTA's last virtual block: publish its flag, then take a ticket. True (in every
// thread) for the CTA that took the last ticket: all partials are visible to it.
__device__ __forceinline__ bool pass1_take_ticket(uint32_t bad, Workspace *ws, int *last_block)
{
    const int block_bad = __syncthreads_or(bad != 0);
    if (threadIdx.x == 0)
    {
        if (block_bad)
        {
            atomicOr(&ws->bad, 1);
        }
        __threadfence();                        // partials and flag before the ticket
        const unsigned int t = atomicAdd(&ws->ticket, 1u);
        *last_block = (t == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!*last_block)
    {
        return false;
    }
    __threadfence();                            // the other blocks' partials after the ticket
    return true;
}

// In the last CTA: the partials in a fixed order, whatever CTA this happens to be. Thread 0
// gets the total and the flag, publishes them in ws->sums and re-arms the ticket and the flag
// (graph replays run no memset). tree: shared memory for P1_THREADS doubles.
__device__ __forceinline__ double pass1_final_sum(const P1Partition &part, Workspace *ws, double *tree, int *any_bad)
{
    double mine = 0.0;
    for (int k = threadIdx.x; k < part.vblocks; k += P1_THREADS)
    {
        mine += __ldcg(&ws->partial[k]);
    }
    tree[threadIdx.x] = mine;
    __syncthreads();
    for (int half = P1_THREADS / 2; half > 0; half >>= 1)
    {
        if (threadIdx.x < half)
        {
            tree[threadIdx.x] += tree[threadIdx.x + half];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        *any_bad = __ldcg(&ws->bad);
        ws->sums[0] = tree[0];
        ws->sums[1] = *any_bad ? 1.0 : 0.0;
        ws->bad = 0;
        ws->ticket = 0;
    }
    return tree[0];
}

} // namespace b200amp
