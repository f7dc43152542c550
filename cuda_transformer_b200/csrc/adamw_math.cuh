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

// Tensor table in shared memory + the cursor over it. Only a CHANGE of the decay flag matters
// to the update, so neighbours with the same flag are merged while the table is loaded: the GPT
// layout's 12 tensors per layer become 8 runs, and a thread that jumps over several small
// tensors between two trips crosses fewer entries.
struct TensorTable
{
    long long first[B200AMP_MAX_TENSORS];       // first element of each run
    unsigned char decay[B200AMP_MAX_TENSORS];   // its flag
    int warp_heads[32];                         // scratch of table_load
};

// Every thread of the block must call this. Returns the number of runs (>= 1).
__device__ __forceinline__ int table_load(TensorTable &tab, const b200amp_tensor_info *tensors, int ntensors)
{
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    int base = 0;                               // runs found in earlier rounds (same value in every thread)
    for (int k0 = 0; k0 < ntensors; k0 += blockDim.x)
    {
        const int k = k0 + threadIdx.x;
        int flag = 0;
        bool head = false;
        long long offset = 0;
        if (k < ntensors)
        {
            flag = tensors[k].decay ? 1 : 0;
            offset = tensors[k].offset;
            head = k == 0 || ((tensors[k - 1].decay ? 1 : 0) != flag);
        }
        const unsigned heads = __ballot_sync(0xffffffffu, head);
        if (lane == 0)
        {
            tab.warp_heads[warp] = __popc(heads);
        }
        __syncthreads();
        int before = base, total = base;
        for (int w = 0; w < warps; w++)
        {
            const int c = tab.warp_heads[w];
            before += w < warp ? c : 0;
            total += c;
        }
        if (head)
        {
            const int slot = before + __popc(heads & ((1u << lane) - 1u));
            tab.first[slot] = offset;
            tab.decay[slot] = static_cast<unsigned char>(flag);
        }
        base = total;
        __syncthreads();                        // warp_heads is rewritten by the next round; first/decay are read after
    }
    return base;
}

// The same runs as a kernel PARAMETER (1 KB in the constant bank) for tables of at most
// B200AMP_MAX_RUNS runs, built on the host by b200amp_decay_runs_build: no shared memory, no
// loading prologue and no CTA barrier in the kernel that takes it. Offsets are multiples of 4,
// so a run's first element is kept divided by 4 in 32 bits; merged runs alternate, so one flag
// (of run 0) gives them all.
using DecayRuns = b200amp_decay_runs;

// ---- what the cursor needs from a table, for both forms
__device__ __forceinline__ long long table_first(const TensorTable &tab, int k)
{
    return tab.first[k];
}

__device__ __forceinline__ long long table_first(const DecayRuns &tab, int k)
{
    return static_cast<long long>(tab.first4[k]) * 4;
}

// Reads of the shared-memory table go through volatile accesses: they belong to the rare trip
// that crosses a run's end, and must not be hoisted by the compiler into the trip that does not.
__device__ __forceinline__ long long table_next(const TensorTable &tab, int ntensors, int k)
{
    return k + 1 < ntensors ? *static_cast<const volatile long long *>(&tab.first[k + 1]) : LLONG_MAX;
}

__device__ __forceinline__ long long table_next(const DecayRuns &tab, int nruns, int k)
{
    return k + 1 < nruns ? static_cast<long long>(tab.first4[k + 1]) * 4 : LLONG_MAX;
}

__device__ __forceinline__ float table_factor(const TensorTable &tab, int k, float wd_decay)
{
    return *static_cast<const volatile unsigned char *>(&tab.decay[k]) ? wd_decay : 1.0f;
}

__device__ __forceinline__ float table_factor(const DecayRuns &tab, int k, float wd_decay)
{
    return ((tab.flag0 ^ k) & 1) ? wd_decay : 1.0f;
}

struct Cursor
{
    int k;              // the last run whose first element is <= the position (0 if none is)
    long long next;     // first element of run k + 1, LLONG_MAX past the end
    float factor;       // what a parameter of run k is multiplied by: the step's decay, or 1
};

template <class Table>
__device__ __forceinline__ Cursor cursor_seek(const Table &tab, int ntensors, long long at, float wd_decay)
{
    int lo = 0, hi = ntensors - 1;
    while (lo < hi)
    {
        const int mid = (lo + hi + 1) >> 1;
        if (table_first(tab, mid) <= at)
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
    c.factor = table_factor(tab, lo, wd_decay);
    return c;
}

// Positions only grow. Nothing to do (one compare, no table access) while the position stays
// inside run k, which is the case for all but a few hundred trips.
template <class Table>
__device__ __forceinline__ void cursor_advance(Cursor &c, const Table &tab, int ntensors, long long at,
                                               float wd_decay)
{
    if (at >= c.next)
    {
        do
        {
            c.k += 1;
            c.next = table_next(tab, ntensors, c.k);
        } while (at >= c.next);
        c.factor = table_factor(tab, c.k, wd_decay);
    }
}

// Decay factors of the two quads of the 8-element group that starts at `at`. Tensor
// offsets are multiples of 4, so a quad never straddles two tensors but a group can.
// The usual case, the whole group inside the cursor's run, costs one compare.
template <class Table>
__device__ __forceinline__ void group_decay(Cursor &c, const Table &tab, int ntensors, long long at,
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

// ---------------------------------------------------------------- one group of pass 2

struct StepFactors          // the step's scalars, read once per thread
{
    float coef, step_size, bc2_sqrt, inv, w1, w2, b2, eps;
};

__device__ __forceinline__ StepFactors step_factors(const b200amp_step_state *st, float b1, float b2, float eps)
{
    return {st->clip_coef, st->step_size, st->bc2_sqrt, st->inv_scale, 1.0f - b1, 1.0f - b2, b2, eps};
}

// One 8-element group at vector index j of the native step: unscale + clip + AdamW on master, m,
// v in place, then emit(j, the 8 new parameters as fp16) for the caller to store wherever the
// fp16 copy lives (one arena, or every rank's). The four loads are issued first; the decay
// factors of the group's two quads are looked up (decay(d_lo, d_hi)) while they are in flight.
template <int ST, class DecayFn, class EmitFn>
__device__ __forceinline__ void update_group(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                                             const uint4 *__restrict__ g16, int j, DecayFn decay, EmitFn emit,
                                             const StepFactors &f)
{
    const size_t e = static_cast<size_t>(j) * 8;    // first element of the group
    const uint4 gw = load_h8<0>(g16 + j);
    Float8 pp = load8<0>(master + e);
    Float8 mm = load8<0>(m + e);
    Float8 vv = load8<0>(v + e);
    float d_lo, d_hi;
    decay(d_lo, d_hi);
    const uint32_t words[4] = {gw.x, gw.y, gw.z, gw.w};
#pragma unroll
    for (int k = 0; k < 4; k++)
    {
        const float2 h = half2_bits_to_float2(words[k]);
        const float d = k < 2 ? d_lo : d_hi;
        // (g16 * inv) is the unscaled fp32 gradient of the reference, then * clip
        adamw_element(pp.v[2 * k], mm.v[2 * k], vv.v[2 * k], (h.x * f.inv) * f.coef, f.w1, f.w2, f.b2, f.eps, d,
                      f.step_size, f.bc2_sqrt);
        adamw_element(pp.v[2 * k + 1], mm.v[2 * k + 1], vv.v[2 * k + 1], (h.y * f.inv) * f.coef, f.w1, f.w2, f.b2,
                      f.eps, d, f.step_size, f.bc2_sqrt);
    }
    store8<ST>(master + e, pp);
    store8<ST>(m + e, mm);
    store8<ST>(v + e, vv);
    uint4 out;
    out.x = float2_to_half2_bits(pp.v[0], pp.v[1]);
    out.y = float2_to_half2_bits(pp.v[2], pp.v[3]);
    out.z = float2_to_half2_bits(pp.v[4], pp.v[5]);
    out.w = float2_to_half2_bits(pp.v[6], pp.v[7]);
    emit(j, out);
}

// ---------------------------------------------------------------- the sweep of pass 2

// How many trips (groups i, i + stride, i + 2 stride, ...) a thread can take from group i on with
// every group wholly inside the cursor's run and inside the range: 0 when group i itself is not.
__device__ __forceinline__ int trips_inside(const Cursor &c, long long at, int i, int groups, int stride)
{
    if (i >= groups || at + 8 > c.next)
    {
        return 0;
    }
    const int by_end = (groups - 1 - i) / stride + 1;
    const long long room = c.next - 8 - at;             // elements between this group and the last one that fits
    if (room >= (static_cast<long long>(by_end) * stride) * 8)
    {
        return by_end;
    }
    const unsigned int room_groups = static_cast<unsigned int>(room >> 3);  // < by_end * stride < 2^31
    return static_cast<int>(room_groups / static_cast<unsigned int>(stride)) + 1;
}

// One thread's share of the range: groups first, first + stride, ... < groups. The sweep
// alternates between ONE trip that looks its decay factors up (the cursor moves, a group may
// straddle two runs) and a stretch of trips that need no lookup at all: as many as every lane of
// the warp can take inside its current run, agreed on with one warp-wide minimum so that the
// lanes stay in step. The stretch's loop is the plain update with a constant factor. Every lane
// of every warp must call this (lanes with nothing left keep the warp-wide votes company).
template <int ST, class Table, class EmitFn>
__device__ __forceinline__ void sweep_groups(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                                             const uint4 *__restrict__ g16, const Table &tab, int nruns,
                                             long long arena_offset, int groups, int first, int stride,
                                             float wd_decay, const StepFactors &f, EmitFn emit)
{
    constexpr unsigned FULL = 0xffffffffu;
    int i = first;
    Cursor cur = cursor_seek(tab, nruns, arena_offset + static_cast<long long>(i) * 8, wd_decay);
    for (;;)
    {
        const bool active = i < groups;
        if (!__any_sync(FULL, active))
        {
            break;
        }
        if (active)
        {
            const long long at = arena_offset + static_cast<long long>(i) * 8;
            update_group<ST>(
                master, m, v, g16, i,
                [&](float &d_lo, float &d_hi) { group_decay(cur, tab, nruns, at, wd_decay, d_lo, d_hi); }, emit, f);
            i += stride;
        }
        const int mine = trips_inside(cur, arena_offset + static_cast<long long>(i) * 8, i, groups, stride);
        const int fast = __reduce_min_sync(FULL, mine);
        const float factor = cur.factor;
        for (int t = 0; t < fast; t++)
        {
            update_group<ST>(
                master, m, v, g16, i, [&](float &d_lo, float &d_hi) { d_lo = factor; d_hi = factor; }, emit, f);
            i += stride;
        }
    }
}

} // namespace b200amp
