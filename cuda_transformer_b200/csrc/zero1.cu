// zero1.cu: the two passes of the step with the ZeRO-1 collectives folded in, for R GPUs of
// one NVLink/NVSwitch box (one process per GPU, every rank's gradient and weight arenas
// mapped into every process).
//
//   rs_pass1_f16_kernel    reduce-scatter + pass 1 in one kernel: for its own slice of the arena
//                          a rank loads the fp16 gradients of ALL ranks (its own from HBM, the
//                          peers' over NVLink with plain 128-bit loads), adds them in fp32 in
//                          rank order, scales by 1/R, rounds ONCE to fp16, stores the averaged
//                          slice locally, and accumulates the squared norm and the inf/NaN flag
//                          of exactly those stored values. The last CTA writes the rank's
//                          {sum, flag} pair straight into every rank's pair table.
//   pass2_ag_f16_kernel    pass 2 + all-gather in one kernel: the fp16 weights of the slice are
//                          stored into every rank's weight arena (plain 128-bit peer stores)
//                          as they are produced.
//
// Neither kernel waits on another GPU: ordering between ranks (gradients ready before they are
// pulled, pair tables complete before the finalize, weight arenas complete before the next
// forward pass) is the caller's, with stream-ordered barriers between the launches. No
// multicast loads, no TMA from peer memory: every remote access is an ordinary ld/st.global.
// The reference has no multi-GPU code; the arithmetic per element is that of pass 1 / pass 2.

#include "adamw_math.cuh"
#include "pass1_common.cuh"

namespace b200amp
{

constexpr int MAX_RANKS = 8;

struct ConstPtrs
{
    const void *p[MAX_RANKS];
};

struct Ptrs
{
    void *p[MAX_RANKS];
};

// fp32 sum of R fp16 vectors (rank order), times 1/R, rounded to fp16 once.
template <int R>
__device__ __forceinline__ uint4 average_h8(const uint4 (&w)[R], float inv_ranks)
{
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; k++)
    {
        acc[k] = 0.0f;
    }
#pragma unroll
    for (int r = 0; r < R; r++)
    {
        const uint32_t words[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
#pragma unroll
        for (int k = 0; k < 4; k++)
        {
            const float2 f = half2_bits_to_float2(words[k]);
            acc[2 * k] += f.x;
            acc[2 * k + 1] += f.y;
        }
    }
    uint4 out;
    out.x = float2_to_half2_bits(acc[0] * inv_ranks, acc[1] * inv_ranks);
    out.y = float2_to_half2_bits(acc[2] * inv_ranks, acc[3] * inv_ranks);
    out.z = float2_to_half2_bits(acc[4] * inv_ranks, acc[5] * inv_ranks);
    out.w = float2_to_half2_bits(acc[6] * inv_ranks, acc[7] * inv_ranks);
    return out;
}

#ifndef B200AMP_RS_UNROLL
#define B200AMP_RS_UNROLL 2
#endif
#ifndef B200AMP_RS_LOAD_HINT
#define B200AMP_RS_LOAD_HINT 0          // plain ld.global: measured 5 % faster over NVLink than .nc.L1::no_allocate
#endif
#ifndef B200AMP_AG_STORE_HINT
#define B200AMP_AG_STORE_HINT 0
#endif
constexpr int RS_UNROLL = B200AMP_RS_UNROLL;    // vectors per thread per trip: R * RS_UNROLL 16-byte loads in flight

// src.p[r]: the start of THIS rank's slice inside rank r's gradient arena. reduced: local.
// pair_tables.p[r]: rank r's table of R pairs {sum, flag}; this rank fills entry my_rank of each.
template <int R>
__global__ void __launch_bounds__(P1_THREADS)
    rs_pass1_f16_kernel(ConstPtrs src, uint4 *__restrict__ reduced, long long n8, const b200amp_step_state *st,
                        Workspace *ws, Ptrs pair_tables, int my_rank)
{
    __shared__ double warp_part[P1_WARPS];
    __shared__ int last_block;

    const float inv = 1.0f / st->loss_scale;
    const float inv_ranks = 1.0f / static_cast<float>(R);      // exact: R is a power of two
    const P1Partition part = p1_partition(n8);
    uint32_t bad = 0;

    for (int vb = blockIdx.x; vb < part.vblocks; vb += gridDim.x)
    {
        const long long begin = static_cast<long long>(vb) * part.vec_per_vblock;
        long long end = begin + part.vec_per_vblock;
        if (end > n8)
        {
            end = n8;
        }
        // the same slots and accumulators as pass1_f16_kernel (4 per trip of 1024 vectors), so the
        // sum over the averaged slice has the bits pass 1 alone would give on it
        float acc[P1_UNROLL];
#pragma unroll
        for (int u = 0; u < P1_UNROLL; u++)
        {
            acc[u] = 0.0f;
        }
        for (long long base = begin + threadIdx.x; base < end; base += P1_UNROLL * P1_THREADS)
        {
#pragma unroll
            for (int half = 0; half < P1_UNROLL / RS_UNROLL; half++)
            {
                uint4 w[RS_UNROLL][R];
#pragma unroll
                for (int u = 0; u < RS_UNROLL; u++)
                {
                    const long long i = base + (half * RS_UNROLL + u) * P1_THREADS;
                    if (i < end)
                    {
#pragma unroll
                        for (int r = 0; r < R; r++)
                        {
                            w[u][r] = load_h8<B200AMP_RS_LOAD_HINT>(static_cast<const uint4 *>(src.p[r]) + i);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < RS_UNROLL; u++)
                {
                    const long long i = base + (half * RS_UNROLL + u) * P1_THREADS;
                    if (i < end)
                    {
                        const uint4 avg = average_h8<R>(w[u], inv_ranks);
                        store_h8<0>(reduced + i, avg);
                        accumulate_h8(avg, inv, acc[half * RS_UNROLL + u], bad);
                    }
                }
            }
        }
        const float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        vblock_store_partial(mine, warp_part, ws, vb);
    }

    if (!pass1_take_ticket(bad, ws, &last_block))
    {
        return;
    }
    __shared__ double tree[P1_THREADS];
    int any_bad = 0;
    const double total = pass1_final_sum(part, ws, tree, &any_bad);
    if (threadIdx.x == 0)
    {
#pragma unroll
        for (int r = 0; r < R; r++)
        {
            double *table = static_cast<double *>(pair_tables.p[r]);
            if (table != nullptr)
            {
                table[2 * my_rank] = total;
                table[2 * my_rank + 1] = any_bad ? 1.0 : 0.0;
            }
        }
        __threadfence_system();                 // the pairs reach the peers before this grid is seen as done
    }
}

// Pass 2 whose fp16 output goes to R arenas. dst.p[r]: the start of this rank's slice inside
// rank r's weight arena (its own included). Otherwise pass2_f16_kernel with one group per trip.
template <int R>
__global__ void __launch_bounds__(256)
    pass2_ag_f16_kernel(float *__restrict__ master, float *__restrict__ m, float *__restrict__ v,
                        const uint4 *__restrict__ g16, Ptrs dst, long long n8, long long arena_offset,
                        const b200amp_tensor_info *__restrict__ tensors, int ntensors,
                        const b200amp_step_state *__restrict__ st, float b1, float b2, float eps)
{
    constexpr int THREADS = 256;
    __shared__ TensorTable tab;
    const int nruns = table_load(tab, tensors, ntensors);
    if (st->found_inf)
    {
        return;                                 // skipped step: no rank's arena is touched
    }
    const float wd_decay = st->decay;
    const StepFactors f = step_factors(st, b1, b2, eps);

    // 32-bit group indices, as pass2_f16_kernel (the launcher refuses longer ranges)
    const int groups = static_cast<int>(n8);
    const int stride = static_cast<int>(gridDim.x) * THREADS;
    int i = static_cast<int>(blockIdx.x) * THREADS + static_cast<int>(threadIdx.x);
    if (i >= groups)
    {
        return;
    }
    Cursor cur = cursor_seek(tab, nruns, arena_offset + static_cast<long long>(i) * 8, wd_decay);
    for (; i < groups; i += stride)
    {
        const long long at = arena_offset + static_cast<long long>(i) * 8;
        update_group<1>(
            master, m, v, g16, i,
            [&](float &d_lo, float &d_hi) { group_decay(cur, tab, nruns, at, wd_decay, d_lo, d_hi); },
            [&](int j, const uint4 &half8) {
#pragma unroll
                for (int r = 0; r < R; r++)
                {
                    store_h8<B200AMP_AG_STORE_HINT>(static_cast<uint4 *>(dst.p[r]) + j, half8);
                }
            },
            f);
    }
}

static int check_ranks(int nranks, int my_rank, const char *who)
{
    B200AMP_REQUIRE(nranks == 1 || nranks == 2 || nranks == 4 || nranks == 8, "%s: nranks = %d, must be 1, 2, 4 or 8",
                    who, nranks);
    B200AMP_REQUIRE(my_rank >= 0 && my_rank < nranks, "%s: my_rank = %d of %d", who, my_rank, nranks);
    return B200AMP_OK;
}

} // namespace b200amp

using namespace b200amp;

extern "C" B200AMP_API int b200amp_rs_pass1_f16(const void *const *grads16_by_rank, int nranks, int my_rank,
                                                void *reduced16, long long n, const b200amp_step_state *st,
                                                void *workspace, double *const *pair_table_by_rank,
                                                b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "rs_pass1");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(grads16_by_rank != nullptr && reduced16 != nullptr && st != nullptr && workspace != nullptr,
                    "rs_pass1: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "rs_pass1: n = %lld must be a positive multiple of 8", n);
    B200AMP_REQUIRE(aligned(reduced16, 16) && aligned(workspace, 16), "rs_pass1: reduced16 and the workspace must be "
                                                                      "16-byte aligned");
    ConstPtrs src = {};
    Ptrs tables = {};
    for (int r = 0; r < nranks; r++)
    {
        B200AMP_REQUIRE(grads16_by_rank[r] != nullptr && aligned(grads16_by_rank[r], 16),
                        "rs_pass1: gradient pointer of rank %d is null or not 16-byte aligned", r);
        src.p[r] = grads16_by_rank[r];
        tables.p[r] = pair_table_by_rank != nullptr ? pair_table_by_rank[r] : nullptr;
        B200AMP_REQUIRE(aligned(tables.p[r], 8), "rs_pass1: pair table of rank %d is not 8-byte aligned", r);
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const long long n8 = n / 8;
    const P1Partition part = p1_partition(n8);
    int grid = sms * tunables().rs_blocks_per_sm;
    if (grid > part.vblocks)
    {
        grid = part.vblocks;
    }
    uint4 *out = static_cast<uint4 *>(reduced16);
    Workspace *ws = static_cast<Workspace *>(workspace);
    cudaStream_t stream = as_stream(s);
    switch (nranks)
    {
    case 1: rs_pass1_f16_kernel<1><<<grid, P1_THREADS, 0, stream>>>(src, out, n8, st, ws, tables, my_rank); break;
    case 2: rs_pass1_f16_kernel<2><<<grid, P1_THREADS, 0, stream>>>(src, out, n8, st, ws, tables, my_rank); break;
    case 4: rs_pass1_f16_kernel<4><<<grid, P1_THREADS, 0, stream>>>(src, out, n8, st, ws, tables, my_rank); break;
    default: rs_pass1_f16_kernel<8><<<grid, P1_THREADS, 0, stream>>>(src, out, n8, st, ws, tables, my_rank); break;
    }
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_pass2_ag_f16(float *master, float *m, float *v, const void *reduced16,
                                                void *const *weights16_by_rank, int nranks, long long n,
                                                long long arena_offset, const b200amp_tensor_info *tensors,
                                                int ntensors, const b200amp_step_state *st, float beta1, float beta2,
                                                float eps, b200amp_stream s)
{
    int rc = check_ranks(nranks, 0, "pass2_ag");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(master != nullptr && m != nullptr && v != nullptr && reduced16 != nullptr && st != nullptr &&
                        weights16_by_rank != nullptr,
                    "pass2_ag: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass2_ag: n = %lld must be a positive multiple of 8", n);
    if (n / 8 > (1LL << 31) - (1LL << 23))      // 32-bit group indices; the largest grid strides by < 2^23 groups
    {
        set_error("pass2_ag: n = %lld is beyond the 17,112,760,320 elements one launch addresses; split the range", n);
        return B200AMP_ERR_LIMIT;
    }
    B200AMP_REQUIRE(arena_offset >= 0 && arena_offset % 4 == 0, "pass2_ag: arena_offset = %lld must be a multiple "
                                                                 "of 4", arena_offset);
    B200AMP_REQUIRE(aligned(master, 32) && aligned(m, 32) && aligned(v, 32),
                    "pass2_ag: master, m and v must be 32-byte aligned");
    B200AMP_REQUIRE(aligned(reduced16, 16), "pass2_ag: the gradient slice must be 16-byte aligned");
    B200AMP_REQUIRE(tensors != nullptr && ntensors > 0 && ntensors <= B200AMP_MAX_TENSORS,
                    "pass2_ag: tensor table null or ntensors = %d outside 1..%d", ntensors, B200AMP_MAX_TENSORS);
    Ptrs dst = {};
    for (int r = 0; r < nranks; r++)
    {
        B200AMP_REQUIRE(weights16_by_rank[r] != nullptr && aligned(weights16_by_rank[r], 16),
                        "pass2_ag: weight pointer of rank %d is null or not 16-byte aligned", r);
        dst.p[r] = weights16_by_rank[r];
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const long long n8 = n / 8;
    long long want = (n8 + 255) / 256;
    // 0 = choose by what binds the kernel: two ranks leave it HBM-bound (2 CTAs/SM, as pass 2 alone);
    // from four ranks on it is NVLink-bound and more CTAs keep more peer stores in flight
    int per_sm = tunables().ag_blocks_per_sm;
    if (per_sm <= 0)
    {
        per_sm = nranks <= 2 ? 2 : 16;
    }
    int grid = sms * per_sm;
    if (grid > want)
    {
        grid = static_cast<int>(want);
    }
    const uint4 *g16 = static_cast<const uint4 *>(reduced16);
    cudaStream_t stream = as_stream(s);
#define B200AMP_AG(R)                                                                                             \
    pass2_ag_f16_kernel<R><<<grid, 256, 0, stream>>>(master, m, v, g16, dst, n8, arena_offset, tensors, ntensors, \
                                                     st, beta1, beta2, eps)
    switch (nranks)
    {
    case 1: B200AMP_AG(1); break;
    case 2: B200AMP_AG(2); break;
    case 4: B200AMP_AG(4); break;
    default: B200AMP_AG(8); break;
    }
#undef B200AMP_AG
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}
