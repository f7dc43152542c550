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
// Ordering between ranks (gradients ready before they are pulled, pair tables complete before
// the finalize, weight arenas complete before the next forward pass) is either the caller's
// (events between the ranks' streams in a one-process host) or the library's own: the ..._sync
// entry points exchange step numbers through a small block of flag words per rank
// (zero1_sync.cuh), every wait bounded, a give-up reported instead of a hang. No multicast
// loads, no TMA from peer memory: every remote access is an ordinary ld/st.global or a
// cudaMemcpyAsync. The reference has no multi-GPU code; the arithmetic per element is that of
// pass 1 / pass 2.

#include <mutex>

#include "adamw_math.cuh"
#include "finalize.cuh"
#include "pass1_common.cuh"
#include "zero1_sync.cuh"

namespace b200amp
{

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
// This launch owns the virtual blocks vb_first .. vb_first + vb_count - 1 of the slice's fixed
// partition (all of them when the slice is reduced in one launch). A launch with last_part == 0
// leaves its partial sums and its flag in the workspace for the launch that ends the slice (same
// stream, so they are complete before that one starts).
// sy: the ranks' flag blocks (off when block[0] is null). SYNC_ENTER_GRADS: every CTA announces
// this rank's gradients and waits for every rank's before it loads anything; a CTA whose wait
// gave up does no work. SYNC_WAIT_PIECE: every CTA waits until piece sy.piece of every peer's pushed
// gradients has landed in this rank's staging rows. SYNC_SIGNAL_PAIRS: the last CTA announces the
// pairs it has written.
template <int R>
__global__ void __launch_bounds__(P1_THREADS)
    rs_pass1_f16_kernel(ConstPtrs src, uint4 *__restrict__ reduced, long long n8, const b200amp_step_state *st,
                        Workspace *ws, Ptrs pair_tables, int my_rank, int vb_first, int vb_count, int last_part,
                        SyncArgs sy)
{
    __shared__ double warp_part[P1_WARPS];
    __shared__ int last_block;

    bool alive = true;
    if (sync_on(sy))
    {
        bool ok = true;
        if (threadIdx.x < R)
        {
            ok = (sy.mode & SYNC_ENTER_GRADS)  ? sync_exchange(sy, SYNC_PHASE_GRADS, threadIdx.x, true, true)
                 : (sy.mode & SYNC_WAIT_PIECE) ? sync_await_piece(sy, threadIdx.x)
                                               : !sync_failed(sy);
        }
        alive = __syncthreads_and(ok) != 0;
    }

    const float inv = 1.0f / st->loss_scale;
    const float inv_ranks = 1.0f / static_cast<float>(R);      // exact: R is a power of two
    const P1Partition part = p1_partition(n8);
    uint32_t bad = 0;

    const int vb_end = alive ? vb_first + vb_count : 0;         // a CTA that gave up walks no blocks
    for (int vb = vb_first + blockIdx.x; vb < vb_end; vb += gridDim.x)
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

    if (!last_part)
    {
        const int block_bad = __syncthreads_or(bad != 0);
        if (threadIdx.x == 0 && block_bad)
        {
            atomicOr(&ws->bad, 1);
        }
        return;
    }
    // the ticket is taken even after a give-up, so the workspace is re-armed for the next launch
    if (!pass1_take_ticket(bad, ws, &last_block))
    {
        return;
    }
    __shared__ double tree[P1_THREADS];
    int any_bad = 0;
    const double total = pass1_final_sum(part, ws, tree, &any_bad);
    if (threadIdx.x == 0)
    {
        if (sync_on(sy) && sync_failed(sy))
        {
            return;                             // some CTA gave up: no pair, no announcement
        }
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
        if (sync_on(sy) && (sy.mode & SYNC_SIGNAL_PAIRS))
        {
            const unsigned int e = sync_epoch(sy);
#pragma unroll
            for (int r = 0; r < R; r++)
            {
                sync_signal(sy, SYNC_PHASE_PAIRS, r, e);
            }
        }
    }
}

// The finalize of the sharded step with its own wait: thread q waits for rank q's "pairs written"
// of the step in flight, then thread 0 adds the pairs in rank order (identical bits on every
// rank) and runs the finalize. When a wait here or earlier in the step gave up, the state is left
// as it is except found_inf = 1, so the pass 2 that follows on the stream changes nothing.
__global__ void finalize_sums_sync_kernel(b200amp_step_state *st, const double *sums, int nranks,
                                          b200amp_schedule cfg, b200amp_step_state *history, int history_len,
                                          SyncArgs sy)
{
    bool ok = true;
    if (static_cast<int>(threadIdx.x) < nranks)
    {
        ok = sync_exchange(sy, SYNC_PHASE_PAIRS, threadIdx.x, false, true);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x != 0)
    {
        return;
    }
    if (!ok)
    {
        st->found_inf = 1;
        return;
    }
    const volatile double *pairs = sums;        // written by the peers: read from memory, not a cache line of before
    double total = 0.0;
    int bad = 0;
    for (int r = 0; r < nranks; r++)
    {
        total += pairs[2 * r];
        bad |= (pairs[2 * r + 1] != 0.0) ? 1 : 0;
    }
    finalize_state(st, total, bad, cfg, history, history_len, true);
}

// One warp. what & 1: announce `phase` of the step in flight to every rank; & 2: wait for it from
// every rank; & 4: the step is over on this rank, advance its counter (only if nothing gave up);
// & 8: write the step in flight into the STAMP word (the source of the copy engines' piece flags).
__global__ void zero1_barrier_kernel(SyncArgs sy, int nranks, int phase, int what)
{
    bool ok = true;
    unsigned int e = 0;
    if (static_cast<int>(threadIdx.x) < nranks)
    {
        e = sync_epoch(sy);
        if (threadIdx.x == 0 && (what & 8))
        {
            sync_local(sy)[SYNC_STAMP] = e;
        }
        ok = (what & 3) ? sync_exchange(sy, phase, threadIdx.x, (what & 1) != 0, (what & 2) != 0) : !sync_failed(sy);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0 && ok && (what & 4))
    {
        sync_local(sy)[SYNC_EPOCH] = e;
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
    const int first = static_cast<int>(blockIdx.x) * THREADS + static_cast<int>(threadIdx.x);
    sweep_groups<1>(master, m, v, g16, tab, nruns, arena_offset, groups, first, stride, wd_decay, f,
                    [&](int j, const uint4 &half8) {
#pragma unroll
                        for (int r = 0; r < R; r++)
                        {
                            store_h8<B200AMP_AG_STORE_HINT>(static_cast<uint4 *>(dst.p[r]) + j, half8);
                        }
                    });
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

// The flag blocks of a b200amp_zero1_sync as kernel arguments. sync == null: off.
static int sync_args(const b200amp_zero1_sync *sync, int nranks, int my_rank, int mode, const char *who,
                     SyncArgs *out, int piece = 0)
{
    SyncArgs a = {};
    a.my_rank = my_rank;
    a.mode = mode;
    a.piece = piece;
    if (sync != nullptr)
    {
        for (int r = 0; r < nranks; r++)
        {
            B200AMP_REQUIRE(sync->block_by_rank[r] != nullptr && aligned(sync->block_by_rank[r], 16),
                            "%s: flag block of rank %d is null or not 16-byte aligned", who, r);
            a.block[r] = static_cast<unsigned int *>(sync->block_by_rank[r]);
        }
        a.limit = sync->wait_limit;
    }
    *out = a;
    return B200AMP_OK;
}

// vblock_count < 0: the whole slice in one launch.
static int rs_pass1_launch(const void *const *grads16_by_rank, int nranks, int my_rank, void *reduced16, long long n,
                           int vblock_first, int vblock_count, int last_part, const b200amp_step_state *st,
                           void *workspace, double *const *pair_table_by_rank, const b200amp_zero1_sync *sync,
                           int sync_mode, b200amp_stream s, int piece = 0)
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
    SyncArgs sy;
    rc = sync_args(sync, nranks, my_rank, sync_mode, "rs_pass1", &sy, piece);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int sms = sm_count();
    if (sms <= 0)
    {
        return B200AMP_ERR_CUDA;
    }
    const long long n8 = n / 8;
    const P1Partition part = p1_partition(n8);
    if (vblock_count < 0)
    {
        vblock_first = 0;
        vblock_count = part.vblocks;
        last_part = 1;
    }
    B200AMP_REQUIRE(vblock_first >= 0 && vblock_count > 0 && vblock_first + vblock_count <= part.vblocks,
                    "rs_pass1: virtual blocks %d .. %d are not inside the slice's %d", vblock_first,
                    vblock_first + vblock_count - 1, part.vblocks);
    int grid = sms * tunables().rs_blocks_per_sm;
    if (grid > vblock_count)
    {
        grid = vblock_count;
    }
    uint4 *out = static_cast<uint4 *>(reduced16);
    Workspace *ws = static_cast<Workspace *>(workspace);
    cudaStream_t stream = as_stream(s);
    const int fin = last_part ? 1 : 0;
#define B200AMP_RS(R)                                                                                            \
    rs_pass1_f16_kernel<R><<<grid, P1_THREADS, 0, stream>>>(src, out, n8, st, ws, tables, my_rank, vblock_first, \
                                                            vblock_count, fin, sy)
    switch (nranks)
    {
    case 1: B200AMP_RS(1); break;
    case 2: B200AMP_RS(2); break;
    case 4: B200AMP_RS(4); break;
    default: B200AMP_RS(8); break;
    }
#undef B200AMP_RS
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_rs_pass1_f16(const void *const *grads16_by_rank, int nranks, int my_rank,
                                                void *reduced16, long long n, const b200amp_step_state *st,
                                                void *workspace, double *const *pair_table_by_rank,
                                                b200amp_stream s)
{
    return rs_pass1_launch(grads16_by_rank, nranks, my_rank, reduced16, n, 0, -1, 1, st, workspace,
                           pair_table_by_rank, nullptr, 0, s);
}

extern "C" B200AMP_API int b200amp_rs_pass1_f16_sync(const void *const *grads16_by_rank, int nranks, int my_rank,
                                                     void *reduced16, long long n, const b200amp_step_state *st,
                                                     void *workspace, double *const *pair_table_by_rank,
                                                     const b200amp_zero1_sync *sync, b200amp_stream s)
{
    B200AMP_REQUIRE(sync != nullptr && pair_table_by_rank != nullptr, "rs_pass1_sync: null sync or pair tables");
    return rs_pass1_launch(grads16_by_rank, nranks, my_rank, reduced16, n, 0, -1, 1, st, workspace,
                           pair_table_by_rank, sync, SYNC_ENTER_GRADS | SYNC_SIGNAL_PAIRS, s);
}

extern "C" B200AMP_API int b200amp_rs_pass1_f16_part(const void *const *grads16_by_rank, int nranks, int my_rank,
                                                     void *reduced16, long long n, int vblock_first,
                                                     int vblock_count, int last_part, const b200amp_step_state *st,
                                                     void *workspace, double *const *pair_table_by_rank,
                                                     b200amp_stream s)
{
    B200AMP_REQUIRE(vblock_count > 0, "rs_pass1 part: vblock_count = %d must be positive", vblock_count);
    return rs_pass1_launch(grads16_by_rank, nranks, my_rank, reduced16, n, vblock_first, vblock_count, last_part, st,
                           workspace, pair_table_by_rank, nullptr, 0, s);
}

extern "C" B200AMP_API int b200amp_pass1_partition(long long n, int *vblocks, long long *elements_per_vblock)
{
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass1_partition: n = %lld must be a positive multiple of 8", n);
    B200AMP_REQUIRE(vblocks != nullptr && elements_per_vblock != nullptr, "pass1_partition: null output pointer");
    const P1Partition part = p1_partition(n / 8);
    *vblocks = part.vblocks;
    *elements_per_vblock = part.vec_per_vblock * 8;
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_copy_async(void *dst, const void *src, long long bytes, b200amp_stream s)
{
    B200AMP_REQUIRE(dst != nullptr && src != nullptr && bytes > 0, "copy_async: null pointer or bytes = %lld", bytes);
    B200AMP_CUDA(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDefault, as_stream(s)));
    return B200AMP_OK;
}

// ---------------------------------------------------------------- the ranks' flag blocks

extern "C" B200AMP_API int b200amp_zero1_sync_init(void *block, b200amp_stream s)
{
    B200AMP_REQUIRE(block != nullptr && aligned(block, 16), "zero1_sync_init: block is null or not 16-byte aligned");
    B200AMP_CUDA(cudaMemsetAsync(block, 0, B200AMP_ZERO1_SYNC_BYTES, as_stream(s)));
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_zero1_sync_read(const void *block, unsigned int *steps_done,
                                                   unsigned int *error)
{
    B200AMP_REQUIRE(block != nullptr, "zero1_sync_read: block is null");
    unsigned int words[2] = {0, 0};
    B200AMP_CUDA(cudaMemcpy(words, static_cast<const unsigned int *>(block) + SYNC_EPOCH, sizeof(words),
                            cudaMemcpyDeviceToHost));
    if (steps_done != nullptr)
    {
        *steps_done = words[0];
    }
    if (error != nullptr)
    {
        *error = words[1];
    }
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_zero1_barrier(const b200amp_zero1_sync *sync, int nranks, int my_rank, int phase,
                                                 int what, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "zero1_barrier");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(sync != nullptr, "zero1_barrier: sync is null");
    B200AMP_REQUIRE(phase >= 0 && phase <= SYNC_PHASE_WEIGHTS, "zero1_barrier: phase = %d, must be 0, 1 or 2", phase);
    B200AMP_REQUIRE(what > 0 && what < 16, "zero1_barrier: what = %d, must be a combination of SIGNAL, WAIT, "
                                           "ADVANCE and STAMP", what);
    SyncArgs sy;
    rc = sync_args(sync, nranks, my_rank, 0, "zero1_barrier", &sy);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    zero1_barrier_kernel<<<1, 32, 0, as_stream(s)>>>(sy, nranks, phase, what);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_finalize_sums_sync(b200amp_step_state *st, const double *sums, int nranks,
                                                      int my_rank, const b200amp_schedule *cfg,
                                                      b200amp_step_state *history, int history_len,
                                                      const b200amp_zero1_sync *sync, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "finalize_sums_sync");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(st != nullptr && sums != nullptr && sync != nullptr && cfg != nullptr,
                    "finalize_sums_sync: null pointer");
    B200AMP_REQUIRE(history == nullptr || history_len > 0, "history given with history_len %d", history_len);
    SyncArgs sy;
    rc = sync_args(sync, nranks, my_rank, 0, "finalize_sums_sync", &sy);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    finalize_sums_sync_kernel<<<1, 32, 0, as_stream(s)>>>(st, sums, nranks, *cfg, history, history_len, sy);
    B200AMP_LAUNCHED();
    return B200AMP_OK;
}

// 1 if a wait on another rank gave up on the current device since the last call (pass2.cu's
// b200amp_device_error reports it together with its own flag).
int b200amp::zero1_sync_timeout_take(int *out)
{
    return sync_timeout_take(out);
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
        per_sm = nranks <= 2 ? 2 : 32;          // measured on four B200s: 2 -> 636, 8 -> 658, 16 -> 672, 32 -> 676 GB/s
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

// ---------------------------------------------------------------- copy-engine forms
//
// The same two steps with the NVLink bytes moved by the copy engines instead of by loads and
// stores that SMs issue. Measured between two B200s with both directions of the links busy: copy
// engines 771-776 GB/s per direction, SM loads 664, SM stores 704. The slice is cut into pieces.
// Reduce-scatter: the peers' pieces are pulled into a local staging buffer on copy streams while
// the kernel, which then reads local memory only, reduces the piece before. All-gather: each
// piece of fp16 weights is pushed to the peers while pass 2 works on the next. Same arithmetic,
// same order of additions, same partition of the norm: bit-identical to the fused kernels.

namespace b200amp
{

constexpr int MAX_LANES = 7;                    // one copy stream per peer at most
constexpr int MAX_PIECES = 64;
constexpr int MAX_DEVICES = 64;

// Per device: the copy streams and a pool of events, created on first use and kept.
struct CopyLanes
{
    bool ready = false;
    cudaStream_t stream[MAX_LANES] = {};
    cudaEvent_t start = nullptr;
    cudaEvent_t done[MAX_LANES] = {};
    cudaEvent_t piece[MAX_PIECES][MAX_LANES] = {};
};

static int copy_lanes(CopyLanes **out)
{
    static CopyLanes lanes[MAX_DEVICES];
    static std::mutex guard;
    std::lock_guard<std::mutex> hold(guard);
    int dev = 0;
    B200AMP_CUDA(cudaGetDevice(&dev));
    B200AMP_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "device index %d out of range", dev);
    CopyLanes &l = lanes[dev];
    if (!l.ready)
    {
        B200AMP_CUDA(cudaEventCreateWithFlags(&l.start, cudaEventDisableTiming));
        for (int k = 0; k < MAX_LANES; k++)
        {
            B200AMP_CUDA(cudaStreamCreateWithFlags(&l.stream[k], cudaStreamNonBlocking));
            B200AMP_CUDA(cudaEventCreateWithFlags(&l.done[k], cudaEventDisableTiming));
            for (int i = 0; i < MAX_PIECES; i++)
            {
                B200AMP_CUDA(cudaEventCreateWithFlags(&l.piece[i][k], cudaEventDisableTiming));
            }
        }
        l.ready = true;
    }
    *out = &l;
    return B200AMP_OK;
}

static int clamp_pieces(int pieces, long long units)
{
    pieces = pieces < 1 ? 1 : pieces;
    pieces = pieces > MAX_PIECES ? MAX_PIECES : pieces;
    return pieces > units ? static_cast<int>(units) : pieces;
}

static int lane_count(int nranks)
{
    int lanes = tunables().ce_lanes;
    lanes = lanes < 1 ? 1 : (lanes > MAX_LANES ? MAX_LANES : lanes);
    return lanes > nranks - 1 ? (nranks > 1 ? nranks - 1 : 1) : lanes;
}

} // namespace b200amp

extern "C" B200AMP_API int b200amp_rs_pass1_f16_ce(const void *const *grads16_by_rank, int nranks, int my_rank,
                                                   void *staging16, void *reduced16, long long n, int pieces,
                                                   const b200amp_step_state *st, void *workspace,
                                                   double *const *pair_table_by_rank,
                                                   const b200amp_zero1_sync *sync, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "rs_pass1_ce");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(grads16_by_rank != nullptr && n > 0 && n % 8 == 0, "rs_pass1_ce: null pointer list or n = %lld "
                                                                       "not a positive multiple of 8", n);
    B200AMP_REQUIRE(nranks == 1 || (staging16 != nullptr && aligned(staging16, 16)),
                    "rs_pass1_ce: the staging buffer ((nranks - 1) * n fp16 values) is null or not 16-byte aligned");
    for (int r = 0; r < nranks; r++)
    {
        B200AMP_REQUIRE(grads16_by_rank[r] != nullptr, "rs_pass1_ce: gradient pointer of rank %d is null", r);
    }
    CopyLanes *lanes = nullptr;
    rc = copy_lanes(&lanes);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int nlanes = lane_count(nranks);
    const P1Partition part = p1_partition(n / 8);
    const long long per = part.vec_per_vblock * 8;             // elements per virtual block
    pieces = clamp_pieces(pieces, part.vblocks);
    cudaStream_t stream = as_stream(s);

    if (sync != nullptr)
    {
        // every rank's gradients are in its arena before the first byte is pulled
        rc = b200amp_zero1_barrier(sync, nranks, my_rank, SYNC_PHASE_GRADS, 3, s);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
    }
    // what the kernel reads: this rank's own arena, and the staging slot of every peer. Peer
    // (my_rank + k) % nranks uses slot k - 1.
    const void *local_src[MAX_RANKS] = {};
    char *staging = static_cast<char *>(staging16);
    for (int k = 0; k < nranks; k++)
    {
        const int r = (my_rank + k) % nranks;
        local_src[r] = k == 0 ? grads16_by_rank[r] : staging + static_cast<size_t>(k - 1) * n * 2;
    }
    // the copies start when everything enqueued on s so far has completed
    B200AMP_CUDA(cudaEventRecord(lanes->start, stream));
    bool forked[MAX_LANES] = {};
    int turn = 0;
    for (int i = 0; i < pieces; i++)
    {
        const int vb0 = static_cast<int>(static_cast<long long>(part.vblocks) * i / pieces);
        const int vb1 = static_cast<int>(static_cast<long long>(part.vblocks) * (i + 1) / pieces);
        const long long e0 = vb0 * per;
        const long long e1 = vb1 * per < n ? vb1 * per : n;
        bool used[MAX_LANES] = {};
        for (int k = 1; k < nranks; k++)
        {
            const int peer = (my_rank + k) % nranks;            // every rank pulls from a different peer at a time
            const int lane = turn++ % nlanes;
            if (!forked[lane])
            {
                B200AMP_CUDA(cudaStreamWaitEvent(lanes->stream[lane], lanes->start, 0));
                forked[lane] = true;
            }
            B200AMP_CUDA(cudaMemcpyAsync(staging + (static_cast<size_t>(k - 1) * n + e0) * 2,
                                         static_cast<const char *>(grads16_by_rank[peer]) + e0 * 2,
                                         static_cast<size_t>(e1 - e0) * 2, cudaMemcpyDefault, lanes->stream[lane]));
            used[lane] = true;
        }
        for (int k = 0; k < nlanes; k++)
        {
            if (used[k])
            {
                B200AMP_CUDA(cudaEventRecord(lanes->piece[i][k], lanes->stream[k]));
                B200AMP_CUDA(cudaStreamWaitEvent(stream, lanes->piece[i][k], 0));
            }
        }
        const bool last = i == pieces - 1;
        rc = rs_pass1_launch(local_src, nranks, my_rank, reduced16, n, vb0, vb1 - vb0, last ? 1 : 0, st, workspace,
                             pair_table_by_rank, sync, last ? SYNC_SIGNAL_PAIRS : 0, s);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
    }
    return B200AMP_OK;
}

// Reduce-scatter by PUSH: writes travel better than reads on links that are busy in both
// directions (a read's request packets share the direction the peer's data uses). Every rank
// copies slice q of its own gradient arena into row my_rank of rank q's staging buffer, piece by
// piece, each piece followed on the same copy stream by a 4-byte copy of this rank's STAMP word
// (the step in flight) into word PIECE[p][my_rank] of rank q's flag block. The owner's reduction of
// piece p (b200amp_rs_pass1_f16_pushed) waits for those words and then reads local memory only.
extern "C" B200AMP_API int b200amp_rs_push_f16_ce(const void *grads16, void *const *staging_by_rank, int nranks,
                                                  int my_rank, long long n, int pieces,
                                                  const b200amp_zero1_sync *sync, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "rs_push_ce");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(grads16 != nullptr && staging_by_rank != nullptr && sync != nullptr, "rs_push_ce: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "rs_push_ce: n = %lld must be a positive multiple of 8", n);
    for (int r = 0; r < nranks; r++)
    {
        B200AMP_REQUIRE(staging_by_rank[r] != nullptr && sync->block_by_rank[r] != nullptr,
                        "rs_push_ce: staging buffer or flag block of rank %d is null", r);
    }
    CopyLanes *lanes = nullptr;
    rc = copy_lanes(&lanes);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int nlanes = lane_count(nranks);
    const P1Partition part = p1_partition(n / 8);
    const long long per = part.vec_per_vblock * 8;
    pieces = clamp_pieces(pieces, part.vblocks);
    pieces = pieces > SYNC_MAX_PIECES ? SYNC_MAX_PIECES : pieces;
    cudaStream_t stream = as_stream(s);
    // the step in flight into the STAMP word, then the copies may start
    rc = b200amp_zero1_barrier(sync, nranks, my_rank, 0, 8, s);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_CUDA(cudaEventRecord(lanes->start, stream));
    const char *mine = static_cast<const char *>(grads16);
    const unsigned int *stamp = static_cast<const unsigned int *>(sync->block_by_rank[my_rank]) + SYNC_STAMP;
    bool forked[MAX_LANES] = {};
    int turn = 0;
    for (int i = 0; i < pieces; i++)
    {
        const int vb0 = static_cast<int>(static_cast<long long>(part.vblocks) * i / pieces);
        const int vb1 = static_cast<int>(static_cast<long long>(part.vblocks) * (i + 1) / pieces);
        const long long e0 = vb0 * per;
        const long long e1 = vb1 * per < n ? vb1 * per : n;
        for (int k = 1; k < nranks; k++)
        {
            const int peer = (my_rank + k) % nranks;            // every rank writes to a different peer at a time
            const int lane = turn++ % nlanes;
            if (!forked[lane])
            {
                B200AMP_CUDA(cudaStreamWaitEvent(lanes->stream[lane], lanes->start, 0));
                forked[lane] = true;
            }
            char *row = static_cast<char *>(staging_by_rank[peer]) + static_cast<size_t>(my_rank) * n * 2;
            B200AMP_CUDA(cudaMemcpyAsync(row + e0 * 2, mine + (static_cast<size_t>(peer) * n + e0) * 2,
                                         static_cast<size_t>(e1 - e0) * 2, cudaMemcpyDefault, lanes->stream[lane]));
            unsigned int *flag = static_cast<unsigned int *>(sync->block_by_rank[peer]) + SYNC_PIECE +
                                 i * MAX_RANKS + my_rank;
            B200AMP_CUDA(cudaMemcpyAsync(flag, stamp, sizeof(unsigned int), cudaMemcpyDefault, lanes->stream[lane]));
        }
    }
    return B200AMP_OK;
}

// The owner's side of the pushed reduce-scatter: pass 1 over R local rows (its own slice of its
// own arena and the R - 1 staging rows the peers filled), in the same pieces, each launch waiting
// (bounded) for its piece of every peer. pieces must be what the peers pushed with. The last
// piece writes the pairs and announces them.
extern "C" B200AMP_API int b200amp_rs_pass1_f16_pushed(const void *own_slice16, const void *staging16, int nranks,
                                                       int my_rank, void *reduced16, long long n, int pieces,
                                                       const b200amp_step_state *st, void *workspace,
                                                       double *const *pair_table_by_rank,
                                                       const b200amp_zero1_sync *sync, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "rs_pass1_pushed");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(own_slice16 != nullptr && staging16 != nullptr && sync != nullptr && n > 0 && n % 8 == 0,
                    "rs_pass1_pushed: null pointer or n = %lld not a positive multiple of 8", n);
    const P1Partition part = p1_partition(n / 8);
    pieces = clamp_pieces(pieces, part.vblocks);
    pieces = pieces > SYNC_MAX_PIECES ? SYNC_MAX_PIECES : pieces;
    const void *src[MAX_RANKS] = {};
    for (int r = 0; r < nranks; r++)
    {
        src[r] = r == my_rank ? own_slice16 : static_cast<const char *>(staging16) + static_cast<size_t>(r) * n * 2;
    }
    for (int i = 0; i < pieces; i++)
    {
        const int vb0 = static_cast<int>(static_cast<long long>(part.vblocks) * i / pieces);
        const int vb1 = static_cast<int>(static_cast<long long>(part.vblocks) * (i + 1) / pieces);
        const bool last = i == pieces - 1;
        rc = rs_pass1_launch(src, nranks, my_rank, reduced16, n, vb0, vb1 - vb0, last ? 1 : 0, st, workspace,
                             pair_table_by_rank, sync, SYNC_WAIT_PIECE | (last ? SYNC_SIGNAL_PAIRS : 0), s, i);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
    }
    return B200AMP_OK;
}

extern "C" B200AMP_API int b200amp_pass2_ag_f16_ce(float *master, float *m, float *v, const void *reduced16,
                                                   void *const *weights16_by_rank, int nranks, int my_rank,
                                                   long long n, long long arena_offset,
                                                   const b200amp_tensor_info *tensors, int ntensors,
                                                   const b200amp_step_state *st, float beta1, float beta2, float eps,
                                                   int pieces, b200amp_stream s)
{
    int rc = check_ranks(nranks, my_rank, "pass2_ag_ce");
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    B200AMP_REQUIRE(master != nullptr && m != nullptr && v != nullptr && reduced16 != nullptr &&
                        weights16_by_rank != nullptr,
                    "pass2_ag_ce: null pointer");
    B200AMP_REQUIRE(n > 0 && n % 8 == 0, "pass2_ag_ce: n = %lld must be a positive multiple of 8", n);
    for (int r = 0; r < nranks; r++)
    {
        B200AMP_REQUIRE(weights16_by_rank[r] != nullptr && aligned(weights16_by_rank[r], 16),
                        "pass2_ag_ce: weight pointer of rank %d is null or not 16-byte aligned", r);
    }
    CopyLanes *lanes = nullptr;
    rc = copy_lanes(&lanes);
    if (rc != B200AMP_OK)
    {
        return rc;
    }
    const int nlanes = lane_count(nranks);
    constexpr long long UNIT = 1024;                            // pieces start at multiples of 1024 elements
    const long long units = (n + UNIT - 1) / UNIT;
    pieces = clamp_pieces(pieces, units);
    cudaStream_t stream = as_stream(s);
    char *mine = static_cast<char *>(weights16_by_rank[my_rank]);
    const char *grads = static_cast<const char *>(reduced16);
    int turn = 0;
    bool used[MAX_LANES] = {};
    for (int i = 0; i < pieces; i++)
    {
        const long long e0 = units * i / pieces * UNIT;
        const long long e1 = i == pieces - 1 ? n : units * (i + 1) / pieces * UNIT;
        rc = b200amp_pass2_f16(master + e0, m + e0, v + e0, grads + e0 * 2, mine + e0 * 2, e1 - e0, arena_offset + e0,
                               tensors, ntensors, st, beta1, beta2, eps, s);
        if (rc != B200AMP_OK)
        {
            return rc;
        }
        if (nranks == 1)
        {
            continue;
        }
        // A skipped step leaves the slice as it was; the copies then rewrite the peers' arenas
        // with the bytes they already hold, which costs link time but keeps the host free of any
        // read of the state.
        B200AMP_CUDA(cudaEventRecord(lanes->piece[i][0], stream));
        for (int k = 1; k < nranks; k++)
        {
            const int peer = (my_rank + k) % nranks;
            const int lane = turn++ % nlanes;
            B200AMP_CUDA(cudaStreamWaitEvent(lanes->stream[lane], lanes->piece[i][0], 0));
            B200AMP_CUDA(cudaMemcpyAsync(static_cast<char *>(weights16_by_rank[peer]) + e0 * 2, mine + e0 * 2,
                                         static_cast<size_t>(e1 - e0) * 2, cudaMemcpyDefault, lanes->stream[lane]));
            used[lane] = true;
        }
    }
    // s continues when every push has landed
    for (int k = 0; k < nlanes; k++)
    {
        if (used[k])
        {
            B200AMP_CUDA(cudaEventRecord(lanes->done[k], lanes->stream[k]));
            B200AMP_CUDA(cudaStreamWaitEvent(stream, lanes->done[k], 0));
        }
    }
    return B200AMP_OK;
}
